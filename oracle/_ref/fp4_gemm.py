"""Stand-in for the reference's CUDA extension: imported at module load, never called on CPU."""
