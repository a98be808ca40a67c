"""CPU restatement of the reference's quantized-linear path.

TEST INFRASTRUCTURE ONLY. Importers: tests/, the smoke check and the CPU-baseline leg of
the benchmark. The shipped package never imports this and has no CPU fallback.
"""
from . import formats, nvfp4, mxfp8, gemm, linear  # noqa: F401
