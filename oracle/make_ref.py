"""Test infrastructure: places the reference's own PyTorch emulation under oracle/_ref/.

    python oracle/make_ref.py /path/to/reference

Copies the reference's Python sources of the quantized-linear path (module/, ops/,
distributed/, utils/: plain .py files, no native code) from a reference checkout into the
git-ignored folder oracle/_ref/miniTransformer/ and writes an empty module named fp4_gemm
beside them (the reference imports its CUDA extension at module load; nothing on the CPU
path calls it). Nothing under oracle/_ref/ is committed, and no product code imports it:
`bench.py --impl reference` and bench.py's `cpu_baseline` leg time it on the host cores, and
the tests use it as a second checker next to the numpy restatement. When oracle/_ref/ is
absent those callers fall back to the numpy restatement and say so.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
SUBDIRS = ("module", "ops", "distributed", "utils")


def make(ref_root: str) -> str:
    src_pkg = os.path.join(ref_root, "miniTransformer")
    if not os.path.isdir(src_pkg):
        raise SystemExit(f"{src_pkg} not found")
    dst_pkg = os.path.join(DEST, "miniTransformer")
    os.makedirs(dst_pkg, exist_ok=True)
    for sub in SUBDIRS:
        os.makedirs(os.path.join(dst_pkg, sub), exist_ok=True)
        for name in sorted(os.listdir(os.path.join(src_pkg, sub))):
            if name.endswith(".py"):
                shutil.copyfile(os.path.join(src_pkg, sub, name), os.path.join(dst_pkg, sub, name))
    with open(os.path.join(DEST, "fp4_gemm.py"), "w") as f:
        f.write('"""Stand-in for the reference\'s CUDA extension: imported at module load, never called on CPU."""\n')
    return DEST


def load():
    """Imports the emulation from oracle/_ref/ and returns a namespace of the pieces the
    callers time or compare against, or None when oracle/_ref/ has not been made."""
    if not os.path.isdir(os.path.join(DEST, "miniTransformer")):
        return None
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    import types
    from miniTransformer.module.config import QuantizeRecipe, get_qlinear_params_from_predefined
    from miniTransformer.module.linear import _QuantizedLinear
    from miniTransformer.ops.nvfp4_quantize_op_ref import Nvfp4TiledQuantizeRefOp
    from miniTransformer.ops.quantization import MMParams, QParams, QuantizeResultCache
    return types.SimpleNamespace(QuantizeRecipe=QuantizeRecipe, get_params=get_qlinear_params_from_predefined,
                                 QuantizedLinear=_QuantizedLinear, RefOp=Nvfp4TiledQuantizeRefOp, QParams=QParams,
                                 MMParams=MMParams, QuantizeResultCache=QuantizeResultCache)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(make(sys.argv[1]))
