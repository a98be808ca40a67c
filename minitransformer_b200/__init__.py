"""B200 (sm_100a) implementation of miniTransformer's quantized-linear hot path.

Public surface (same names as the reference package):
    minitransformer_b200.module.linear.Linear
    minitransformer_b200.module.group_linear.GroupedLinear
    minitransformer_b200.module.config   (QLinearParams, QuantizeRecipe, ...)
    minitransformer_b200.ops.quantization (QuantizeOpBase, QParams, MMParams, ...)
    minitransformer_b200.kernels          (torch front end of the C ABI in include/mt_b200.h)
"""
import importlib
import sys

__version__ = "0.1.0"

_ALIASED = ("module", "module.linear", "module.group_linear", "module.config", "module.base", "module._common",
            "ops", "ops.quantization", "ops.nvfp4_quantize_op", "ops.mxfp8_quantize_op",
            "distributed", "distributed.distributed", "utils", "utils.utils")


def install_as(name: str = "miniTransformer") -> None:
    """Registers this package under another top-level name, so that existing code doing
    `from miniTransformer.module.linear import Linear` (e.g. Megatron's `class TELinear(Linear)`)
    picks up this implementation without edits."""
    pkg = importlib.import_module(__name__)
    sys.modules[name] = pkg
    for sub in _ALIASED:
        sys.modules[f"{name}.{sub}"] = importlib.import_module(f"{__name__}.{sub}")
