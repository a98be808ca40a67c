"""Recipes for the quantized linear layers: which quantize backend and block format each of
x, w and dy uses. Same classes and environment variables as the reference
(miniTransformer/module/config.py:15-201); the recipes point at the sm_100a backends.
"""
import dataclasses
import enum
import logging
import os
from typing import Mapping, Optional

import torch

from ..ops import quantization
from ..ops.quantization import MMParams, QParams
from ..ops.mxfp8_quantize_op import Mxfp8QuantizeOp
from ..ops.nvfp4_quantize_op import Nvfp4TiledQuantizeOp

logger = logging.getLogger(__name__)


@enum.unique
class QuantizeType(enum.Enum):
    NONE = "none"
    FP8 = "fp8"
    MXFP8 = "mxfp8"
    INT4 = "int4"
    NVFP4 = "nvfp4"


def should_switch_to_hybrid_linear() -> bool:
    return int(os.getenv("QAT_PARAMS", "0")) > 0


def get_keep_in_bf16_layer_numbers():
    raw = os.getenv("QAT_KEEP_IN_BF16_LAYER_NUMBERS")
    return [] if raw is None else [int(s) for s in raw.split(",")]


@dataclasses.dataclass
class QLinearParams:
    """Quantization settings of one linear layer. `quantize_op` is the backend plug-in slot."""
    quantize: bool = False
    quantize_type: Optional[QuantizeType] = None
    x_params: QParams = QParams()
    w_params: QParams = QParams()
    g_params: QParams = QParams()
    mm_fprop: MMParams = MMParams()
    mm_dgrad: MMParams = MMParams()
    mm_wgrad: MMParams = MMParams()
    # gather quantized activations (codes + scales) instead of bf16 under sequence parallelism
    allgather_quantize: bool = False
    # keep only this rank's shard of the transposed activation copy between forward and backward
    memory_saving: bool = False
    quantize_op: Optional[quantization.QuantizeOpBase] = None
    overrides_for_layer_name: Mapping[str, "QLinearParams"] = dataclasses.field(default_factory=dict)

    def __post_init__(self):
        for v in self.overrides_for_layer_name.values():
            assert not v.overrides_for_layer_name, "only the top-level QLinearParams may carry overrides"

    def customize_for_layer_name(self, layer_name: str) -> "QLinearParams":
        return self.overrides_for_layer_name.get(layer_name, self)


@enum.unique
class QuantizeRecipe(enum.Enum):
    NON_QUANTIZE = "non_quantize"
    INT4_SUB_CHANNEL = "int4_subchannel_scaling"
    FP4_SUB_CHANNEL = "fp4_subchannel_scaling"
    FP4_SUB_CHANNEL_REF = "fp4_subchannel_scaling_ref"
    # additions of this implementation
    MXFP8_SUB_CHANNEL = "mxfp8_subchannel_scaling"
    FP4_SUB_CHANNEL_NO_RHT = "fp4_subchannel_scaling_no_rht"
    FP4_SUB_CHANNEL_SR = "fp4_subchannel_scaling_sr"      # gradients rounded stochastically


def _nvfp4_params(with_rht: bool, allgather_quantize: bool = True, grad_sr: bool = False) -> QLinearParams:
    act = QParams(output_dtype=torch.uint8, scaling_dtype=torch.float8_e4m3fn, quant_tile_shape=(1, 16),
                  with_2d_quantization=False, with_rht=with_rht)
    grad = dataclasses.replace(act, stochastic_rounding=True) if grad_sr else act
    wgt = QParams(output_dtype=torch.uint8, scaling_dtype=torch.float8_e4m3fn, quant_tile_shape=(16, 16),
                  with_2d_quantization=False, with_rht=False)
    return QLinearParams(quantize=True, quantize_type=QuantizeType.NVFP4, x_params=act, w_params=wgt, g_params=grad,
                         quantize_op=Nvfp4TiledQuantizeOp(), allgather_quantize=allgather_quantize)


def _mxfp8_params() -> QLinearParams:
    p = QParams(output_dtype=torch.float8_e4m3fn, scaling_dtype=torch.uint8, quant_tile_shape=(1, 32),
                pow_2_scales=True)
    return QLinearParams(quantize=True, quantize_type=QuantizeType.MXFP8, x_params=p, w_params=p, g_params=p,
                         quantize_op=Mxfp8QuantizeOp(), allgather_quantize=True)


def get_qlinear_params_from_predefined(recipe: QuantizeRecipe) -> QLinearParams:
    if recipe == QuantizeRecipe.NON_QUANTIZE:
        return QLinearParams(quantize=False, quantize_type=QuantizeType.NONE)
    if recipe in (QuantizeRecipe.FP4_SUB_CHANNEL, QuantizeRecipe.FP4_SUB_CHANNEL_REF):
        # x, dy: 1x16 blocks, Hadamard transform on the transposed copies; w: (16,16) tile
        # without 2-D scaling (miniTransformer/module/config.py:118-176). Both reference
        # recipes map to the one native backend; the emulation is not shipped.
        return _nvfp4_params(with_rht=True)
    if recipe == QuantizeRecipe.FP4_SUB_CHANNEL_NO_RHT:
        return _nvfp4_params(with_rht=False)
    if recipe == QuantizeRecipe.FP4_SUB_CHANNEL_SR:
        return _nvfp4_params(with_rht=True, grad_sr=True)
    if recipe == QuantizeRecipe.MXFP8_SUB_CHANNEL:
        return _mxfp8_params()
    raise ValueError(f"Unsupported quantize recipe: {recipe}")


def get_qlinear_params_from_env_qat_params() -> QLinearParams:
    """QAT_PARAMS: 1 = bf16, 3 = NVFP4 (the reference's working indices,
    miniTransformer/module/config.py:181-201); 4 = MXFP8, 5 = NVFP4 without the Hadamard
    transform, 6 = NVFP4 with stochastically rounded gradients (additions). Anything else is an error, as in the reference."""
    raw = os.environ.get("QAT_PARAMS")
    if not raw:
        raise ValueError("QAT_PARAMS is not set; use 1 (bf16), 3 (NVFP4), 4 (MXFP8) or 5 (NVFP4, no RHT)")
    table = {1: QuantizeRecipe.NON_QUANTIZE, 3: QuantizeRecipe.FP4_SUB_CHANNEL, 4: QuantizeRecipe.MXFP8_SUB_CHANNEL,
             5: QuantizeRecipe.FP4_SUB_CHANNEL_NO_RHT, 6: QuantizeRecipe.FP4_SUB_CHANNEL_SR}
    idx = int(raw)
    if idx not in table:
        raise ValueError(f"Unsupported QAT_PARAMS index: {idx}")
    return get_qlinear_params_from_predefined(table[idx])
