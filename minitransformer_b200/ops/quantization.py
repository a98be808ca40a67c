"""Operator interface between the linear modules and a quantize/GEMM implementation.

Mirrors the plugin slot of the reference (miniTransformer/ops/quantization.py:11-182): a
`QuantizeOpBase` instance sits in `QLinearParams.quantize_op`; the autograd functions call
its `quantize` and `qgemm`. Names, fields and argument meaning are kept so that existing
recipes and callers keep working; the implementations behind them are the sm_100a kernels.
"""
import dataclasses
from typing import Optional, Tuple

import torch

from ..utils import utils


@dataclasses.dataclass(frozen=True)
class QParams:
    """How one tensor is quantized.

    scaling_dtype: dtype of the block scales (float8_e4m3fn for NVFP4, uint8 holding E8M0
        bytes for MXFP8). output_dtype: container dtype of the codes. eps: unused lower bound
        on amax. pow_2_scales: block scales are powers of two (MXFP8). quant_tile_shape:
        (rows, cols) of one scale block. with_2d_quantization: one scale per 16x16 block.
        with_rht: 16-point randomized Hadamard transform on the transposed copy.
        stochastic_rounding (an addition; the reference carries the device code compiled out,
        miniTransformer/csrc/util/ptx.cuh:222-260): E2M1 codes are rounded stochastically, for
        gradients.
    """
    scaling_dtype: Optional[torch.dtype] = None
    output_dtype: Optional[torch.dtype] = None
    eps: float = 0.0
    pow_2_scales: bool = False
    quant_tile_shape: Optional[Tuple[int, int]] = None
    with_2d_quantization: bool = False
    with_rht: bool = False
    stochastic_rounding: bool = False


@dataclasses.dataclass(frozen=True)
class MMParams:
    out_dtype: Optional[torch.dtype] = None
    use_split_accumulator: bool = True


@dataclasses.dataclass
class QuantizeResult:
    """Codes and decode scales of a tensor, optionally also of its transpose, plus the
    per-tensor abs-max values NVFP4 needs. `scale_swz` / `scale_t_swz` (an addition of this
    implementation) hold the same scale bytes in the layout the tensor-core GEMM reads."""
    data: torch.Tensor
    scale: torch.Tensor
    data_t: Optional[torch.Tensor] = None
    scale_t: Optional[torch.Tensor] = None
    global_amax_row: Optional[torch.Tensor] = None
    global_amax_col: Optional[torch.Tensor] = None
    scale_swz: Optional[torch.Tensor] = None
    scale_t_swz: Optional[torch.Tensor] = None


@dataclasses.dataclass
class QuantizeResultCache:
    """Quantized weight kept between the microbatches of one step."""
    data: Optional[torch.Tensor] = None
    scale: Optional[torch.Tensor] = None
    data_t: Optional[torch.Tensor] = None
    scale_t: Optional[torch.Tensor] = None
    global_amax_row: Optional[torch.Tensor] = None
    global_amax_col: Optional[torch.Tensor] = None
    scale_swz: Optional[torch.Tensor] = None
    scale_t_swz: Optional[torch.Tensor] = None

    def store(self, r: QuantizeResult) -> None:
        for f in dataclasses.fields(QuantizeResult):
            setattr(self, f.name, getattr(r, f.name))

    def to_qresult(self) -> QuantizeResult:
        assert self.data is not None and self.scale is not None, "weight cache is empty"
        return QuantizeResult(**{f.name: getattr(self, f.name) for f in dataclasses.fields(QuantizeResult)})

    def clear(self) -> None:
        for f in dataclasses.fields(QuantizeResult):
            setattr(self, f.name, None)

    def state(self) -> dict:
        """The cached tensors as plain byte / fp32 tensors for a checkpoint."""
        out = {}
        for f in dataclasses.fields(QuantizeResult):
            t = getattr(self, f.name)
            if t is not None:
                out[f.name] = (t.detach().clone().view(torch.uint8) if t.element_size() == 1 else t.detach().clone(),
                               str(t.dtype))
        return out

    def load_state(self, state: dict) -> None:
        self.clear()
        for name, (t, dtype) in state.items():
            dt = getattr(torch, dtype.split(".")[-1])
            setattr(self, name, t.view(dt) if t.dtype != dt else t)
        # the GEMM-layout scales ride along with the row-major ones
        for lin, swz in (("scale", "scale_swz"), ("scale_t", "scale_t_swz")):
            if getattr(self, lin) is not None and getattr(self, swz) is not None:
                getattr(self, lin)._mt_swz = getattr(self, swz)


@dataclasses.dataclass
class QuantizeInputMetaBase:
    """Side information about a quantize input (e.g. an abs-max computed by the producer)."""
    amax: Optional[torch.Tensor] = None


@dataclasses.dataclass
class QuantizeInputMeta(QuantizeInputMetaBase):
    """What the sm_100a backends take through the `input_meta` hook:
    amax: fp32 device scalar, max |x| of exactly the tensor being quantized, computed by its
        producer (a GEMM with mt_gemm_opts.d_amax, or the reduce step of a fused reduce-scatter);
        the quantizer then skips its own abs-max pass where that is all it needs (NVFP4 without
        the Hadamard transform). amax_col: the abs-max of the transformed transposed copy, when
        the producer knows it too.
    into: byte ranges ("q", "s_swz", "q_t", "s_t_swz") the outputs are written into instead of
        fresh tensors (a rank's slot of a peer all-gather buffer).
    amax_reduce: callable that MAX-reduces the 2-element abs-max buffer across the ranks in
        place, used instead of the process-group all-reduce when reduce_amax is set.
    col_sum: fp32 [features] tensor that receives the column sums of the input from the
        quantizer's abs-max pass (the bias gradient, when the input is dy); the quantizer sets
        col_sum_done when it has filled it (formats without an abs-max pass leave it alone)."""
    amax_col: Optional[torch.Tensor] = None
    into: Optional[dict] = None
    amax_reduce: Optional[object] = None
    col_sum: Optional[torch.Tensor] = None
    col_sum_done: bool = False


class QuantizeOpBase:
    """Interface of a quantize + GEMM backend."""

    def quantize(self, x: torch.Tensor, qparams: QParams, return_transpose: bool = False,
                 reduce_amax: bool = False, tp_group=None,
                 input_meta: Optional[QuantizeInputMetaBase] = None) -> QuantizeResult:
        raise NotImplementedError

    def qgemm(self, qx: torch.Tensor, qw: torch.Tensor, m_params: MMParams, out_dtype: torch.dtype,
              sx: torch.Tensor, sw: torch.Tensor, bias: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, accumulate: bool = False,
              global_amax_qx: Optional[torch.Tensor] = None, global_amax_qw: Optional[torch.Tensor] = None,
              qparams_x: Optional[QParams] = None, qparams_w: Optional[QParams] = None) -> torch.Tensor:
        """y[M,N] = qx[M,K] . qw[N,K]^T (+ bias); with accumulate the result is added into
        `out` in place and `out` is returned."""
        raise NotImplementedError

    @property
    def supports_allgather(self) -> bool:
        """True if a token-sharded input may be quantized per shard and the quantized shards
        all-gathered (bit-identical to quantizing the gathered tensor)."""
        raise NotImplementedError


class QuantizeOpNonQuantize(QuantizeOpBase):
    """Pass-through backend: keeps tensors in high precision and multiplies with torch."""

    @property
    def supports_allgather(self) -> bool:
        return False

    def quantize(self, x, qparams, return_transpose=False, reduce_amax=False, tp_group=None, input_meta=None):
        assert x.dtype in utils.HIGH_PRECISION_FLOAT_DTYPES and not reduce_amax
        qx = x if qparams.output_dtype is None else x.to(qparams.output_dtype)
        empty = torch.empty(0, device=x.device)
        return QuantizeResult(qx, empty, qx.t() if return_transpose else None, empty if return_transpose else None)

    def qgemm(self, qx, qw, m_params, out_dtype, sx, sw, bias=None, out=None, accumulate=False,
              global_amax_qx=None, global_amax_qw=None, qparams_x=None, qparams_w=None):
        y = torch.nn.functional.linear(qx, qw, bias if bias is not None and bias.numel() else None)
        if accumulate:
            assert out is not None
            out.add_(y)
            return out
        return y.to(out_dtype) if y.dtype != out_dtype else y
