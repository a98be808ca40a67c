"""NVFP4 backend on the sm_100a kernels.

Takes the place of both reference operators: the native wrapper whose GEMM is a stub
(miniTransformer/ops/nvfp4_quantize_op.py:97-178) and the PyTorch emulation
(miniTransformer/ops/nvfp4_quantize_op_ref.py:160-596), whose numerics the kernels
reproduce (codes, scale bytes and abs-max bit for bit; GEMM within 1e-3 relative
Frobenius error on the same operands). There is no CPU path.
"""
from typing import Optional

import torch

from .. import kernels
from ..distributed.distributed import allreduce_max_
from . import quantization as Q

nvfp4_output_t = torch.uint8
nvfp4_scale_t = torch.float8_e4m3fn


def _as_2d_bf16(x: torch.Tensor) -> torch.Tensor:
    """The kernels read bf16. fp32 / fp16 tensors (the reference module accepts them,
    miniTransformer/module/linear.py:864-870) are rounded to bf16 first, one extra pass; the
    bit-exact contract with the reference emulation holds for bf16 inputs only."""
    if x.dim() > 2:
        x = x.reshape(-1, x.shape[-1])
    if x.dtype in (torch.float32, torch.float16):
        x = x.to(torch.bfloat16)
    elif x.dtype != torch.bfloat16:
        raise kernels._lib.MtError(f"the sm_100a quantize kernels take bf16 / fp16 / fp32 inputs, got {x.dtype}")
    return x.contiguous()


def _gemm_dtype(out_dtype: torch.dtype) -> torch.dtype:
    """Type the GEMM kernel writes for a requested output type: bf16 and fp32 natively, anything
    else (fp16) through fp32 and a cast."""
    return out_dtype if out_dtype in (torch.bfloat16, torch.float32) else torch.float32


def _swizzled(scale: torch.Tensor, rows: int) -> torch.Tensor:
    """GEMM-layout copy of a row-major scale tensor: the one attached by quantize() when the
    same tensor object is passed back, otherwise produced by the swizzle kernel."""
    swz = getattr(scale, "_mt_swz", None)
    if swz is not None:
        return swz
    return kernels.swizzle_scales(scale.view(torch.uint8), rows)


class Nvfp4TiledQuantizeOp(Q.QuantizeOpBase):
    format_name = "nvfp4"
    _sr_calls = 0

    def _next_sr_seed(self) -> int:
        """A fresh seed per stochastic-rounding call, derived from torch's seed so that a run is
        reproducible (a captured graph replays the seed it was captured with)."""
        Nvfp4TiledQuantizeOp._sr_calls += 1
        return (torch.initial_seed() * 0x9E3779B97F4A7C15 + Nvfp4TiledQuantizeOp._sr_calls * 0xD1B54A32D192ED03) & (2 ** 64 - 1)

    @property
    def supports_allgather(self) -> bool:
        # Row-wise 1x16 blocks never cross a token shard, so quantizing shards with the
        # MAX-all-reduced abs-max and gathering codes + scales equals quantizing the gathered
        # tensor.
        return True

    def quantize(self, x, qparams, return_transpose=False, reduce_amax=False, tp_group=None, input_meta=None):
        assert qparams.quant_tile_shape in ((1, 16), (16, 16)), "NVFP4 uses 1x16 or 16x16 tiles"
        assert not qparams.pow_2_scales, "NVFP4 block scales are E4M3, not powers of two"
        x = _as_2d_bf16(x)
        rht = bool(qparams.with_rht) and return_transpose
        known = getattr(input_meta, "amax", None)
        known_col = getattr(input_meta, "amax_col", None)
        if known is not None and (not rht or known_col is not None):
            # the producer already knows max |x|: no abs-max pass over x
            assert known.numel() == 1 and known.dtype == torch.float32
            both = torch.cat([known.reshape(1), (known_col if rht else known).reshape(1)])
            amax_row, amax_col = both[0:1], both[1:2]
        else:
            col_sum = getattr(input_meta, "col_sum", None)
            if col_sum is not None and x.shape[0] % 16 == 0 and x.shape[0] > 0:
                input_meta.col_sum_done = True
            else:
                col_sum = None
            amax_row, amax_col = kernels.amax_bf16(x, with_rht=rht, need_col=return_transpose, col_sum=col_sum)
        if reduce_amax:
            # both scalars live in one 2-element buffer: one tiny exchange
            both = getattr(amax_row, "_mt_pair", None)
            if both is None:
                both = amax_row._base if amax_row._base is not None else amax_row
            reduce = getattr(input_meta, "amax_reduce", None)
            if reduce is not None:
                reduce(both)
            else:
                allreduce_max_(both, tp_group)
        r = kernels.quantize_nvfp4(x, tile=qparams.quant_tile_shape, with_2d=qparams.with_2d_quantization,
                                   with_rht=rht, return_transpose=return_transpose,
                                   amax_row=amax_row, amax_col=amax_col, into=getattr(input_meta, "into", None),
                                   sr_seed=self._next_sr_seed() if getattr(qparams, "stochastic_rounding", False) else None)
        scale = r.scale.view(nvfp4_scale_t)
        scale._mt_swz = r.scale_swz
        scale_t = None
        if return_transpose:
            scale_t = r.scale_t.view(nvfp4_scale_t)
            scale_t._mt_swz = r.scale_t_swz
        return Q.QuantizeResult(r.data, scale, r.data_t, scale_t, r.amax_row, r.amax_col,
                                r.scale_swz, r.scale_t_swz)

    def sm_margin(self, sms: int):
        """Context in which this op's GEMMs leave `sms` SMs idle (for a collective in flight)."""
        return kernels.sm_margin(sms)

    def gemm_options(self, **kw):
        """Context with per-call options of this op's GEMMs (kernels.gemm_options)."""
        return kernels.gemm_options(**kw)

    def qgemm(self, qx, qw, m_params, out_dtype, sx, sw, bias=None, out=None, accumulate=False,
              global_amax_qx=None, global_amax_qw=None, qparams_x=None, qparams_w=None):
        assert global_amax_qx is not None and global_amax_qw is not None, "NVFP4 needs the per-tensor abs-max"
        if out is not None:
            assert out.dtype == out_dtype, "output dtype mismatch"
        M, N = qx.shape[-2], qw.shape[-2]   # a 3-D operand is [K slabs, rows, bytes per slab row]
        bias = bias if bias is not None and bias.numel() else None
        kdt = _gemm_dtype(out_dtype)
        if kdt != out_dtype:
            assert out is None, "in-place output needs a bf16 or fp32 tensor"
        if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
            bias = bias.float()
        y = kernels.gemm_nvfp4(qx, _swizzled(sx, M), global_amax_qx, qw, _swizzled(sw, N), global_amax_qw,
                               out_dtype=kdt, out=out, accumulate=accumulate, bias=bias)
        return y if kdt == out_dtype or not isinstance(y, torch.Tensor) else y.to(out_dtype)
