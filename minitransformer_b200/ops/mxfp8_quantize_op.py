"""MXFP8 backend on the sm_100a kernels: E4M3 elements, one E8M0 scale byte per 1x32 block.

The reference has no MXFP8 operator (only QuantizeType.MXFP8,
miniTransformer/module/config.py:22); this one follows the pieces it does ship: the E8M0
scale rule cast_to_e8 (ops/nvfp4_quantize_op_ref.py:12-21) and the power-of-two branch of
its emulated GEMM (:472-493). The transposed copy is stored physically transposed
([K, M], blocks along M) so all three GEMMs of a linear layer see K-major operands.
"""
import torch

from .. import kernels
from . import quantization as Q
from .nvfp4_quantize_op import _as_2d_bf16, _swizzled

mxfp8_output_t = torch.float8_e4m3fn
mxfp8_scale_t = torch.uint8  # E8M0 byte = exponent + 127


class Mxfp8QuantizeOp(Q.QuantizeOpBase):
    @property
    def supports_allgather(self) -> bool:
        return True  # no per-tensor scale: shards quantize independently

    def quantize(self, x, qparams, return_transpose=False, reduce_amax=False, tp_group=None, input_meta=None):
        assert qparams.quant_tile_shape in (None, (1, 32)), "MXFP8 uses 1x32 tiles"
        x = _as_2d_bf16(x)
        r = kernels.quantize_mxfp8(x, return_transpose=return_transpose)
        r.scale._mt_swz = r.scale_swz
        data_t = None
        if return_transpose:
            r.scale_t._mt_swz = r.scale_t_swz
            data_t = r.data_t.view(mxfp8_output_t)
        return Q.QuantizeResult(r.data.view(mxfp8_output_t), r.scale, data_t, r.scale_t, None, None,
                                r.scale_swz, r.scale_t_swz)

    def qgemm(self, qx, qw, m_params, out_dtype, sx, sw, bias=None, out=None, accumulate=False,
              global_amax_qx=None, global_amax_qw=None, qparams_x=None, qparams_w=None):
        if out is not None:
            assert out.dtype == out_dtype, "output dtype mismatch"
        M, N = qx.shape[0], qw.shape[0]
        return kernels.gemm_mxfp8(qx.view(torch.uint8), _swizzled(sx, M), qw.view(torch.uint8), _swizzled(sw, N),
                                  out_dtype=out_dtype, out=out, accumulate=accumulate,
                                  bias=bias if bias is not None and bias.numel() else None)
