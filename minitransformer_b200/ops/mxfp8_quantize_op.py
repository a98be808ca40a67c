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
from .nvfp4_quantize_op import _as_2d_bf16, _gemm_dtype, _swizzled

mxfp8_output_t = torch.float8_e4m3fn
mxfp8_scale_t = torch.uint8  # E8M0 byte = exponent + 127


class Mxfp8QuantizeOp(Q.QuantizeOpBase):
    format_name = "mxfp8"

    @property
    def supports_allgather(self) -> bool:
        return True  # no per-tensor scale: shards quantize independently

    def quantize(self, x, qparams, return_transpose=False, reduce_amax=False, tp_group=None, input_meta=None):
        assert qparams.quant_tile_shape in (None, (1, 32)), "MXFP8 uses 1x32 tiles"
        x = _as_2d_bf16(x)
        r = kernels.quantize_mxfp8(x, return_transpose=return_transpose, into=getattr(input_meta, "into", None))
        r.scale._mt_swz = r.scale_swz
        data_t = None
        if return_transpose:
            r.scale_t._mt_swz = r.scale_t_swz
            data_t = r.data_t.view(mxfp8_output_t)
        return Q.QuantizeResult(r.data.view(mxfp8_output_t), r.scale, data_t, r.scale_t, None, None,
                                r.scale_swz, r.scale_t_swz)

    def sm_margin(self, sms: int):
        """Context in which this op's GEMMs leave `sms` SMs idle (for a collective in flight)."""
        return kernels.sm_margin(sms)

    def gemm_options(self, **kw):
        """Context with per-call options of this op's GEMMs (kernels.gemm_options)."""
        return kernels.gemm_options(**kw)

    def qgemm(self, qx, qw, m_params, out_dtype, sx, sw, bias=None, out=None, accumulate=False,
              global_amax_qx=None, global_amax_qw=None, qparams_x=None, qparams_w=None):
        if out is not None:
            assert out.dtype == out_dtype, "output dtype mismatch"
        M, N = qx.shape[-2], qw.shape[-2]   # a 3-D operand is [K slabs, rows, bytes per slab row]
        bias = bias if bias is not None and bias.numel() else None
        kdt = _gemm_dtype(out_dtype)
        if kdt != out_dtype:
            assert out is None, "in-place output needs a bf16 or fp32 tensor"
        if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
            bias = bias.float()
        y = kernels.gemm_mxfp8(qx.view(torch.uint8), _swizzled(sx, M), qw.view(torch.uint8), _swizzled(sw, N),
                               out_dtype=kdt, out=out, accumulate=accumulate, bias=bias)
        return y if kdt == out_dtype or not isinstance(y, torch.Tensor) else y.to(out_dtype)

    # ---- grouped (per-expert) operations used by GroupedLinear ----
    def grouped_quantize(self, w: torch.Tensor, qparams, return_transpose: bool = False) -> Q.QuantizeResult:
        """w [G, N, K] (stacked expert weights) -> row-wise copy [G*N, K] and, optionally, the
        transposed copy [K, G*N] (1x32 blocks along each expert's N, never across experts since
        N is a multiple of 32). One kernel launch for all experts."""
        assert w.dim() == 3 and w.shape[1] % 32 == 0
        G, N, K = w.shape
        return self.quantize(w.reshape(G * N, K), qparams, return_transpose=return_transpose)

    def grouped_qgemm(self, qx, qw, m_params, out_dtype, sx, sw, m_splits=None, biases=None, qparams_x=None,
                      qparams_w=None, weights_transposed: bool = False, n_out=None):
        """Rows of qx are split by m_splits; group g multiplies with expert g.
        weights_transposed=False: qw is the stacked row-wise copy [G*N, K]; y[R, N].
        weights_transposed=True:  qw is the transposed stacked copy [K_in, G*N]; y[R, K_in]."""
        assert biases is None, "biases are added by the module"
        G = len(m_splits)
        if n_out is None:
            n_out = qw.shape[0] if weights_transposed else qw.shape[0] // G
        return kernels.grouped_gemm_mxfp8(qx.view(torch.uint8), _swizzled(sx, qx.shape[0]), qw.view(torch.uint8),
                                          _swizzled(sw, qw.shape[0]), m_splits, n_out=n_out,
                                          transposed_weights=weights_transposed, out_dtype=out_dtype)

    def grouped_transpose_quantize(self, t: torch.Tensor, m_splits, dtype=None):
        """t [R, C] -> (q_t [C, Rp], s_t_swz, padded offsets): t^T with every group zero-padded
        to 128 tokens and 1x32 blocks restarting at each group."""
        q_t, s_t_swz, _, pad = kernels.grouped_transpose_quantize_mxfp8(_as_2d_bf16(t), m_splits)
        return q_t, s_t_swz, pad

    def grouped_quantize_with_transpose(self, t: torch.Tensor, qparams, m_splits):
        """quantize(t) and grouped_transpose_quantize(t, m_splits) from one read of t:
        returns (QuantizeResult of the row-wise copy, (q_t, s_t_swz, padded offsets))."""
        assert qparams.quant_tile_shape in (None, (1, 32)), "MXFP8 uses 1x32 tiles"
        r, t_copy = kernels.grouped_quantize_mxfp8(_as_2d_bf16(t), m_splits)
        r.scale._mt_swz = r.scale_swz
        return Q.QuantizeResult(r.data.view(mxfp8_output_t), r.scale, None, None, None, None, r.scale_swz, None), t_copy

    def grouped_gemm_1d1d(self, a, b, out_dtype=torch.float32, single_output: bool = True, out=None,
                          accumulate: bool = False):
        """a = grouped_transpose_quantize(dy), b = grouped_transpose_quantize(x) ->
        per-expert weight gradients [G, N, K] (or a list of G views)."""
        (qa, sa, pad), (qb, sb, pad_b) = a, b
        assert list(pad) == list(pad_b) and pad.splits == pad_b.splits
        w = kernels.grouped_wgrad_mxfp8(qa, sa, qb, sb, pad, out_dtype=out_dtype, out=out, accumulate=accumulate)
        return w if single_output else list(w.unbind(0))
