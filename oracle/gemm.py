"""Block-scaled GEMM y = qx . qw^T on quantized operands, numpy.

TEST INFRASTRUCTURE ONLY: CPU checker for the CUDA GEMM kernels; never imported by the
shipped package.

Restates Nvfp4TiledQuantizeRefOp._ref_qgemm
(miniTransformer/ops/nvfp4_quantize_op_ref.py:449-560): operands are K-major,
qx [M, K], qw [N, K]; per K block (16 for NVFP4, 32 for power-of-two scales)
y += outer(sx[:, k], sw[:, k]) * (Xk @ Wk^T) in fp32; NVFP4 then multiplies by
alpha = amax_x * amax_w / (6*6*448*448). The MXFP8 variant swaps the FP4 lookup for an
E4M3 decode and uses the reference's power-of-two branch (:472-493, alpha = 1).
"""
import numpy as np

from . import formats as F

NVFP4_ALPHA_DENOM = np.float32(6.0 * 6.0 * 448.0 * 448.0)


def nvfp4_alpha(amax_x, amax_w) -> np.float32:
    return np.float32(np.float32(amax_x) * np.float32(amax_w)) / NVFP4_ALPHA_DENOM


def _blockwise(xv, wv, sx, sw, block):
    M, K = xv.shape
    N = wv.shape[0]
    assert K % block == 0 and sx.shape == (M, K // block) and sw.shape == (N, K // block)
    y = np.zeros((M, N), dtype=np.float32)
    for k in range(K // block):
        xs = xv[:, k * block:(k + 1) * block]
        ws = wv[:, k * block:(k + 1) * block]
        y += np.outer(sx[:, k], sw[:, k]).astype(np.float32) * (xs @ ws.T)
    return y


def _fused(xv, wv, sx, sw, block):
    """Same sum with the scales folded into the operands first (code x scale is exact in
    fp32 for both formats), one sgemm instead of K/block; differs from _blockwise only in
    fp32 summation order. Used where the block loop would take minutes."""
    xd = xv * np.repeat(sx, block, axis=1)
    wd = wv * np.repeat(sw, block, axis=1)
    return xd @ wd.T


def _finish(y, out_dtype_round, out, accumulate):
    if accumulate:
        assert out is not None
        y = out.astype(np.float32) + y
    return out_dtype_round(y)


def qgemm_nvfp4(qx, sx_bytes, amax_x, qw, sw_bytes, amax_w, out_bf16=True, out=None,
                accumulate=False, fused=False):
    """qx [M, K/2] u8, sx [>=M, K/16] e4m3 bytes, qw [N, K/2], sw [>=N, K/16] -> [M, N] f32
    (rounded to bf16 when out_bf16)."""
    xv = F.unpack_e2m1(qx)
    wv = F.unpack_e2m1(qw)
    M, N = xv.shape[0], wv.shape[0]
    sx = F.e4m3_decode(sx_bytes[:M])
    sw = F.e4m3_decode(sw_bytes[:N])
    y = (_fused if fused else _blockwise)(xv, wv, sx, sw, 16)
    if xv.shape[1] > 0:
        y = nvfp4_alpha(amax_x, amax_w) * y
    rnd = F.bf16_round if out_bf16 else (lambda a: a.astype(np.float32))
    return _finish(y.astype(np.float32), rnd, out, accumulate)


def qgemm_mxfp8(qx, sx_bytes, qw, sw_bytes, out_bf16=True, out=None, accumulate=False,
                fused=False):
    """qx [M, K] e4m3 bytes, sx [M, K/32] e8m0 bytes, qw [N, K], sw [N, K/32]."""
    xv = F.e4m3_decode(qx)
    wv = F.e4m3_decode(qw)
    sx = F.e8m0_decode(sx_bytes)
    sw = F.e8m0_decode(sw_bytes)
    # a ragged contraction length was quantized with zero padding up to the block: the codes
    # were sliced back, the scales kept the padded block; restore the zero elements
    kpad = sx.shape[1] * 32 - xv.shape[1]
    if kpad > 0:
        xv = np.pad(xv, ((0, 0), (0, kpad)))
        wv = np.pad(wv, ((0, 0), (0, kpad)))
    y = (_fused if fused else _blockwise)(xv, wv, sx, sw, 32)
    rnd = F.bf16_round if out_bf16 else (lambda a: a.astype(np.float32))
    return _finish(y.astype(np.float32), rnd, out, accumulate)


def rel_frobenius(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a - b))
