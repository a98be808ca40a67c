"""NVFP4 block quantize (E2M1 codes, E4M3 block scales, fp32 per-tensor amax), numpy.

TEST INFRASTRUCTURE ONLY: CPU checker for the CUDA quantize kernels; never imported by
the shipped package.

Restates Nvfp4TiledQuantizeRefOp._quantize and _quantize_blockwise_reference
(miniTransformer/ops/nvfp4_quantize_op_ref.py:258-417). Parity is pinned: the
committed fixtures under tests/golden/ were produced by the reference's own PyTorch
emulation and this file reproduces them bit for bit.
"""
import numpy as np

from . import formats as F

# Fixed sign vector of the randomized Hadamard transform
# (miniTransformer/ops/nvfp4_quantize_op_ref.py:152-157).
RHT_SIGNS = np.array(
    [1, 1, 1, -1, 1, -1, -1, -1, -1, -1, -1, 1, -1, 1, -1, -1], dtype=np.float32
)


def hadamard16() -> np.ndarray:
    """diag(signs) @ Sylvester-Hadamard(16), entries +-1
    (miniTransformer/ops/nvfp4_quantize_op_ref.py:168-191)."""
    h = np.ones((1, 1), dtype=np.float32)
    while h.shape[0] < 16:
        h = np.block([[h, h], [h, -h]])
    return (RHT_SIGNS[:, None] * h).astype(np.float32)


def apply_rht(x: np.ndarray) -> np.ndarray:
    """16-point transform along the last dim, scale 1/4, result rounded to bf16
    (miniTransformer/ops/nvfp4_quantize_op_ref.py:193-218).

    The reference does this as a bf16 matmul; here the 16-term sum is taken in float64
    (exact for bf16 inputs of any realistic exponent spread) and rounded once.
    """
    assert x.shape[-1] % 16 == 0
    h = hadamard16().astype(np.float64) * 0.25
    y = x.reshape(-1, 16).astype(np.float64) @ h
    return F.bf16_round(y.astype(np.float32)).reshape(x.shape)


def _pad(x: np.ndarray, row_div: int, col_div: int) -> np.ndarray:
    m, n = x.shape
    pr = (-m) % row_div
    pc = (-n) % col_div
    if pr == 0 and pc == 0:
        return x
    return np.pad(x, ((0, pr), (0, pc)))


def global_encode_scale(global_amax: np.float32) -> np.float32:
    """448*6/amax clipped to FLT_MAX; 0 (amax = inf) becomes 1
    (miniTransformer/ops/nvfp4_quantize_op_ref.py:304-314)."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        ges = np.minimum(np.float32(F.E4M3_MAX * F.E2M1_MAX) / np.float32(global_amax), F.FLT_MAX)
    if ges == np.float32(0.0):
        ges = np.float32(1.0)
    return np.float32(ges)


def quantize_blockwise(x: np.ndarray, global_amax: np.float32, with_2d: bool):
    """One direction: x [m, n] (already padded; n % 16 == 0, and m % 16 == 0 when with_2d)
    -> (packed codes u8 [m, n/2], scale bytes u8 [m, n/16]).
    miniTransformer/ops/nvfp4_quantize_op_ref.py:258-342 with pow_2_scales=False."""
    m, n = x.shape
    x = x.astype(np.float32)
    if with_2d:
        blk = np.abs(x).reshape(m // 16, 16, n // 16, 16).max(axis=(1, 3))
        vec_max = np.repeat(blk, 16, axis=0)[:, :, None]
    else:
        vec_max = np.abs(x).reshape(m, n // 16, 16).max(axis=-1, keepdims=True)
    xb = x.reshape(m, n // 16, 16)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore", under="ignore"):
        decode = (vec_max / F.E2M1_MAX).astype(np.float32)
        ges = global_encode_scale(global_amax)
        gds = np.float32(1.0) / ges
        decode = np.minimum((decode * ges).astype(np.float32), F.FLT_MAX)
        decode = np.clip(decode, -F.E4M3_MAX, F.E4M3_MAX)
        sbytes = F.e4m3_encode(decode)
        sdec = F.e4m3_decode(sbytes)
        encode = np.minimum(np.float32(1.0) / (sdec * gds).astype(np.float32), F.FLT_MAX)
        scaled = (xb * encode).astype(np.float32)
    clipped = np.clip(scaled, -F.E2M1_MAX, F.E2M1_MAX).reshape(m, n)
    return F.pack_e2m1(F.e2m1_encode(clipped)), sbytes[:, :, 0]


def quantize(x: np.ndarray, tile=(1, 16), with_2d=False, with_rht=False, return_transpose=True):
    """x [M, K] float32 holding bf16 values.

    Returns dict(data [M, K//2], scale [Mp, Kp/16], data_t [K, M//2], scale_t [Kp', Mp'/16],
    amax_row, amax_col) following
    miniTransformer/ops/nvfp4_quantize_op_ref.py:344-417: the transposed copy is a
    row-wise quantization of x.T (after the Hadamard transform when with_rht), padded with
    zeros to the tile, codes sliced back to the unpadded shape, scales kept padded.
    """
    assert tile in ((1, 16), (16, 16))
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    out = {}
    amax_row = np.float32(np.abs(x).max()) if x.size else np.float32(0.0)
    qx, sx = quantize_blockwise(_pad(x, tile[0], tile[1]), amax_row, with_2d)
    out["data"] = np.ascontiguousarray(qx[:M, : K // 2])
    out["scale"] = sx
    out["amax_row"] = amax_row
    if return_transpose:
        xt = np.ascontiguousarray(x.T)
        if with_rht:
            xt = apply_rht(xt)
        amax_col = np.float32(np.abs(xt).max()) if xt.size else np.float32(0.0)
        qt, st = quantize_blockwise(_pad(xt, tile[0], tile[1]), amax_col, with_2d)
        out["data_t"] = np.ascontiguousarray(qt[:K, : M // 2])
        out["scale_t"] = st
        out["amax_col"] = amax_col
    else:
        out["data_t"] = None
        out["scale_t"] = None
        out["amax_col"] = amax_row
    return out


def dequantize(codes: np.ndarray, scale_bytes: np.ndarray, global_amax) -> np.ndarray:
    """codes [R, C/2], scales [R, C/16] -> float32 [R, C] (what the GEMM sees, including
    the per-tensor factor amax/(6*448))."""
    v = F.unpack_e2m1(codes)
    s = np.repeat(F.e4m3_decode(scale_bytes[: v.shape[0]]), 16, axis=1)[:, : v.shape[1]]
    return v * s * (np.float32(global_amax) / np.float32(6.0 * 448.0))
