"""MXFP8 block quantize (E4M3 elements, 1x32 blocks, E8M0 power-of-two scales), numpy.

TEST INFRASTRUCTURE ONLY: CPU checker for the CUDA quantize kernels; never imported by
the shipped package.

PARITY UNPINNED: the reference ships no MXFP8 quantizer (only the enum value
miniTransformer/module/config.py:22). This file assembles one from the pieces the
reference does ship, and nothing else:
  * block amax over the last dim             nvfp4_quantize_op_ref.py:288-292 (block = 32)
  * decode scale = cast_to_e8(amax / fmt_max) nvfp4_quantize_op_ref.py:12-21, 293-298
  * encode scale = 1 / decode                 nvfp4_quantize_op_ref.py:299-302
  * elements = clamp(x * encode, +-448) -> RNE E4M3   nvfp4_quantize_op_ref.py:24-35
  * scale byte = exponent + 127, so that the emulated GEMM decodes 2**(byte-127)
                                              nvfp4_quantize_op_ref.py:474-487
The committed fixtures for it were produced by the same pieces evaluated with PyTorch
(cast_to_e8 called directly), which pins this file to those pieces but not to a
reference MXFP8 implementation, since none exists.
"""
import numpy as np

from . import formats as F

BLOCK = 32


def e8m0_exponent(amax: np.ndarray) -> np.ndarray:
    """ceil(log2(amax/448)) clamped to [-127, 127]; amax = 0 gives -127."""
    with np.errstate(divide="ignore", invalid="ignore"):
        decode = (amax.astype(np.float32) / F.E4M3_MAX).astype(np.float32)
        e = np.ceil(np.log2(decode))
    e = np.clip(e, -127.0, 127.0)
    return e.astype(np.int32)


def quantize_rowwise(x: np.ndarray):
    """x [m, n], n % 32 == 0 -> (E4M3 bytes [m, n], E8M0 bytes [m, n/32])."""
    m, n = x.shape
    assert n % BLOCK == 0
    xb = x.astype(np.float32).reshape(m, n // BLOCK, BLOCK)
    amax = np.abs(xb).max(axis=-1, keepdims=True)
    e = e8m0_exponent(amax)
    with np.errstate(over="ignore", under="ignore", invalid="ignore"):
        decode = np.ldexp(np.float32(1.0), e).astype(np.float32)
        encode = (np.float32(1.0) / decode).astype(np.float32)
        scaled = np.clip((xb * encode).astype(np.float32), -F.E4M3_MAX, F.E4M3_MAX)
    return F.e4m3_encode(scaled).reshape(m, n), (e[:, :, 0] + 127).astype(np.uint8)


def quantize(x: np.ndarray, return_transpose=True):
    """Row-wise copy (blocks along K) and, optionally, the copy of x.T with blocks along M.
    A ragged M is zero-padded to a multiple of 32 for the transposed copy; codes are sliced
    back, scales keep the padded column (same convention as the NVFP4 path,
    miniTransformer/ops/nvfp4_quantize_op_ref.py:391-409)."""
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    q, s = quantize_rowwise(x)
    out = {"data": q, "scale": s, "data_t": None, "scale_t": None}
    if return_transpose:
        xt = np.ascontiguousarray(x.T)
        pad = (-M) % BLOCK
        if pad:
            xt = np.pad(xt, ((0, 0), (0, pad)))
        qt, st = quantize_rowwise(xt)
        out["data_t"] = np.ascontiguousarray(qt[:, :M])
        out["scale_t"] = st
    return out


def dequantize(codes: np.ndarray, scale_bytes: np.ndarray) -> np.ndarray:
    v = F.e4m3_decode(codes)
    s = np.repeat(F.e8m0_decode(scale_bytes), BLOCK, axis=1)[:, : v.shape[1]]
    return v * s
