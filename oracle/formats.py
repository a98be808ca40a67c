"""Number formats used by the block-quantized linear path, restated in numpy.

TEST INFRASTRUCTURE ONLY: this package is the CPU checker for the CUDA kernels.
Nothing in the shipped package imports it.

Every helper works on plain numpy arrays. bf16 tensors are carried as float32
arrays whose values are exactly representable in bf16 (or as raw uint16 bit
patterns where stated).
"""
import numpy as np

FLT_MAX = np.float32(np.finfo(np.float32).max)
E2M1_MAX = np.float32(6.0)
E4M3_MAX = np.float32(448.0)

# Value of each E2M1 nibble; same table as cast_from_fp4x2
# (miniTransformer/ops/nvfp4_quantize_op_ref.py:63-104).
E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32,
)


def _build_e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = s * v
    return t


E4M3_VALUES = _build_e4m3_table()


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bf16 (ties to even); result stays float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    b = x.view(np.uint32).astype(np.uint64)
    lsb = (b >> 16) & 1
    r = ((b + 0x7FFF + lsb) >> 16) << 16
    out = (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32).reshape(x.shape)
    return np.where(np.isnan(x), x, out)


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Bit pattern of bf16_round(x)."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 (fn variant) byte, round to nearest even.

    Follows the `.to(torch.float8_e4m3fn)` cast the reference applies after clamping to
    +-448 (miniTransformer/ops/nvfp4_quantize_op_ref.py:326-327). Values above 448 never
    reach it on the reference path; here they saturate to 0x7E. NaN -> 0x7F.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = (x.view(np.uint32) >> 24).astype(np.uint8) & 0x80
    a = np.abs(x)
    # normal range: keep 3 mantissa bits
    b = a.view(np.uint32).astype(np.uint64)
    lsb = (b >> 20) & 1
    r = (b + 0x7FFFF + lsb) & ~np.uint64(0xFFFFF)
    e = (r >> 23).astype(np.int64) - 127
    m = ((r >> 20) & 7).astype(np.int64)
    normal = ((e + 7) << 3) | m
    # subnormal range: multiples of 2^-9
    with np.errstate(invalid="ignore", over="ignore"):
        sub = np.rint(a * np.float32(512.0))
    sub = np.where(np.isfinite(sub), sub, 0).astype(np.int64)
    code = np.where(a < np.float32(2.0 ** -6), sub, normal)
    code = np.where(a > E4M3_MAX, 0x7E, code)
    code = np.where(np.isnan(x), 0x7F, code)
    return (code.astype(np.uint8) | sign).reshape(x.shape)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return E4M3_VALUES[b.astype(np.int64)]


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E2M1 nibble (one per byte).

    Same interval table as cast_to_fp4x2
    (miniTransformer/ops/nvfp4_quantize_op_ref.py:38-58): nearest, ties to the even code,
    saturating at 6; -0.0 and NaN give code 0; values in [-0.25, -0) give code 8.
    """
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    mag = np.zeros(x.shape, dtype=np.uint8)
    mag[(a > 0.25) & (a < 0.75)] = 1
    mag[(a >= 0.75) & (a <= 1.25)] = 2
    mag[(a > 1.25) & (a < 1.75)] = 3
    mag[(a >= 1.75) & (a <= 2.5)] = 4
    mag[(a > 2.5) & (a < 3.5)] = 5
    mag[(a >= 3.5) & (a <= 5.0)] = 6
    mag[a > 5.0] = 7
    neg = (x < 0.0).astype(np.uint8) * 8  # false for -0.0 and NaN
    return mag | neg


def pack_e2m1(nibbles: np.ndarray) -> np.ndarray:
    """Two nibbles per byte, even column in the low nibble
    (miniTransformer/ops/nvfp4_quantize_op_ref.py:60)."""
    return (nibbles[:, 0::2] | (nibbles[:, 1::2] << 4)).astype(np.uint8)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """Packed bytes [R, C/2] -> float32 values [R, C]."""
    out = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.float32)
    out[:, 0::2] = E2M1_VALUES[packed & 0xF]
    out[:, 1::2] = E2M1_VALUES[packed >> 4]
    return out


def e8m0_decode(b: np.ndarray) -> np.ndarray:
    """2**(byte-127), the decoding used by the emulated GEMM
    (miniTransformer/ops/nvfp4_quantize_op_ref.py:474-487)."""
    return np.ldexp(np.float32(1.0), b.astype(np.int32) - 127).astype(np.float32)
