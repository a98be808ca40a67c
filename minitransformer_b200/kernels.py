"""Thin torch-tensor front end over the C-ABI kernels: allocates outputs with torch, passes
raw pointers and the current CUDA stream, raises on any error. No arithmetic happens here."""
import contextlib
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import MT_BF16, MT_F32, MT_Q_2D, MT_Q_RHT, MT_Q_ROWPAD16  # noqa: F401


# Number of kernels of this library launched through this module since it was last reset
# (the benchmark reports it; memsets are not counted).
LAUNCH_COUNT = 0


def _count(n: int) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += n


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise _lib.MtError(f"{name} must be a CUDA tensor: these kernels have no CPU path")


def swizzled_scale_bytes(rows: int, k_blocks: int) -> int:
    return int(_lib.load().mt_swizzled_scale_bytes(rows, k_blocks))


@dataclass
class Quantized:
    """Outputs of one quantize call. `scale*` are row-major byte tensors (E4M3 or E8M0 bit
    patterns), `scale*_swz` the same values in the layout the GEMM reads."""
    data: torch.Tensor
    scale: torch.Tensor
    scale_swz: torch.Tensor
    data_t: Optional[torch.Tensor] = None
    scale_t: Optional[torch.Tensor] = None
    scale_t_swz: Optional[torch.Tensor] = None
    amax_row: Optional[torch.Tensor] = None
    amax_col: Optional[torch.Tensor] = None


def amax_bf16(x: torch.Tensor, with_rht: bool = False, need_col: bool = True):
    """Per-tensor abs-max (and abs-max of the Hadamard-transformed transpose) as device scalars."""
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    amax = torch.empty(2, dtype=torch.float32, device=x.device)
    flags = MT_Q_RHT if with_rht else 0
    _lib.call("mt_amax_bf16", x.data_ptr(), x.shape[0], x.shape[1], flags, amax[0:1].data_ptr(),
              amax[1:2].data_ptr() if need_col else None, _stream())
    if x.numel():
        _count(1 if with_rht else (2 if need_col else 1))
    return amax[0:1], (amax[1:2] if need_col else amax[0:1])


def quantize_nvfp4(x: torch.Tensor, *, tile=(1, 16), with_2d: bool = False, with_rht: bool = False,
                   return_transpose: bool = True, amax_row: Optional[torch.Tensor] = None,
                   amax_col: Optional[torch.Tensor] = None) -> Quantized:
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    M, K = x.shape
    dev = x.device
    if amax_row is None:
        amax_row, amax_col = amax_bf16(x, with_rht=with_rht and return_transpose, need_col=return_transpose)
    flags = (MT_Q_2D if with_2d else 0) | (MT_Q_RHT if with_rht else 0)
    pad16 = with_2d or tile[0] == 16
    if pad16:
        flags |= MT_Q_ROWPAD16
    rows_s = (M + 15) // 16 * 16 if pad16 else M
    cols_s = (K + 15) // 16 * 16 if pad16 else K
    u8 = torch.uint8
    q = torch.empty((M, K // 2), dtype=u8, device=dev)
    s = torch.empty((rows_s, K // 16), dtype=u8, device=dev)
    s_swz = torch.empty(swizzled_scale_bytes(M, K // 16), dtype=u8, device=dev)
    q_t = s_t = s_t_swz = None
    mb = (M + 15) // 16
    if return_transpose:
        q_t = torch.empty((K, M // 2), dtype=u8, device=dev)
        s_t = torch.empty((cols_s, mb), dtype=u8, device=dev)
        s_t_swz = torch.empty(swizzled_scale_bytes(K, mb), dtype=u8, device=dev)
    _lib.call("mt_quantize_nvfp4", x.data_ptr(), M, K, flags, amax_row.data_ptr(), _ptr(amax_col),
              q.data_ptr(), s.data_ptr(), K // 16, s_swz.data_ptr(),
              _ptr(q_t), _ptr(s_t), mb, _ptr(s_t_swz), _stream())
    _count(1 if x.numel() else 0)
    return Quantized(q, s, s_swz, q_t, s_t, s_t_swz, amax_row, amax_col if return_transpose else amax_row)


def quantize_mxfp8(x: torch.Tensor, *, return_transpose: bool = True) -> Quantized:
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    M, K = x.shape
    dev = x.device
    u8 = torch.uint8
    q = torch.empty((M, K), dtype=u8, device=dev)
    s = torch.empty((M, K // 32), dtype=u8, device=dev)
    s_swz = torch.empty(swizzled_scale_bytes(M, K // 32), dtype=u8, device=dev)
    q_t = s_t = s_t_swz = None
    mb = (M + 31) // 32
    if return_transpose:
        q_t = torch.empty((K, M), dtype=u8, device=dev)
        s_t = torch.empty((K, mb), dtype=u8, device=dev)
        s_t_swz = torch.empty(swizzled_scale_bytes(K, mb), dtype=u8, device=dev)
    _lib.call("mt_quantize_mxfp8", x.data_ptr(), M, K, q.data_ptr(), s.data_ptr(), K // 32, s_swz.data_ptr(),
              _ptr(q_t), _ptr(s_t), mb, _ptr(s_t_swz), _stream())
    _count(1 if x.numel() else 0)
    return Quantized(q, s, s_swz, q_t, s_t, s_t_swz)


def swizzle_scales(s: torch.Tensor, rows: Optional[int] = None) -> torch.Tensor:
    """Row-major scale bytes [R, KB] -> GEMM layout. `rows` limits the rows taken from s."""
    _require_cuda(s, "s")
    s = s.view(torch.uint8) if s.dtype != torch.uint8 else s
    assert s.dim() == 2 and s.stride(1) == 1
    R = s.shape[0] if rows is None else rows
    out = torch.empty(swizzled_scale_bytes(R, s.shape[1]), dtype=torch.uint8, device=s.device)
    _lib.call("mt_swizzle_scales", s.data_ptr(), R, s.shape[1], s.stride(0), out.data_ptr(), _stream())
    _count(1 if R and s.shape[1] else 0)
    return out


def _out_dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return MT_BF16
    if dt == torch.float32:
        return MT_F32
    raise _lib.MtError(f"GEMM output dtype {dt} is not supported (bf16 or fp32)")


def _gemm_out(M, N, out_dtype, out, accumulate, device):
    if out is None:
        if accumulate:
            raise _lib.MtError("accumulate=True needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=device)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
    return out


@contextlib.contextmanager
def sm_margin(sms: int):
    """GEMMs launched inside leave `sms` SMs idle, so that a collective in flight on another
    stream runs beside them instead of behind them."""
    _lib.call("mt_set_sm_margin", int(sms))
    try:
        yield
    finally:
        _lib.call("mt_set_sm_margin", 0)


def _slabs(q):
    """(slab count, rows, bytes per row over all slabs) of a GEMM operand: a 3-D tensor
    [slabs, rows, bytes per slab row] is the contraction dimension split into slabs stored one
    after another (what an all-gather of per-rank transposed shards produces)."""
    if q.dim() == 3:
        assert q.is_contiguous()
        return q.shape[0], q.shape[1], q.shape[0] * q.shape[2]
    return 1, q.shape[0], q.shape[1]


def gemm_nvfp4(qa, sa_swz, amax_a, qb, sb_swz, amax_b, *, out_dtype=torch.bfloat16, out=None,
               accumulate=False, bias=None, check_kernel=False, sa_lin=None, sb_lin=None):
    """D[M,N] = alpha * qa[M,K/2] . qb[N,K/2]^T. With check_kernel=True the CUDA-core
    checker runs instead (it takes the row-major scales sa_lin / sb_lin). A 3-D operand
    [slabs, rows, K/2/slabs] is read slab by slab along K (its scales likewise)."""
    _require_cuda(qa, "qa")
    (a_slabs, M, ka), (b_slabs, N, kb) = _slabs(qa), _slabs(qb)
    if a_slabs > 1 or b_slabs > 1:
        assert ka == kb and not check_kernel
        out = _gemm_out(M, N, out_dtype, out, accumulate, qa.device)
        _count(1)
        _lib.call("mt_gemm_nvfp4_kslab", qa.data_ptr(), sa_swz.data_ptr(), amax_a.data_ptr(), a_slabs, qb.data_ptr(),
                  sb_swz.data_ptr(), amax_b.data_ptr(), b_slabs, M, N, ka * 2, out.data_ptr(),
                  _out_dtype_code(out_dtype), out.stride(0), _ptr(bias),
                  0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate), _stream())
        return out
    M, N, K = qa.shape[0], qb.shape[0], qa.shape[1] * 2
    assert qb.shape[1] * 2 == K
    if K % 32 and not check_kernel:
        # TMA rows must be multiples of 16 bytes: append one block of zero codes (value 0; its
        # scale bytes in the GEMM layout are already zero padding)
        qa = torch.nn.functional.pad(qa, (0, 8))
        qb = torch.nn.functional.pad(qb, (0, 8))
        K += 16
    out = _gemm_out(M, N, out_dtype, out, accumulate, qa.device)
    _count(1 if M and N and K else 0)
    if check_kernel:
        _lib.call("mt_gemm_nvfp4_check", qa.data_ptr(), sa_lin.data_ptr(), sa_lin.stride(0), amax_a.data_ptr(),
                  qb.data_ptr(), sb_lin.data_ptr(), sb_lin.stride(0), amax_b.data_ptr(), M, N, K,
                  out.data_ptr(), _out_dtype_code(out_dtype), out.stride(0), int(accumulate), _stream())
        return out
    _lib.call("mt_gemm_nvfp4", qa.data_ptr(), sa_swz.data_ptr(), amax_a.data_ptr(), qb.data_ptr(),
              sb_swz.data_ptr(), amax_b.data_ptr(), M, N, K, out.data_ptr(), _out_dtype_code(out_dtype),
              out.stride(0), _ptr(bias), 0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate),
              _stream())
    return out


def gemm_mxfp8(qa, sa_swz, qb, sb_swz, *, out_dtype=torch.bfloat16, out=None, accumulate=False, bias=None,
               check_kernel=False, sa_lin=None, sb_lin=None):
    _require_cuda(qa, "qa")
    (a_slabs, M, ka), (b_slabs, N, kb) = _slabs(qa), _slabs(qb)
    if a_slabs > 1 or b_slabs > 1:
        assert ka == kb and not check_kernel
        out = _gemm_out(M, N, out_dtype, out, accumulate, qa.device)
        _count(1)
        _lib.call("mt_gemm_mxfp8_kslab", qa.data_ptr(), sa_swz.data_ptr(), a_slabs, qb.data_ptr(), sb_swz.data_ptr(),
                  b_slabs, M, N, ka, out.data_ptr(), _out_dtype_code(out_dtype), out.stride(0), _ptr(bias),
                  0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate), _stream())
        return out
    M, N, K = qa.shape[0], qb.shape[0], qa.shape[1]
    assert qb.shape[1] == K
    out = _gemm_out(M, N, out_dtype, out, accumulate, qa.device)
    _count(1 if M and N and K else 0)
    if check_kernel:
        _lib.call("mt_gemm_mxfp8_check", qa.data_ptr(), sa_lin.data_ptr(), sa_lin.stride(0), qb.data_ptr(),
                  sb_lin.data_ptr(), sb_lin.stride(0), M, N, K, out.data_ptr(), _out_dtype_code(out_dtype),
                  out.stride(0), int(accumulate), _stream())
        return out
    _lib.call("mt_gemm_mxfp8", qa.data_ptr(), sa_swz.data_ptr(), qb.data_ptr(), sb_swz.data_ptr(), M, N, K,
              out.data_ptr(), _out_dtype_code(out_dtype), out.stride(0), _ptr(bias),
              0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate), _stream())
    return out


# ---- grouped (per-expert) MXFP8 path ----
# The same m_splits list is used by every grouped call of a training step (fc1 / fc2, forward and
# backward): its prefix sums and their ctypes form are kept for the last few distinct lists.
_OFFSETS_CACHE: dict = {}


def _offsets_array(m_splits):
    import ctypes
    key = tuple(m_splits)
    hit = _OFFSETS_CACHE.get(key)
    if hit is None:
        off = [0]
        for m in key:
            off.append(off[-1] + int(m))
        pad = [0]
        for m in key:
            pad.append(pad[-1] + (int(m) + 127) // 128 * 128)
        if len(_OFFSETS_CACHE) >= 8:
            _OFFSETS_CACHE.pop(next(iter(_OFFSETS_CACHE)))
        hit = _OFFSETS_CACHE[key] = ((ctypes.c_int64 * len(off))(*off), off, pad)
    return hit[0], hit[1]


def grouped_padded_offsets(m_splits):
    """Token offsets after padding every group to a multiple of 128 tokens."""
    _offsets_array(m_splits)
    return _OFFSETS_CACHE[tuple(m_splits)][2]


def _grouped_scratch(rows: int, groups: int, device) -> torch.Tensor:
    n = int(_lib.load().mt_grouped_scratch_bytes(rows, groups))
    return torch.empty(max(n, 256), dtype=torch.uint8, device=device)


def grouped_transpose_quantize_mxfp8(x: torch.Tensor, m_splits, want_linear_scales: bool = False):
    """x [R, K] bf16 -> (q_t [K, Rp] u8, s_t_swz, s_t or None, padded offsets)."""
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    R, K = x.shape
    arr, off = _offsets_array(m_splits)
    assert off[-1] == R, "m_splits must sum to the number of rows"
    pad = grouped_padded_offsets(m_splits)
    Rp = pad[-1]
    dev = x.device
    q_t = torch.empty((K, Rp), dtype=torch.uint8, device=dev)
    s_t_swz = torch.empty(swizzled_scale_bytes(K, Rp // 32), dtype=torch.uint8, device=dev)
    s_t = torch.empty((K, Rp // 32), dtype=torch.uint8, device=dev) if want_linear_scales else None
    scratch = _grouped_scratch(R, len(m_splits), dev)
    _lib.call("mt_grouped_transpose_quantize_mxfp8", x.data_ptr(), R, K, arr, len(m_splits), q_t.data_ptr(),
              _ptr(s_t), Rp // 32, s_t_swz.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream())
    _count(1 if Rp else 0)
    return q_t, s_t_swz, s_t, pad


def grouped_quantize_mxfp8(x: torch.Tensor, m_splits):
    """One pass over x [R, K] bf16 -> (Quantized row-wise copy, (q_t [K, Rp], s_t_swz, padded
    offsets)): what quantize_mxfp8(x, return_transpose=False) and
    grouped_transpose_quantize_mxfp8(x, m_splits) return, from a single read of x."""
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    R, K = x.shape
    arr, off = _offsets_array(m_splits)
    assert off[-1] == R, "m_splits must sum to the number of rows"
    pad = grouped_padded_offsets(m_splits)
    Rp = pad[-1]
    dev = x.device
    q = torch.empty((R, K), dtype=torch.uint8, device=dev)
    s = torch.empty((R, K // 32), dtype=torch.uint8, device=dev)
    # rows of the last 128-row chunk beyond R are not written by the kernel: start from zeros
    s_swz = torch.zeros(swizzled_scale_bytes(R, K // 32), dtype=torch.uint8, device=dev)
    q_t = torch.empty((K, Rp), dtype=torch.uint8, device=dev)
    s_t_swz = torch.empty(swizzled_scale_bytes(K, Rp // 32), dtype=torch.uint8, device=dev)
    if R:
        scratch = _grouped_scratch(R, len(m_splits), dev)
        _lib.call("mt_grouped_quantize_mxfp8", x.data_ptr(), R, K, arr, len(m_splits), q.data_ptr(), s.data_ptr(),
                  K // 32, s_swz.data_ptr(), q_t.data_ptr(), None, Rp // 32, s_t_swz.data_ptr(), scratch.data_ptr(),
                  scratch.numel(), _stream())
        _count(1)
    return Quantized(q, s, s_swz), (q_t, s_t_swz, pad)


def grouped_gemm_mxfp8(qa, sa_swz, qb, sb_swz, m_splits, *, n_out: int, transposed_weights: bool,
                       out_dtype=torch.bfloat16):
    """Rows of qa [R, K] are split by m_splits; group g uses its own weight.
    transposed_weights=False: qb = stacked weights [G*n_out, K] (forward).
    transposed_weights=True:  qb = transposed stacked weights [n_out, G*K] (dgrad)."""
    _require_cuda(qa, "qa")
    R, K = qa.shape
    G = len(m_splits)
    arr, off = _offsets_array(m_splits)
    assert off[-1] == R
    if transposed_weights:
        assert qb.shape == (n_out, G * K)
        b_rows, ldb, grp_rows, grp_k = n_out, G * K, 0, K
    else:
        assert qb.shape == (G * n_out, K)
        b_rows, ldb, grp_rows, grp_k = G * n_out, K, n_out, 0
    out = torch.empty((R, n_out), dtype=out_dtype, device=qa.device)
    scratch = _grouped_scratch(R, G, qa.device)
    _lib.call("mt_grouped_gemm_mxfp8", qa.data_ptr(), sa_swz.data_ptr(), qb.data_ptr(), sb_swz.data_ptr(), b_rows, ldb,
              arr, G, n_out, K, grp_rows, grp_k, out.data_ptr(), _out_dtype_code(out_dtype), n_out,
              scratch.data_ptr(), scratch.numel(), _stream())
    _count(1 if R else 0)
    return out


def grouped_wgrad_mxfp8(qa_t, sa_t_swz, qb_t, sb_t_swz, pad_offsets, *, out_dtype=torch.float32, out=None,
                        accumulate=False):
    """Per-group D_g[N, K] = qa_t[N, cols_g] . qb_t[K, cols_g]^T; returns [G, N, K]."""
    import ctypes
    _require_cuda(qa_t, "qa_t")
    G = len(pad_offsets) - 1
    N, K = qa_t.shape[0], qb_t.shape[0]
    assert qa_t.shape[1] == qb_t.shape[1] == pad_offsets[-1]
    if out is None:
        assert not accumulate
        out = torch.empty((G, N, K), dtype=out_dtype, device=qa_t.device)
    else:
        assert out.shape == (G, N, K) and out.dtype == out_dtype and out.is_contiguous()
    arr = (ctypes.c_int64 * (G + 1))(*pad_offsets)
    scratch = _grouped_scratch(pad_offsets[-1], G, qa_t.device)
    _lib.call("mt_grouped_wgrad_mxfp8", qa_t.data_ptr(), sa_t_swz.data_ptr(), qb_t.data_ptr(), sb_t_swz.data_ptr(),
              arr, G, N, K, out.data_ptr(), _out_dtype_code(out_dtype), int(accumulate), scratch.data_ptr(),
              scratch.numel(), _stream())
    _count(1)
    return out


def read_device_status() -> int:
    """Status word raised by bounded device-side waits (0 = clean); clears it."""
    import ctypes
    v = ctypes.c_int(0)
    _lib.check(_lib.load().mt_read_device_status(ctypes.byref(v), _stream()), "mt_read_device_status")
    return v.value
