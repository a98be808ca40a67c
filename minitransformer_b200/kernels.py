"""Thin torch-tensor front end over the C-ABI kernels: allocates outputs with torch, passes
raw pointers and the current CUDA stream, raises on any error. No arithmetic happens here."""
import contextlib
import threading
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import MT_BF16, MT_F32, MT_Q_2D, MT_Q_RHT, MT_Q_ROWPAD16, MT_Q_AMAX_ZEROED  # noqa: F401


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


# Zero-initialised fp32 scalars for abs-max results, handed out from one tensor per (device, stream)
# that a single fill kernel zeroes for 256 calls: with them an abs-max is one kernel launch and no
# memset sits between it and the kernel before it. A slot is never handed out twice; a tensor
# stays alive as long as a result refers to it. Not used while the stream is being captured: a
# replayed graph has to zero its own scalars.
_ZEROED = {}
_ZEROED_LOCK = threading.Lock()      # forward and autograd threads may quantize at the same time


def _zeroed_scalars(device, n: int):
    if torch.cuda.is_current_stream_capturing():
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    with _ZEROED_LOCK:
        pool = _ZEROED.get(key)
        if pool is None or pool[1] + n > pool[0].numel():
            pool = [torch.zeros(512, dtype=torch.float32, device=device), 0]
            _ZEROED[key] = pool
        i = pool[1]
        pool[1] = i + 2          # slots stay 8-byte aligned
    return pool[0][i:i + n]


def amax_bf16(x: torch.Tensor, with_rht: bool = False, need_col: bool = True, col_sum: Optional[torch.Tensor] = None):
    """Per-tensor abs-max (and abs-max of the Hadamard-transformed transpose) as device scalars.
    col_sum (optional fp32 [cols], rows % 16 == 0): also receives the column sums of x from the
    same read."""
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    two = col_sum is not None or (need_col and with_rht)
    flags = MT_Q_RHT if with_rht else 0
    amax = _zeroed_scalars(x.device, 2 if two else 1) if col_sum is None else None
    if amax is not None:
        flags |= MT_Q_AMAX_ZEROED
    else:
        amax = torch.empty(2 if two else 1, dtype=torch.float32, device=x.device)
    if col_sum is not None:
        assert col_sum.dtype == torch.float32 and col_sum.numel() == x.shape[1] and col_sum.is_contiguous()
        _lib.call("mt_amax_colsum_bf16", x.data_ptr(), x.shape[0], x.shape[1], flags, amax[0:1].data_ptr(),
                  amax[1:2].data_ptr() if need_col else None, col_sum.data_ptr(), _stream())
        _count(1 if x.numel() else 0)
    else:
        # without the transform the transposed copy has the same abs-max: one scalar serves both
        col = amax[1:2] if (need_col and with_rht) else amax[0:1]
        _lib.call("mt_amax_bf16", x.data_ptr(), x.shape[0], x.shape[1], flags, amax[0:1].data_ptr(),
                  col.data_ptr() if need_col else None, _stream())
        if x.numel():
            _count(1)
        row = amax[0:1]
        row._mt_pair = amax      # both scalars as one tensor (what a tensor-parallel abs-max exchange reduces)
        return row, col
    row = amax[0:1]
    row._mt_pair = amax
    return row, (amax[1:2] if need_col else row)


def _out_bytes(into, key: str, shape, device) -> torch.Tensor:
    """Output buffer `key`: a view of the caller's byte range when `into` names one (the shared
    buffer of a peer all-gather), else a fresh tensor."""
    n = 1
    for d in shape:
        n *= d
    if into is not None and key in into:
        buf = into[key]
        assert buf.dtype == torch.uint8 and buf.is_contiguous() and buf.numel() >= n and buf.data_ptr() % 16 == 0
        return buf[:n].view(*shape)
    return torch.empty(shape, dtype=torch.uint8, device=device)


def quantized_shard_bytes(fmt: str, rows: int, cols: int):
    """Byte sizes of (codes, GEMM-layout scales, transposed codes, transposed GEMM-layout scales) of
    a [rows, cols] tensor in format "nvfp4" or "mxfp8"."""
    if fmt == "nvfp4":
        return (rows * cols // 2, swizzled_scale_bytes(rows, cols // 16), cols * (rows // 2),
                swizzled_scale_bytes(cols, (rows + 15) // 16))
    return (rows * cols, swizzled_scale_bytes(rows, cols // 32), cols * rows, swizzled_scale_bytes(cols, (rows + 31) // 32))


def quantize_nvfp4(x: torch.Tensor, *, tile=(1, 16), with_2d: bool = False, with_rht: bool = False,
                   return_transpose: bool = True, amax_row: Optional[torch.Tensor] = None,
                   amax_col: Optional[torch.Tensor] = None, into=None, sr_seed: Optional[int] = None) -> Quantized:
    """`into` (optional): dict of uint8 byte ranges for "q", "s_swz", "q_t", "s_t_swz" that the
    kernel writes instead of fresh tensors. sr_seed: round the codes stochastically with this seed."""
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
    q = _out_bytes(into, "q", (M, K // 2), dev)
    s = torch.empty((rows_s, K // 16), dtype=u8, device=dev)
    s_swz = _out_bytes(into, "s_swz", (swizzled_scale_bytes(M, K // 16),), dev)
    q_t = s_t = s_t_swz = None
    mb = (M + 15) // 16
    if return_transpose:
        q_t = _out_bytes(into, "q_t", (K, M // 2), dev)
        s_t = torch.empty((cols_s, mb), dtype=u8, device=dev)
        s_t_swz = _out_bytes(into, "s_t_swz", (swizzled_scale_bytes(K, mb),), dev)
    if sr_seed is None:
        _lib.call("mt_quantize_nvfp4", x.data_ptr(), M, K, flags, amax_row.data_ptr(), _ptr(amax_col),
                  q.data_ptr(), s.data_ptr(), K // 16, s_swz.data_ptr(),
                  _ptr(q_t), _ptr(s_t), mb, _ptr(s_t_swz), _stream())
    else:
        _lib.call("mt_quantize_nvfp4_sr", x.data_ptr(), M, K, flags, amax_row.data_ptr(), _ptr(amax_col),
                  q.data_ptr(), s.data_ptr(), K // 16, s_swz.data_ptr(),
                  _ptr(q_t), _ptr(s_t), mb, _ptr(s_t_swz), int(sr_seed) & 0xFFFFFFFFFFFFFFFF, _stream())
    _count(1 if x.numel() else 0)
    return Quantized(q, s, s_swz, q_t, s_t, s_t_swz, amax_row, amax_col if return_transpose else amax_row)


def quantize_mxfp8(x: torch.Tensor, *, return_transpose: bool = True, into=None) -> Quantized:
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    M, K = x.shape
    dev = x.device
    u8 = torch.uint8
    q = _out_bytes(into, "q", (M, K), dev)
    s = torch.empty((M, K // 32), dtype=u8, device=dev)
    s_swz = _out_bytes(into, "s_swz", (swizzled_scale_bytes(M, K // 32),), dev)
    q_t = s_t = s_t_swz = None
    mb = (M + 31) // 32
    if return_transpose:
        q_t = _out_bytes(into, "q_t", (K, M), dev)
        s_t = torch.empty((K, mb), dtype=u8, device=dev)
        s_t_swz = _out_bytes(into, "s_t_swz", (swizzled_scale_bytes(K, mb),), dev)
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


class _NoOutput:
    """Stand-in output of a scattering GEMM (its rows go to the ranks' staging buffers)."""
    @staticmethod
    def data_ptr():
        return None

    @staticmethod
    def stride(_):
        return 0


def _gemm_out(M, N, out_dtype, out, accumulate, device):
    if _scattering():
        assert out is None and not accumulate and out_dtype == torch.bfloat16
        return _NoOutput()
    if out is None:
        if accumulate:
            raise _lib.MtError("accumulate=True needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=device)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
    return out


_GEMM_OPTS = threading.local()


@contextlib.contextmanager
def gemm_options(sm_margin: Optional[int] = None, d_amax: Optional[torch.Tensor] = None, scatter=None):
    """Per-call options of the GEMMs launched inside by this thread (mt_gemm_opts):
    sm_margin: SMs each launch leaves idle, so that a collective in flight on another stream
    runs beside it instead of behind it; d_amax: fp32 device scalar (zeroed by the caller) that
    the GEMM raises to the largest |value| it stores; scatter = (addresses of the ranks' staging
    buffers, this rank, rows per rank): the output rows go to the ranks' staging buffers instead
    of an output tensor (the GEMM call then returns None)."""
    prev = getattr(_GEMM_OPTS, "value", None)
    base = prev or (0, None, None)     # nested contexts inherit what they do not set
    _GEMM_OPTS.value = (base[0] if sm_margin is None else int(sm_margin), base[1] if d_amax is None else d_amax,
                        base[2] if scatter is None else scatter)
    try:
        yield
    finally:
        _GEMM_OPTS.value = prev


def sm_margin(sms: int):
    return gemm_options(sm_margin=sms)


def _opts():
    cur = getattr(_GEMM_OPTS, "value", None)
    if cur is None or (cur[0] == 0 and cur[1] is None and cur[2] is None):
        return None
    margin, amax, scatter = cur
    if amax is not None:
        assert amax.dtype == torch.float32 and amax.is_cuda and amax.numel() == 1
    o = _lib.GemmOpts(margin, None if amax is None else amax.data_ptr())
    if scatter is not None:
        ptrs, me, rows = scatter
        o.n_dest, o.my_rank, o.dest_rows = len(ptrs), int(me), int(rows)
        for i, p_ in enumerate(ptrs):
            o.dest[i] = p_
    return _lib.ctypes.byref(o)


def _scattering() -> bool:
    cur = getattr(_GEMM_OPTS, "value", None)
    return cur is not None and cur[2] is not None


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
                  0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate), _opts(), _stream())
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
              _opts(), _stream())
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
                  0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate), _opts(), _stream())
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
              0 if bias is None else _out_dtype_code(bias.dtype), int(accumulate), _opts(), _stream())
    return out


# ---- grouped (per-expert) MXFP8 path ----
class PadOffsets(list):
    """Padded token offsets of the groups (a plain list) that also remember the split sizes
    they were derived from, so that a later grouped call finds the same plan."""
    splits: tuple = ()


class GroupedPlan:
    """Device-side description of one m_splits list, shared by every grouped call that uses the
    list (fc1 / fc2, forward and backward): the plan buffer mt_grouped_plan_build fills, plus
    the host-side numbers needed to size outputs (row total, padded offsets)."""

    def __init__(self, m_splits, device):
        self.splits = tuple(int(m) for m in m_splits)
        self.groups = len(self.splits)
        off, pad = [0], [0]
        for m in self.splits:
            assert m >= 0, "negative group size"
            off.append(off[-1] + m)
            pad.append(pad[-1] + (m + 127) // 128 * 128)
        self.offsets, self.pad_offsets = off, PadOffsets(pad)
        self.pad_offsets.splits = self.splits
        self.rows, self.padded_rows = off[-1], pad[-1]
        # the offsets reach the device by one small asynchronous copy from pinned memory; the
        # tile tables are derived there
        host = torch.tensor(off, dtype=torch.int64).pin_memory()
        self._host = host                      # kept until the copy has certainly been issued and consumed
        self.offsets_dev = host.to(device, non_blocking=True)
        n = int(_lib.load().mt_grouped_plan_bytes(self.rows, self.groups))
        assert n > 0, "group description out of range"
        self.buffer = torch.empty(n, dtype=torch.uint8, device=device)
        _lib.call("mt_grouped_plan_build", self.offsets_dev.data_ptr(), self.groups, self.rows, self.buffer.data_ptr(),
                  n, _stream())
        _count(1)

    def ptr(self):
        return self.buffer.data_ptr()


# The same m_splits list is used by every grouped call of a training step: plans are kept for the
# last few distinct lists per device (and stream, since the plan is built on the current stream).
_PLAN_CACHE: dict = {}


def grouped_plan(m_splits, device) -> GroupedPlan:
    if isinstance(m_splits, GroupedPlan):
        return m_splits
    device = torch.device(device)
    key = (tuple(int(m) for m in m_splits), device.index, _stream())
    hit = _PLAN_CACHE.get(key)
    if hit is None:
        if len(_PLAN_CACHE) >= 8:
            _PLAN_CACHE.pop(next(iter(_PLAN_CACHE)))
        hit = _PLAN_CACHE[key] = GroupedPlan(key[0], device)
    return hit


def grouped_padded_offsets(m_splits):
    """Token offsets after padding every group to a multiple of 128 tokens."""
    pad = [0]
    for m in m_splits:
        pad.append(pad[-1] + (int(m) + 127) // 128 * 128)
    return pad


def grouped_transpose_quantize_mxfp8(x: torch.Tensor, m_splits, want_linear_scales: bool = False):
    """x [R, K] bf16 -> (q_t [K, Rp] u8, s_t_swz, s_t or None, padded offsets)."""
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    R, K = x.shape
    plan = grouped_plan(m_splits, x.device)
    assert plan.rows == R, "m_splits must sum to the number of rows"
    Rp = plan.padded_rows
    dev = x.device
    q_t = torch.empty((K, Rp), dtype=torch.uint8, device=dev)
    s_t_swz = torch.empty(swizzled_scale_bytes(K, Rp // 32), dtype=torch.uint8, device=dev)
    s_t = torch.empty((K, Rp // 32), dtype=torch.uint8, device=dev) if want_linear_scales else None
    _lib.call("mt_grouped_transpose_quantize_mxfp8", x.data_ptr(), R, K, plan.ptr(), plan.groups, Rp, q_t.data_ptr(),
              _ptr(s_t), Rp // 32, s_t_swz.data_ptr(), _stream())
    _count(1 if Rp else 0)
    return q_t, s_t_swz, s_t, plan.pad_offsets


def grouped_quantize_mxfp8(x: torch.Tensor, m_splits):
    """One pass over x [R, K] bf16 -> (Quantized row-wise copy, (q_t [K, Rp], s_t_swz, padded
    offsets)): what quantize_mxfp8(x, return_transpose=False) and
    grouped_transpose_quantize_mxfp8(x, m_splits) return, from a single read of x."""
    _require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    R, K = x.shape
    plan = grouped_plan(m_splits, x.device)
    assert plan.rows == R, "m_splits must sum to the number of rows"
    Rp = plan.padded_rows
    dev = x.device
    q = torch.empty((R, K), dtype=torch.uint8, device=dev)
    s = torch.empty((R, K // 32), dtype=torch.uint8, device=dev)
    # rows of the last 128-row chunk beyond R are not written by the kernel: start from zeros
    s_swz = torch.zeros(swizzled_scale_bytes(R, K // 32), dtype=torch.uint8, device=dev)
    q_t = torch.empty((K, Rp), dtype=torch.uint8, device=dev)
    s_t_swz = torch.empty(swizzled_scale_bytes(K, Rp // 32), dtype=torch.uint8, device=dev)
    if R:
        _lib.call("mt_grouped_quantize_mxfp8", x.data_ptr(), R, K, plan.ptr(), plan.groups, Rp, q.data_ptr(),
                  s.data_ptr(), K // 32, s_swz.data_ptr(), q_t.data_ptr(), None, Rp // 32, s_t_swz.data_ptr(), _stream())
        _count(1)
    return Quantized(q, s, s_swz), (q_t, s_t_swz, plan.pad_offsets)


def grouped_gemm_mxfp8(qa, sa_swz, qb, sb_swz, m_splits, *, n_out: int, transposed_weights: bool,
                       out_dtype=torch.bfloat16):
    """Rows of qa [R, K] are split by m_splits; group g uses its own weight.
    transposed_weights=False: qb = stacked weights [G*n_out, K] (forward).
    transposed_weights=True:  qb = transposed stacked weights [n_out, G*K] (dgrad)."""
    _require_cuda(qa, "qa")
    R, K = qa.shape
    plan = grouped_plan(m_splits, qa.device)
    G = plan.groups
    assert plan.rows == R
    if transposed_weights:
        assert qb.shape == (n_out, G * K)
        b_rows, ldb, grp_rows, grp_k = n_out, G * K, 0, K
    else:
        assert qb.shape == (G * n_out, K)
        b_rows, ldb, grp_rows, grp_k = G * n_out, K, n_out, 0
    out = torch.empty((R, n_out), dtype=out_dtype, device=qa.device)
    _lib.call("mt_grouped_gemm_mxfp8", qa.data_ptr(), sa_swz.data_ptr(), qb.data_ptr(), sb_swz.data_ptr(), b_rows, ldb,
              plan.ptr(), G, R, n_out, K, grp_rows, grp_k, out.data_ptr(), _out_dtype_code(out_dtype), n_out, _stream())
    _count(1 if R else 0)
    return out


def grouped_wgrad_mxfp8(qa_t, sa_t_swz, qb_t, sb_t_swz, m_splits, *, out_dtype=torch.float32, out=None,
                        accumulate=False):
    """Per-group D_g[N, K] = qa_t[N, cols_g] . qb_t[K, cols_g]^T; returns [G, N, K]."""
    _require_cuda(qa_t, "qa_t")
    if isinstance(m_splits, PadOffsets):   # the padded offsets a grouped quantize returned
        m_splits = m_splits.splits
    plan = grouped_plan(m_splits, qa_t.device)
    G = plan.groups
    N, K = qa_t.shape[0], qb_t.shape[0]
    assert qa_t.shape[1] == qb_t.shape[1] == plan.padded_rows
    if out is None:
        assert not accumulate
        out = torch.empty((G, N, K), dtype=out_dtype, device=qa_t.device)
    else:
        assert out.shape == (G, N, K) and out.dtype == out_dtype and out.is_contiguous()
    _lib.call("mt_grouped_wgrad_mxfp8", qa_t.data_ptr(), sa_t_swz.data_ptr(), qb_t.data_ptr(), sb_t_swz.data_ptr(),
              plan.ptr(), G, plan.rows, plan.padded_rows, N, K, out.data_ptr(), _out_dtype_code(out_dtype),
              int(accumulate), _stream())
    _count(1)
    return out


def set_launch_overlap(enabled: bool) -> bool:
    """Process-wide switch of the programmatically dependent kernel launches (on by default, see
    mt_set_launch_overlap in include/mt_b200.h); returns the previous setting."""
    return bool(_lib.load().mt_set_launch_overlap(1 if enabled else 0))


def read_device_status() -> int:
    """Status word raised by bounded device-side waits (0 = clean); clears it."""
    import ctypes
    v = ctypes.c_int(0)
    _lib.check(_lib.load().mt_read_device_status(ctypes.byref(v), _stream()), "mt_read_device_status")
    return v.value
