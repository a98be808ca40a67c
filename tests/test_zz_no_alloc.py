"""The grouped GEMM entry point that brings its own scratch memory.

Some users of this library cannot pass a buffer for the grouped plan: another allocator already
owns all free GPU memory, or they are inside a loop where a device allocation (and the
device-wide synchronisation it implies) is not acceptable. `mt_grouped_gemm_mxfp8_static` serves
them from a fixed array inside the library. This file checks, through the C ABI, that it returns
what `mt_grouped_gemm_mxfp8` returns for the same operands, twice in a row with different group
layouts (the array keeps the first call's tables), and that problems beyond its built-in
limits are refused with a clear message. It is named to be collected last.
"""
import pytest
import torch

from minitransformer_b200 import _lib, kernels as K

pytestmark = pytest.mark.gpu
TOL = 1e-3  # relative Frobenius error, the tolerance of the other GEMM tests


def _offsets(m_splits):
    """Group offsets as a device int64 tensor, and the row total."""
    off = [0]
    for m in m_splits:
        off.append(off[-1] + m)
    return torch.tensor(off, dtype=torch.int64, device="cuda"), off[-1]


def _run_both(m_splits, Kd, N, seed):
    lib = _lib.load()
    G = len(m_splits)
    arr, R = _offsets(m_splits)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(R, Kd, device="cuda", generator=gen).to(torch.bfloat16)
    w = (torch.randn(G * N, Kd, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    qx = K.quantize_mxfp8(x, return_transpose=False)
    qw = K.quantize_mxfp8(w, return_transpose=False)
    stream = torch.cuda.current_stream().cuda_stream

    want = torch.zeros(R, N, dtype=torch.bfloat16, device="cuda")
    plan = torch.empty(int(lib.mt_grouped_plan_bytes(R, G)), dtype=torch.uint8, device="cuda")
    _lib.check(lib.mt_grouped_plan_build(arr.data_ptr(), G, R, plan.data_ptr(), plan.numel(), stream),
               "mt_grouped_plan_build")
    _lib.check(lib.mt_grouped_gemm_mxfp8(qx.data.data_ptr(), qx.scale_swz.data_ptr(), qw.data.data_ptr(),
                                         qw.scale_swz.data_ptr(), G * N, Kd, plan.data_ptr(), G, R, N, Kd, N, 0,
                                         want.data_ptr(), _lib.MT_BF16, N, stream),
               "mt_grouped_gemm_mxfp8")
    got = torch.zeros(R, N, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.mt_grouped_gemm_mxfp8_static(qx.data.data_ptr(), qx.scale_swz.data_ptr(), qw.data.data_ptr(),
                                                qw.scale_swz.data_ptr(), G * N, Kd, arr.data_ptr(), G, R, N, Kd, N, 0,
                                                got.data_ptr(), _lib.MT_BF16, N, stream),
               "mt_grouped_gemm_mxfp8_static")
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    # first call: many groups and row blocks; second call: fewer of both, so leftovers of the
    # first call's tables sit behind the part the second call rewrites
    for m_splits, seed in (([300, 0, 129, 64, 1, 500, 77, 0, 200], 1), ([40, 260], 2)):
        got, want = _run_both(m_splits, 256, 384, seed)
        assert float(want.float().abs().max()) > 0
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err <= TOL, (m_splits, err)
        assert torch.equal(got, want)
    assert K.read_device_status() == 0


def test_static_scratch_entry_point_refuses_oversized_problems():
    lib = _lib.load()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    too_many = 1025
    arr, rows = _offsets([0] * too_many)
    rc = lib.mt_grouped_gemm_mxfp8_static(p, p, p, p, 128, 128, arr.data_ptr(), too_many, rows, 128, 128, 128, 0, p,
                                          _lib.MT_BF16, 128, None)
    assert rc == -1 and b"limit of 1024" in lib.mt_last_error_string()
    arr, rows = _offsets([1048576 + 128])
    rc = lib.mt_grouped_gemm_mxfp8_static(p, p, p, p, 128, 128, arr.data_ptr(), 1, rows, 128, 128, 128, 0, p,
                                          _lib.MT_BF16, 128, None)
    assert rc == -1 and b"limit of 1048576" in lib.mt_last_error_string()
