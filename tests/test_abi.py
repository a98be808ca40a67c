"""CPU-side checks of the drop-in boundary: the shared library loads and exports every
function the public header declares, and argument validation fails loudly without a GPU."""
import ctypes
import os

import pytest

from minitransformer_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _lib.declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mt_b200.h but not exported"
    assert set(names) == set(_lib._SIGNATURES), "ctypes signatures out of sync with the header"
    assert lib.mt_version() >= 100


def test_swizzled_scale_bytes():
    lib = _lib.load()
    assert lib.mt_swizzled_scale_bytes(128, 4) == 4 * 512      # one chunk, padded to four
    assert lib.mt_swizzled_scale_bytes(8192, 256) == 64 * 64 * 512
    assert lib.mt_swizzled_scale_bytes(130, 17) == 2 * 8 * 512


def test_invalid_arguments_are_rejected_with_a_message():
    lib = _lib.load()
    rc = lib.mt_quantize_nvfp4(None, 16, 16, 0, None, None, None, None, 1, None, None, None, 1, None, None)
    assert rc == -1
    assert b"null" in lib.mt_last_error_string()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 15) // 16 * 16
    rc = lib.mt_quantize_nvfp4(p, 16, 24, 0, p, p, p, p, 1, None, None, None, 1, None, None)
    assert rc == -1 and b"multiple of 16" in lib.mt_last_error_string()
    rc = lib.mt_gemm_nvfp4(p, p, p, p, p, p, 128, 128, 40, p, 0, 128, None, 0, 0, None, None)
    assert rc == -1 and b"multiple of 32" in lib.mt_last_error_string()
    rc = lib.mt_gemm_mxfp8(p, p, p, p, 128, 128, 64, p, 7, 128, None, 0, 0, None, None)
    assert rc == -1 and b"dtype" in lib.mt_last_error_string()
    with pytest.raises(_lib.MtError):
        _lib.call("mt_swizzle_scales", None, 1, 1, 1, None, None)
    # K-slab operands: every slab must hold whole 128-byte K steps, and the shapes must be ones
    # the CTA-pair kernel takes
    rc = lib.mt_gemm_nvfp4_kslab(p, p, p, 3, p, p, p, 1, 512, 512, 1024, p, 0, 512, None, 0, 0, None, None)
    assert rc == -1 and b"slab" in lib.mt_last_error_string()
    rc = lib.mt_gemm_mxfp8_kslab(p, p, 2, p, p, 1, 128, 512, 1024, p, 0, 512, None, 0, 0, None, None)
    assert rc == -1 and b"M > 128" in lib.mt_last_error_string()
    rc = lib.mt_gemm_mxfp8_kslab(p, p, 0, p, p, 1, 512, 512, 1024, p, 0, 512, None, 0, 0, None, None)
    assert rc == -1 and b"positive" in lib.mt_last_error_string()
    bad = _lib.GemmOpts(-1, None)
    rc = lib.mt_gemm_mxfp8(p, p, p, p, 256, 256, 128, p, 0, 256, None, 0, 0, ctypes.byref(bad), None)
    assert rc == -1 and b"SM count" in lib.mt_last_error_string()
    both = _lib.GemmOpts(0, p)
    rc = lib.mt_gemm_mxfp8(p, p, p, p, 256, 256, 128, p, 1, 256, None, 0, 1, ctypes.byref(both), None)
    assert rc == -1 and b"accumulate" in lib.mt_last_error_string()
    rc = lib.mt_grouped_quantize_mxfp8(p, 9, 64, p, 2, 256, None, None, 2, None, p, None, 8, p, None)
    assert rc == -1 and b"null q" in lib.mt_last_error_string()
    # grouped plan: sizes and argument checks (the plan itself is built on the device)
    assert lib.mt_grouped_plan_bytes(131072, 128) >= 64 + 2 * 129 * 8 + (1024 + 128) * 32
    assert lib.mt_grouped_plan_bytes(-1, 4) == 0 and lib.mt_grouped_plan_bytes(16, 0) == 0
    rc = lib.mt_grouped_plan_build(p, 2, 9, p, 16, None)
    assert rc == -1 and b"too small" in lib.mt_last_error_string()
    rc = lib.mt_grouped_wgrad_mxfp8(p, p, p, p, p, 2, 9, 100, 128, 128, p, 1, 0, None)
    assert rc == -1 and b"multiple of 128" in lib.mt_last_error_string()
    rc = lib.mt_test_bounded_wait(0, None)
    assert rc == -1 and b"limit" in lib.mt_last_error_string()


def test_front_end_refuses_cpu_tensors():
    import torch
    from minitransformer_b200 import kernels
    with pytest.raises(_lib.MtError):
        kernels.quantize_nvfp4(torch.zeros(16, 16, dtype=torch.bfloat16))


def test_stacked_view_of_adjacent_parameters_is_copy_free():
    """Expert weights allocated as views of one block are read as one stacked tensor; separate
    allocations are reported as not stackable (the caller then copies)."""
    import torch
    from minitransformer_b200.module._common import stacked_view
    from minitransformer_b200.module import group_linear  # noqa: F401  (the module imports cleanly)
    block = torch.randn(4, 3, 5)
    params = [torch.nn.Parameter(block[i]) for i in range(4)]
    view = stacked_view(params)
    assert view is not None and view.shape == (4, 3, 5)
    assert view.data_ptr() == block.data_ptr() and torch.equal(view, block)
    assert stacked_view([torch.randn(3, 5) for _ in range(3)]) is None
    assert stacked_view([block[0], block[2]]) is None
    # the verdict is remembered per set of addresses: re-pointing a middle tensor must be noticed
    params[2].data = torch.randn(3, 5)
    assert stacked_view(params) is None
    params[2] = torch.nn.Parameter(torch.randn(3, 5))
    assert stacked_view(params) is None


def test_padded_offsets_of_a_split_list():
    from minitransformer_b200 import kernels
    assert kernels.grouped_padded_offsets([3, 0, 5]) == [0, 128, 128, 256]
    assert kernels.grouped_padded_offsets([128, 129]) == [0, 128, 384]


def test_launch_overlap_switch_reports_the_previous_setting():
    """Pure host state: on by default, the call returns what was set before."""
    lib = _lib.load()
    before = lib.mt_set_launch_overlap(0)
    try:
        assert before in (0, 1)
        assert lib.mt_set_launch_overlap(1) == 0
        assert lib.mt_set_launch_overlap(1) == 1
    finally:
        lib.mt_set_launch_overlap(before)


def test_quantize_flag_values_match_the_header():
    import re
    text = open(_lib.HEADER_PATHS[0]).read()
    for name in ("MT_Q_2D", "MT_Q_RHT", "MT_Q_ROWPAD16", "MT_Q_AMAX_ZEROED"):
        m = re.search(name + r"\s*=\s*(\d+)", text)
        assert m and int(m.group(1)) == getattr(_lib, name), name
