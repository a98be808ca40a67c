"""Head-to-head check against the reference's own CUDA kernel (`quantize_transpose_nvfp4`, its only
native code), when it has been built into oracle/_ref/ by oracle/build_ref_kernel.py. The
reference kernel fixes the per-tensor scale to 1 and has no Hadamard transform
(csrc/ops/fp4/quantization/quantize_transpose_nvfp4.cu:219-225), so this library is run with a
per-tensor abs-max of 448 * 6 = 2688, for which its scale is 1 as well."""
import importlib.util
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "fp4_gemm.so")


def _load_reference_kernel():
    if not os.path.exists(_SO):
        pytest.skip("oracle/_ref/fp4_gemm.so has not been built (python oracle/build_ref_kernel.py <reference>)")
    spec = importlib.util.spec_from_file_location("fp4_gemm", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("use_2d", [False, True])
def test_codes_and_scales_equal_the_reference_kernel(use_2d):
    """Shape and seed of the reference's own kernel test
    (tests/python/nvfp4/test_nvfp4_quantize_exact.py:22-49): randn(1024, 4096) bf16, seed 0."""
    ref = _load_reference_kernel()
    from minitransformer_b200 import kernels as K
    torch.manual_seed(0)
    M, N = 1024, 4096
    x = torch.randn(M, N, dtype=torch.bfloat16, device="cuda")
    qx = torch.empty(M, N // 2, dtype=torch.uint8, device="cuda")
    sx = torch.empty(M, N // 16, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    qx_t = torch.empty(N, M // 2, dtype=torch.uint8, device="cuda")
    sx_t = torch.empty(N, M // 16, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    ref.quantize_transpose_nvfp4(x, qx, sx, qx_t, sx_t, use_2d, True)
    torch.cuda.synchronize()

    amax = torch.full((2,), 2688.0, dtype=torch.float32, device="cuda")
    ours = K.quantize_nvfp4(x, tile=(16, 16) if use_2d else (1, 16), with_2d=use_2d, with_rht=False,
                            return_transpose=True, amax_row=amax[0:1], amax_col=amax[1:2])
    torch.cuda.synchronize()

    def frac_diff(a, b):
        a, b = a.view(torch.uint8), b.view(torch.uint8)
        return float((a != b).float().mean())

    # the reference multiplies the block abs-max by fp32(1/6) where the emulation (and this
    # library) divides by 6: a scale byte may differ where the two quotients straddle an E4M3
    # rounding boundary, which random data practically never hits
    d = {
        "scale": frac_diff(ours.scale[:M], sx), "codes": frac_diff(ours.data, qx),
        "scale_t": frac_diff(ours.scale_t[:N], sx_t), "codes_t": frac_diff(ours.data_t, qx_t),
    }
    assert max(d.values()) <= 1e-4, d
    assert K.read_device_status() == 0
