"""GPU parity of the tcgen05 block-scaled GEMM kernels through the C ABI: relative
Frobenius error <= 1e-3 (the stated tolerance) against the oracle GEMM on the SAME
quantized operands; at full configuration sizes against the CUDA-core checker."""
import numpy as np
import pytest
import torch

from conftest import bf16_bits_to_f32
from helpers import from_bits, seeded_bf16
from minitransformer_b200 import kernels as K
from oracle import formats as F, gemm, mxfp8, nvfp4

pytestmark = pytest.mark.gpu

TOL = 1e-3  # relative Frobenius error against the reference GEMM on identical operands


def _operands_nvfp4(M, N, Kd, seed=1):
    ta, a = seeded_bf16((M, Kd), seed)
    tb, b = seeded_bf16((N, Kd), seed + 1, 0.02)
    return (nvfp4.quantize(a, return_transpose=False), nvfp4.quantize(b, return_transpose=False),
            K.quantize_nvfp4(ta.cuda(), return_transpose=False), K.quantize_nvfp4(tb.cuda(), return_transpose=False))


def _operands_mxfp8(M, N, Kd, seed=1):
    ta, a = seeded_bf16((M, Kd), seed)
    tb, b = seeded_bf16((N, Kd), seed + 1, 0.02)
    return (mxfp8.quantize(a, return_transpose=False), mxfp8.quantize(b, return_transpose=False),
            K.quantize_mxfp8(ta.cuda(), return_transpose=False), K.quantize_mxfp8(tb.cuda(), return_transpose=False))


SHAPES = [(128, 128, 256), (128, 256, 256), (128, 128, 32), (256, 512, 1024), (100, 72, 96), (384, 640, 2048),
          (1, 8, 64), (129, 257, 288), (512, 128, 4096),
          # register-store epilogue of the pair kernel: a row mask inside a 32-row block, a last
          # column tile of 16 (bf16) / 8 (fp32) columns
          (300, 272, 512), (520, 264, 256)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_nvfp4_matches_oracle(shape, out_dtype):
    M, N, Kd = shape
    oa, ob, ra, rb = _operands_nvfp4(M, N, Kd)
    ref = gemm.qgemm_nvfp4(oa["data"], oa["scale"], oa["amax_row"], ob["data"], ob["scale"], ob["amax_row"],
                           out_bf16=out_dtype == torch.bfloat16, fused=M * N * Kd > 5e7)
    y = K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row, rb.data, rb.scale_swz, rb.amax_row, out_dtype=out_dtype)
    assert gemm.rel_frobenius(y.float().cpu().numpy(), ref) <= TOL
    chk = K.gemm_nvfp4(ra.data, None, ra.amax_row, rb.data, None, rb.amax_row, out_dtype=out_dtype,
                       check_kernel=True, sa_lin=ra.scale, sb_lin=rb.scale)
    assert gemm.rel_frobenius(chk.float().cpu().numpy(), ref) <= TOL
    assert K.read_device_status() == 0


@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_mxfp8_matches_oracle(shape):
    M, N, Kd = shape
    Kd = max(32, Kd // 32 * 32)
    oa, ob, ra, rb = _operands_mxfp8(M, N, Kd)
    ref = gemm.qgemm_mxfp8(oa["data"], oa["scale"], ob["data"], ob["scale"], out_bf16=False, fused=M * N * Kd > 5e7)
    y = K.gemm_mxfp8(ra.data, ra.scale_swz, rb.data, rb.scale_swz, out_dtype=torch.float32)
    assert gemm.rel_frobenius(y.cpu().numpy(), ref) <= TOL
    chk = K.gemm_mxfp8(ra.data, None, rb.data, None, out_dtype=torch.float32, check_kernel=True,
                       sa_lin=ra.scale, sb_lin=rb.scale)
    assert gemm.rel_frobenius(chk.cpu().numpy(), ref) <= TOL
    assert K.read_device_status() == 0


def test_gemm_matches_reference_fixture(golden_nvfp4_linear):
    """Operands quantized on the GPU from the fixture inputs, GEMM against the reference's own
    qgemm output stored in the fixture."""
    g = golden_nvfp4_linear
    for tag in ("a", "b"):
        x, w = from_bits(g[f"{tag}/x"]).cuda(), from_bits(g[f"{tag}/w"]).cuda()
        rx = K.quantize_nvfp4(x, with_rht=True)
        rw = K.quantize_nvfp4(w, tile=(16, 16))
        y = K.gemm_nvfp4(rx.data, rx.scale_swz, rx.amax_row, rw.data, rw.scale_swz, rw.amax_row)
        ref = bf16_bits_to_f32(g[f"{tag}/gemm_y"])
        assert gemm.rel_frobenius(y.float().cpu().numpy(), ref) <= TOL
        acc = torch.from_numpy(g[f"{tag}/acc_in"]).cuda()
        K.gemm_nvfp4(rx.data, rx.scale_swz, rx.amax_row, rw.data, rw.scale_swz, rw.amax_row,
                     out_dtype=torch.float32, out=acc, accumulate=True)
        assert gemm.rel_frobenius(acc.cpu().numpy(), g[f"{tag}/acc_out"]) <= TOL


def test_gemm_accumulate_bias_and_strided_output():
    M, N, Kd = 256, 384, 512
    oa, ob, ra, rb = _operands_nvfp4(M, N, Kd, seed=11)
    base = gemm.qgemm_nvfp4(oa["data"], oa["scale"], oa["amax_row"], ob["data"], ob["scale"], ob["amax_row"],
                            out_bf16=False)
    g = torch.Generator().manual_seed(5)
    prev = torch.randn(M, N, generator=g)
    bias = torch.randn(N, generator=g)
    out = prev.clone().cuda()
    K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row, rb.data, rb.scale_swz, rb.amax_row, out_dtype=torch.float32,
                 out=out, accumulate=True)
    assert gemm.rel_frobenius(out.cpu().numpy(), prev.numpy() + base) <= TOL
    y = K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row, rb.data, rb.scale_swz, rb.amax_row,
                     out_dtype=torch.float32, bias=bias.cuda())
    assert gemm.rel_frobenius(y.cpu().numpy(), base + bias.numpy()[None, :]) <= TOL
    # bf16 accumulate into a view with a row stride larger than N
    big = torch.zeros(M, N + 64, dtype=torch.bfloat16, device="cuda")
    view = big[:, :N]
    view.copy_(prev.to(torch.bfloat16))
    K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row, rb.data, rb.scale_swz, rb.amax_row, out=view, accumulate=True)
    exp = F.bf16_round(F.bf16_round(prev.numpy()) + base)
    assert gemm.rel_frobenius(view.float().cpu().numpy(), exp) <= 4e-3  # one bf16 ulp of slack
    assert float(big[:, N:].abs().max()) == 0.0


def test_gemm_zero_k_and_zero_operands():
    a = torch.zeros(128, 0, dtype=torch.uint8, device="cuda")
    one = torch.ones(1, device="cuda")
    y = torch.full((128, 64), 7.0, device="cuda")
    K.gemm_nvfp4(a, a, one, a[:64], a, one, out_dtype=torch.float32, out=y)
    assert float(y.abs().max()) == 0.0
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    r = K.quantize_nvfp4(x, return_transpose=False)
    y = K.gemm_nvfp4(r.data, r.scale_swz, r.amax_row, r.data, r.scale_swz, r.amax_row, out_dtype=torch.float32)
    assert float(y.abs().max()) == 0.0 and not bool(torch.isnan(y).any())


FULL_SIZE = {
    # configuration 2 (tokens 8192, in 4096, out 14336): (M, N, K, output type, accumulate)
    "fprop": (8192, 14336, 4096, torch.float32, False),
    "dgrad": (8192, 4096, 14336, torch.bfloat16, False),
    "wgrad": (14336, 4096, 8192, torch.float32, False),
    "wgrad_accumulate": (14336, 4096, 8192, torch.float32, True),
}


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("which", list(FULL_SIZE))
def test_gemm_full_size_against_device_checker(fmt, which):
    """The three GEMMs of configuration 2 at size (fprop 8192 x 14336 x 4096; dgrad with K = 14336
    and bf16 output; wgrad with K = 8192 and fp32 output, written and accumulated): the
    tensor-core kernel against the CUDA-core checker, which itself is pinned to the oracle at
    small sizes above."""
    M, N, Kd, out_dtype, accumulate = FULL_SIZE[which]
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, Kd, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kd, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    prev = torch.randn(M, N, device="cuda", generator=g) * 0.5 if accumulate else None
    out = prev.clone() if accumulate else None
    if fmt == "nvfp4":
        ra, rb = K.quantize_nvfp4(x, return_transpose=False), K.quantize_nvfp4(w, return_transpose=False)
        y = K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row, rb.data, rb.scale_swz, rb.amax_row, out_dtype=out_dtype,
                         out=out, accumulate=accumulate)
        c = K.gemm_nvfp4(ra.data, None, ra.amax_row, rb.data, None, rb.amax_row, out_dtype=torch.float32,
                         check_kernel=True, sa_lin=ra.scale, sb_lin=rb.scale)
    else:
        ra, rb = K.quantize_mxfp8(x, return_transpose=False), K.quantize_mxfp8(w, return_transpose=False)
        y = K.gemm_mxfp8(ra.data, ra.scale_swz, rb.data, rb.scale_swz, out_dtype=out_dtype, out=out,
                         accumulate=accumulate)
        c = K.gemm_mxfp8(ra.data, None, rb.data, None, out_dtype=torch.float32, check_kernel=True,
                         sa_lin=ra.scale, sb_lin=rb.scale)
    if accumulate:
        c = c + prev
    # bf16 outputs carry one rounding of the fp32 accumulator (relative 2^-9 per element at most)
    tol = TOL if out_dtype == torch.float32 else 3e-3
    assert float((y.float() - c).norm() / c.norm()) <= tol
    # linearity in the per-tensor scale (NVFP4): doubling amax_a doubles the output
    if fmt == "nvfp4" and not accumulate:
        y2 = K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row * 2, rb.data, rb.scale_swz, rb.amax_row,
                          out_dtype=out_dtype)
        assert torch.equal(y2, y * 2)
    assert K.read_device_status() == 0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("shape,out_dtype", [((512, 768, 1024), torch.bfloat16), ((512, 768, 1024), torch.float32),
                                             ((100, 72, 96), torch.bfloat16), ((300, 520, 512), torch.bfloat16)])
def test_gemm_emits_abs_max_of_its_output(fmt, shape, out_dtype):
    """mt_gemm_opts.d_amax: the GEMM raises a device scalar to max |stored value|, bit-identical
    to a separate abs-max pass over the stored output (what the next layer's NVFP4 quantize
    would otherwise compute by re-reading it)."""
    M, N, Kd = shape
    if fmt == "nvfp4":
        _, _, ra, rb = _operands_nvfp4(M, N, Kd, seed=21)
        run = lambda: K.gemm_nvfp4(ra.data, ra.scale_swz, ra.amax_row, rb.data, rb.scale_swz, rb.amax_row,
                                   out_dtype=out_dtype)
    else:
        _, _, ra, rb = _operands_mxfp8(M, N, Kd, seed=21)
        run = lambda: K.gemm_mxfp8(ra.data, ra.scale_swz, rb.data, rb.scale_swz, out_dtype=out_dtype)
    plain = run()
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    with K.gemm_options(d_amax=amax):
        y = run()
    assert torch.equal(y, plain)
    assert float(amax) == float(y.float().abs().max()) and float(amax) > 0
    if out_dtype == torch.bfloat16 and M % 16 == 0 and N % 16 == 0:
        a2, _ = K.amax_bf16(y, need_col=False)
        assert float(a2) == float(amax)
    assert K.read_device_status() == 0


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier nobody signals returns after its limit (1 ms here), raises its bit in
    the device status word once, and the context stays usable."""
    from minitransformer_b200 import _lib
    assert K.read_device_status() == 0
    _lib.call("mt_test_bounded_wait", 1_000_000, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert K.read_device_status() == 1      # DS_TMA_WAIT
    assert K.read_device_status() == 0      # cleared by the read
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0


def test_launch_overlap_switch_changes_no_result():
    """quantize -> GEMM -> quantize -> GEMM with the programmatically dependent launches on and
    off: bit-identical outputs, clean status word, and the switch reports its previous setting."""
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(1024, 512, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(768, 512, device="cuda", generator=g) * 0.05).to(torch.bfloat16)

    def chain():
        qx, qw = K.quantize_nvfp4(x, with_rht=True), K.quantize_nvfp4(w)
        y = K.gemm_nvfp4(qx.data, qx.scale_swz, qx.amax_row, qw.data, qw.scale_swz, qw.amax_row)
        qy = K.quantize_mxfp8(y, return_transpose=False)
        qw8 = K.quantize_mxfp8(w.t().contiguous()[:, :768].contiguous(), return_transpose=False)
        z = K.gemm_mxfp8(qy.data, qy.scale_swz, qw8.data, qw8.scale_swz, out_dtype=torch.float32)
        return y, z

    before = K.set_launch_overlap(False)
    try:
        y0, z0 = chain()
        assert K.set_launch_overlap(True) is False
        y1, z1 = chain()
        assert K.set_launch_overlap(True) is True
    finally:
        K.set_launch_overlap(before)
    assert torch.equal(y0, y1) and torch.equal(z0, z1)
    assert K.read_device_status() == 0
