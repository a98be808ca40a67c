"""GPU parity of the drop-in modules (Linear, GroupedLinear) against the reference fixtures
and the numpy oracle: forward, dgrad and wgrad within 1e-3 relative Frobenius error, the
quantized operands underneath bit-exact."""
import numpy as np
import pytest
import torch

from conftest import bf16_bits_to_f32
from helpers import from_bits, mismatch, np_u8, padded_chunks, seeded_bf16, unswizzle_scales_ref
from minitransformer_b200 import kernels as K
from minitransformer_b200.module import config
from minitransformer_b200.module.group_linear import GroupedLinear
from minitransformer_b200.module.linear import Linear
from oracle import formats as F, gemm, linear as oracle_linear, mxfp8

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _relf(t, ref):
    return gemm.rel_frobenius(t.detach().float().cpu().numpy(), ref)


def _make_linear(K_in, N_out, recipe, w, **kw):
    params = config.get_qlinear_params_from_predefined(recipe)
    lin = Linear(K_in, N_out, bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params, **kw)
    with torch.no_grad():
        lin.weight.copy_(w)
    return lin


def test_linear_nvfp4_matches_reference_fixture(golden_nvfp4_linear):
    """Same inputs as the reference's _QuantizedLinear run stored in the fixture."""
    g = golden_nvfp4_linear
    for tag in ("a", "b"):
        x, w, dy = (from_bits(g[f"{tag}/{n}"]).cuda() for n in ("x", "w", "dy"))
        lin = _make_linear(x.shape[1], w.shape[0], config.QuantizeRecipe.FP4_SUB_CHANNEL, w)
        xd = x.clone().requires_grad_(True)
        y = lin(xd)
        y.backward(dy)
        assert _relf(y, bf16_bits_to_f32(g[f"{tag}/lin_y"])) <= TOL
        assert _relf(xd.grad, bf16_bits_to_f32(g[f"{tag}/lin_dx"])) <= TOL
        assert _relf(lin.weight.grad, g[f"{tag}/lin_dw"]) <= TOL
    assert K.read_device_status() == 0


@pytest.mark.parametrize("shape", [(256, 512, 384), (32 * 128, 1024, 4096), (16, 1024, 4096)])
@pytest.mark.parametrize("rht", [True, False])
def test_linear_nvfp4_matches_oracle(shape, rht):
    """Shapes from the reference's own module tests (batch 32 x seq 128 rows; 1024 -> 4096)."""
    M, Kd, N = shape
    tx, x = seeded_bf16((M, Kd), 1234)
    tw, w = seeded_bf16((N, Kd), 1235, 0.02)
    tdy, dy = seeded_bf16((M, N), 1236, 1e-3)
    ref = oracle_linear.nvfp4_linear_fwd_bwd(x, w, dy, with_rht=rht, fused=M * N * Kd > 5e7)
    recipe = config.QuantizeRecipe.FP4_SUB_CHANNEL if rht else config.QuantizeRecipe.FP4_SUB_CHANNEL_NO_RHT
    lin = _make_linear(Kd, N, recipe, tw.cuda(), fuse_wgrad_accumulation=True)
    lin.weight.main_grad = torch.zeros(N, Kd, dtype=torch.float32, device="cuda")
    xd = tx.cuda().requires_grad_(True)
    y = lin(xd.view(M // 16, 16, Kd), is_first_microbatch=True)   # 3-D input, like [seq, batch, hidden]
    assert y.shape == (M // 16, 16, N)
    y.backward(tdy.cuda().view(M // 16, 16, N))
    assert _relf(y.view(M, N), ref["y"]) <= TOL
    assert _relf(xd.grad, ref["dx"]) <= TOL
    assert _relf(lin.weight.main_grad, ref["dw"]) <= TOL
    assert lin.weight.grad is None  # the gradient went to main_grad
    # second microbatch: cached quantized weight, accumulation into main_grad
    xd2 = tx.cuda().requires_grad_(True)
    lin(xd2, is_first_microbatch=False).backward(tdy.cuda())
    assert _relf(lin.weight.main_grad, 2 * ref["dw"]) <= TOL
    assert K.read_device_status() == 0


def test_linear_mxfp8_matches_oracle():
    M, Kd, N = 512, 1024, 768
    tx, x = seeded_bf16((M, Kd), 11)
    tw, w = seeded_bf16((N, Kd), 12, 0.02)
    tdy, dy = seeded_bf16((M, N), 13, 1e-3)
    ref = oracle_linear.mxfp8_linear_fwd_bwd(x, w, dy, fused=True)
    lin = _make_linear(Kd, N, config.QuantizeRecipe.MXFP8_SUB_CHANNEL, tw.cuda())
    xd = tx.cuda().requires_grad_(True)
    y = lin(xd)
    y.backward(tdy.cuda())
    assert _relf(y, ref["y"]) <= TOL
    assert _relf(xd.grad, ref["dx"]) <= TOL
    assert _relf(lin.weight.grad, F.bf16_round(ref["dw"])) <= TOL


def test_linear_bias_and_return_bias():
    M, Kd, N = 128, 256, 256
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.FP4_SUB_CHANNEL_NO_RHT)
    lin = Linear(Kd, N, bias=True, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params)
    with torch.no_grad():
        lin.bias.normal_()
    x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    lin2 = Linear(Kd, N, bias=True, return_bias=True, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params)
    with torch.no_grad():
        lin2.weight.copy_(lin.weight)
        lin2.bias.copy_(lin.bias)
    y2, b2 = lin2(x)
    assert torch.allclose(y.float(), (y2.float() + b2.float()), atol=2e-2, rtol=2e-2)
    y.sum().backward()
    assert torch.allclose(lin.bias.grad.float(), torch.full((N,), float(M), device="cuda"))


def test_grouped_transpose_quantize_matches_oracle():
    m_splits = [130, 0, 64, 1, 257, 60]
    R, Kd = sum(m_splits), 256
    t, x = seeded_bf16((R, Kd), 5)
    q_t, s_swz, s_lin, pad = K.grouped_transpose_quantize_mxfp8(t.cuda(), m_splits, want_linear_scales=True)
    q_t, s_lin = np_u8(q_t), np_u8(s_lin)
    off = 0
    for g, m in enumerate(m_splits):
        p0, p1 = pad[g], pad[g + 1]
        assert p1 - p0 == (m + 127) // 128 * 128
        if m:
            o = mxfp8.quantize(x[off:off + m])
            assert mismatch(q_t[:, p0:p0 + m], o["data_t"]) == 0
            nb = (m + 31) // 32
            assert mismatch(s_lin[:, p0 // 32:p0 // 32 + nb], o["scale_t"]) == 0
        assert not q_t[:, p0 + m:p1].any()   # zero padding
        off += m
    assert mismatch(unswizzle_scales_ref(np_u8(s_swz), Kd, pad[-1] // 32), s_lin) == 0


@pytest.mark.parametrize("m_splits,cols", [([130, 0, 64, 1, 257, 60], 256), ([5, 7, 9, 11], 160), ([0, 384, 0], 96),
                                          ([128, 128, 128], 128)])
def test_grouped_quantize_with_transpose_equals_the_two_separate_passes(m_splits, cols):
    """The single-read kernel must write exactly the bytes of the row-wise quantize plus those of
    the grouped transposed quantize (checked against the oracle by the test above)."""
    R = sum(m_splits)
    t, _ = seeded_bf16((R, cols), 11)
    xt = t.cuda()
    row, (q_t, s_t_swz, pad) = K.grouped_quantize_mxfp8(xt, m_splits)
    ref = K.quantize_mxfp8(xt, return_transpose=False)
    ref_t, ref_s_t_swz, _, ref_pad = K.grouped_transpose_quantize_mxfp8(xt, m_splits)
    assert list(pad) == list(ref_pad)
    assert torch.equal(row.data, ref.data) and torch.equal(row.scale, ref.scale)
    kb = padded_chunks(cols // 32) * 4   # including the zero-filled padding blocks of the valid rows
    assert mismatch(unswizzle_scales_ref(np_u8(row.scale_swz), R, kb), unswizzle_scales_ref(np_u8(ref.scale_swz), R, kb)) == 0
    assert torch.equal(q_t, ref_t) and torch.equal(s_t_swz, ref_s_t_swz)
    assert K.read_device_status() == 0


@pytest.mark.parametrize("m_splits", [[128, 128, 128], [130, 0, 64, 1, 257, 60], [0, 0, 300], [5, 7, 9, 11]])
def test_grouped_linear_mxfp8_matches_oracle(m_splits):
    G, Kd, N = len(m_splits), 256, 384
    R = sum(m_splits)
    tx, x = seeded_bf16((R, Kd), 21)
    tdy, dy = seeded_bf16((R, N), 22, 1e-3)
    ws = [seeded_bf16((N, Kd), 30 + g, 0.02) for g in range(G)]
    ref = oracle_linear.mxfp8_grouped_fwd_bwd(x, [w[1] for w in ws], dy, m_splits)
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    gl = GroupedLinear(G, Kd, N, bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params)
    with torch.no_grad():
        for g in range(G):
            getattr(gl, f"weight{g}").copy_(ws[g][0])
    xd = tx.cuda().requires_grad_(True)
    y = gl(xd, m_splits)
    y.backward(tdy.cuda())
    assert _relf(y, ref["y"]) <= TOL
    assert _relf(xd.grad, ref["dx"]) <= TOL
    for g in range(G):
        got = getattr(gl, f"weight{g}").grad
        want = F.bf16_round(ref["dw"][g])
        if m_splits[g] == 0:
            assert float(got.abs().max()) == 0.0
        else:
            assert _relf(got, want) <= TOL
    assert K.read_device_status() == 0


def test_grouped_linear_main_grad_accumulation_in_place():
    """Megatron main_grad protocol for experts: with the main_grad buffers in one block the wgrad
    GEMM writes (first microbatch) or accumulates (later ones) in place; with separate buffers it
    goes through per-expert copies. Both must hold the same fp32 values."""
    m_splits = [130, 0, 64, 1, 257, 60]
    G, Kd, N = len(m_splits), 256, 384
    R = sum(m_splits)
    tx, _ = seeded_bf16((R, Kd), 41)
    tdy, _ = seeded_bf16((R, N), 42, 1e-3)
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    kw = dict(bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params)
    plain = GroupedLinear(G, Kd, N, **kw)
    layers = {"block": GroupedLinear(G, Kd, N, fuse_wgrad_accumulation=True, **kw),
              "separate": GroupedLinear(G, Kd, N, fuse_wgrad_accumulation=True, **kw)}
    block = torch.full((G, N, Kd), 7.0, dtype=torch.float32, device="cuda")   # stale contents must be overwritten
    for name, gl in layers.items():
        with torch.no_grad():
            for g in range(G):
                getattr(gl, f"weight{g}").copy_(getattr(plain, f"weight{g}"))
        for g in range(G):
            getattr(gl, f"weight{g}").main_grad = block[g] if name == "block" else \
                torch.full((N, Kd), 7.0, dtype=torch.float32, device="cuda")
    xd = tx.cuda().requires_grad_(True)
    plain(xd, m_splits).backward(tdy.cuda())
    for first in (True, False):
        for gl in layers.values():
            gl(tx.cuda().requires_grad_(True), m_splits, is_first_microbatch=first).backward(tdy.cuda())
    for g in range(G):
        a = getattr(layers["block"], f"weight{g}").main_grad
        b = getattr(layers["separate"], f"weight{g}").main_grad
        assert torch.equal(a, b), g
        want = 2.0 * getattr(plain, f"weight{g}").grad.float().cpu().numpy()
        if m_splits[g] == 0:
            assert float(a.abs().max()) == 0.0
        else:
            assert _relf(a, want) <= 5e-3, g     # the plain layer's gradient is rounded to bf16
    assert K.read_device_status() == 0


def test_grouped_linear_full_size_spot_checks():
    """Configuration-3 scale (128 experts, 131072 rows, seeded Zipf(1.1) group sizes with empty
    groups, hidden 2048 -> 768): expert slices of the grouped output against the dense kernel
    on the same slice; the padded transposed copies against per-group quantization."""
    G, R, Kd, N = 128, 131072, 2048, 768
    rng = np.random.default_rng(1234)
    p = 1.0 / np.arange(1, G + 1) ** 1.1
    ids = rng.choice(G, size=R, p=p / p.sum())
    m_splits = np.bincount(ids, minlength=G).tolist()
    assert sum(m_splits) == R
    gen = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(R, Kd, device="cuda", generator=gen).to(torch.bfloat16)
    w = (torch.randn(G, N, Kd, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    op = params.quantize_op
    qx = op.quantize(x, params.x_params)
    qw = op.grouped_quantize(w, params.w_params, return_transpose=True)
    y = op.grouped_qgemm(qx.data, qw.data, params.mm_fprop, torch.bfloat16, qx.scale, qw.scale, m_splits=m_splits,
                         weights_transposed=False, n_out=N)
    off = np.concatenate([[0], np.cumsum(m_splits)])
    for g in (0, 1, 17, 63, 127):
        r0, r1 = int(off[g]), int(off[g + 1])
        if r1 == r0:
            continue
        xs = K.quantize_mxfp8(x[r0:r1].contiguous(), return_transpose=False)
        ws = K.quantize_mxfp8(w[g].contiguous(), return_transpose=False)
        ref = K.gemm_mxfp8(xs.data, xs.scale_swz, ws.data, ws.scale_swz)
        err = float((y[r0:r1].float() - ref.float()).norm() / ref.float().norm())
        assert err <= TOL, (g, err)
    assert K.read_device_status() == 0


def test_grouped_linear_full_size_module_against_oracle():
    """Configuration 3 at size through the GroupedLinear module (128 experts, 131072 rows, seeded
    Zipf(1.1) sizes, hidden 2048 -> ffn 768; one expert forced to a single row and one to none):
    forward output, input gradient and weight gradient of a large expert, the one-row expert, the
    empty expert and the last expert against the oracle run on that expert's slice alone."""
    G, R, Kd, N = 128, 131072, 2048, 768
    rng = np.random.default_rng(1234)
    p = 1.0 / np.arange(1, G + 1) ** 1.1
    m = np.bincount(rng.choice(G, size=R, p=p / p.sum()), minlength=G)
    m[0] += m[40] - 1 + m[41]           # expert 40 keeps one row, expert 41 none; expert 0 takes the rest
    m[40], m[41] = 1, 0
    m_splits = m.tolist()
    assert sum(m_splits) == R and m_splits[127] > 0
    tx, x = seeded_bf16((R, Kd), 71)
    tdy, dy = seeded_bf16((R, N), 72, 1e-3)
    gen = torch.Generator().manual_seed(73)
    w_all = (torch.randn(G, N, Kd, generator=gen) * 0.02).to(torch.bfloat16)
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    gl = GroupedLinear(G, Kd, N, bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params,
                       fuse_wgrad_accumulation=True)
    block = torch.full((G, N, Kd), 3.0, dtype=torch.float32, device="cuda")   # stale values must be overwritten
    with torch.no_grad():
        for g in range(G):
            getattr(gl, f"weight{g}").copy_(w_all[g])
            getattr(gl, f"weight{g}").main_grad = block[g]
    xd = tx.cuda().requires_grad_(True)
    y = gl(xd, m_splits, is_first_microbatch=True)
    y.backward(tdy.cuda())
    torch.cuda.synchronize()
    off = np.concatenate([[0], np.cumsum(m_splits)])
    for g in (1, 40, 41, 127):
        r0, r1 = int(off[g]), int(off[g + 1])
        dw = block[g]
        if r1 == r0:
            assert float(dw.abs().max()) == 0.0
            continue
        ref = oracle_linear.mxfp8_linear_fwd_bwd(x[r0:r1], w_all[g].float().numpy(), dy[r0:r1], fused=True)
        assert _relf(y[r0:r1], ref["y"]) <= TOL, g
        assert _relf(xd.grad[r0:r1], ref["dx"]) <= TOL, g
        assert _relf(dw, ref["dw"]) <= TOL, g
    assert K.read_device_status() == 0


def test_grouped_plan_rejects_bad_offsets_without_touching_outputs():
    """Offsets that do not partition [0, rows) leave an empty plan: the grouped GEMM computes
    nothing and the device status word carries the bad-plan bit (32)."""
    from minitransformer_b200 import _lib
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    G, R, Kd, N = 3, 384, 128, 256
    off = torch.tensor([0, 200, 100, 384], dtype=torch.int64, device="cuda")     # not monotonic
    plan = torch.zeros(int(lib.mt_grouped_plan_bytes(R, G)), dtype=torch.uint8, device="cuda")
    _lib.check(lib.mt_grouped_plan_build(off.data_ptr(), G, R, plan.data_ptr(), plan.numel(), st), "plan")
    x = torch.randn(R, Kd, device="cuda").to(torch.bfloat16)
    w = torch.randn(G * N, Kd, device="cuda").to(torch.bfloat16)
    qx, qw = K.quantize_mxfp8(x, return_transpose=False), K.quantize_mxfp8(w, return_transpose=False)
    out = torch.full((R, N), 5.0, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.mt_grouped_gemm_mxfp8(qx.data.data_ptr(), qx.scale_swz.data_ptr(), qw.data.data_ptr(),
                                         qw.scale_swz.data_ptr(), G * N, Kd, plan.data_ptr(), G, R, N, Kd, N, 0,
                                         out.data_ptr(), _lib.MT_BF16, N, st), "gemm")
    torch.cuda.synchronize()
    assert float((out.float() - 5.0).abs().max()) == 0.0
    assert K.read_device_status() == 32
    assert K.read_device_status() == 0


@pytest.mark.parametrize("recipe", [config.QuantizeRecipe.FP4_SUB_CHANNEL, config.QuantizeRecipe.MXFP8_SUB_CHANNEL])
def test_kept_quantized_weights_and_their_checkpoint(recipe):
    """keep_quantized_weights(): the forward stops re-quantizing (whatever is_first_microbatch says)
    until refresh_quantized_weights(); the quantized copies travel in the state dict and a fresh
    layer that loads it computes with them, forward and backward, without a quantize pass."""
    M, Kd, N = 256, 512, 384
    tx, _ = seeded_bf16((M, Kd), 81)
    tw, _ = seeded_bf16((N, Kd), 82, 0.02)
    tdy, _ = seeded_bf16((M, N), 83, 1e-3)
    lin = _make_linear(Kd, N, recipe, tw.cuda())
    lin.keep_quantized_weights()
    x = tx.cuda()
    y0 = lin(x, is_first_microbatch=True).detach()
    with torch.no_grad():
        lin.weight.mul_(2)                       # the kept copies still describe the old weight
    assert torch.equal(lin(x, is_first_microbatch=True).detach(), y0)
    sd = lin.state_dict()
    assert sd["_extra_state"] is not None
    fresh = _make_linear(Kd, N, recipe, torch.zeros(N, Kd, dtype=torch.bfloat16, device="cuda"))
    fresh.load_state_dict(sd)
    xd = x.clone().requires_grad_(True)
    y1 = fresh(xd)
    assert torch.equal(y1.detach(), y0)
    y1.backward(tdy.cuda())
    ref = _make_linear(Kd, N, recipe, tw.cuda())
    xr = x.clone().requires_grad_(True)
    ref(xr).backward(tdy.cuda())
    assert torch.equal(xd.grad, xr.grad)         # dgrad used the restored transposed copy of the old weight
    lin.refresh_quantized_weights()
    assert torch.equal(lin(x).detach(), 2 * y0)  # now the doubled weight: same codes, doubled scale
    assert K.read_device_status() == 0


def test_prefetched_weight_quantization_gives_the_same_step():
    """prefetch_quantized_weight() moves the weight's quantize pass to a side stream ahead of the
    forward call; outputs and gradients are those of the ordinary call."""
    M, Kd, N = 512, 1024, 768
    tx, _ = seeded_bf16((M, Kd), 91)
    tw, _ = seeded_bf16((N, Kd), 92, 0.02)
    tdy, _ = seeded_bf16((M, N), 93, 1e-3)
    outs = []
    for prefetch in (False, True):
        lin = _make_linear(Kd, N, config.QuantizeRecipe.FP4_SUB_CHANNEL, tw.cuda())
        x = tx.cuda().requires_grad_(True)
        if prefetch:
            lin.prefetch_quantized_weight()
        y = lin(x, is_first_microbatch=True)
        y.backward(tdy.cuda())
        outs.append((y.detach(), x.grad, lin.weight.grad))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert K.read_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_linear_accepts_fp32_and_fp16_activations(dtype):
    """The reference module takes fp32 / fp16 / bf16 activations with parameters of the same type
    (its own module grid runs fp32 as well). Here such inputs are rounded to bf16 before the
    quantize kernels, so the result equals the bf16 layer on the rounded tensors, returned in the
    caller's type."""
    M, Kd, N = 256, 512, 384
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, Kd, generator=g).to(dtype).cuda()
    w = (torch.randn(N, Kd, generator=g) * 0.02).to(dtype).cuda()
    dy = (torch.randn(M, N, generator=g) * 1e-3).to(dtype).cuda()
    params = config.get_qlinear_params_from_predefined(config.QuantizeRecipe.FP4_SUB_CHANNEL)
    lin = Linear(Kd, N, bias=True, params_dtype=dtype, device="cuda", qlinear_params=params)
    with torch.no_grad():
        lin.weight.copy_(w)
        lin.bias.fill_(0.25)
    xd = x.clone().requires_grad_(True)
    y = lin(xd)
    y.backward(dy)
    assert y.dtype == dtype and xd.grad.dtype == dtype and lin.weight.grad.dtype == dtype
    ref = _make_linear(Kd, N, config.QuantizeRecipe.FP4_SUB_CHANNEL, w.to(torch.bfloat16))
    xr = x.to(torch.bfloat16).requires_grad_(True)
    yr = ref(xr)
    yr.backward(dy.to(torch.bfloat16))
    tol = 1e-2 if dtype == torch.float16 else 5e-3     # the bf16 layer rounds its outputs to bf16
    assert _relf(y - 0.25, yr.detach().float().cpu().numpy()) <= tol
    assert _relf(xd.grad, xr.grad.float().cpu().numpy()) <= tol
    assert _relf(lin.weight.grad, ref.weight.grad.float().cpu().numpy()) <= tol
    assert torch.allclose(lin.bias.grad.float(), dy.float().sum(0), rtol=1e-2, atol=1e-4)
    assert K.read_device_status() == 0


@pytest.mark.parametrize("recipe", [config.QuantizeRecipe.FP4_SUB_CHANNEL, config.QuantizeRecipe.FP4_SUB_CHANNEL_NO_RHT,
                                    config.QuantizeRecipe.MXFP8_SUB_CHANNEL])
def test_bias_gradient_from_the_quantize_pass(recipe):
    """b_grad = sum over tokens of dy (miniTransformer/module/linear.py:352): with the NVFP4 recipes
    it is taken from the abs-max pass of the dy quantization, with MXFP8 (no such pass) from a
    reduction of its own; both must equal the fp64 column sums to bf16 rounding."""
    M, Kd, N = 512, 256, 384
    tx, _ = seeded_bf16((M, Kd), 101)
    tw, _ = seeded_bf16((N, Kd), 102, 0.02)
    tdy, dy = seeded_bf16((M, N), 103, 1e-3)
    params = config.get_qlinear_params_from_predefined(recipe)
    lin = Linear(Kd, N, bias=True, params_dtype=torch.bfloat16, device="cuda", qlinear_params=params)
    with torch.no_grad():
        lin.weight.copy_(tw)
    lin(tx.cuda().requires_grad_(True)).backward(tdy.cuda())
    want = dy.astype(np.float64).sum(0)
    got = lin.bias.grad.float().cpu().numpy().astype(np.float64)
    assert np.abs(got - want).max() <= 2 ** -8 * np.abs(want).max() + 1e-9
    assert K.read_device_status() == 0
