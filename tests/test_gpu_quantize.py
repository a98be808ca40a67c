"""GPU parity of the block-quantize kernels, called through the C ABI: bit-exact codes,
scale bytes and per-tensor abs-max against the committed reference fixtures and against the
numpy oracle on seeded inputs, plus full-size structural properties."""
import numpy as np
import pytest
import torch

from conftest import bf16_bits_to_f32
from helpers import (from_bits, mismatch, np_u8, seeded_bf16, swizzle_scales_ref,
                     unswizzle_scales_ref)
from minitransformer_b200 import kernels as K
from oracle import mxfp8, nvfp4

pytestmark = pytest.mark.gpu

MODES = {"1d": ((1, 16), False, False), "1d_rht": ((1, 16), False, True),
         "w16": ((16, 16), False, False), "2d": ((16, 16), True, False)}


def _check_nvfp4(r, o, M, Kd):
    for k in ("data", "scale", "data_t", "scale_t"):
        assert mismatch(np_u8(getattr(r, k)), o[k]) == 0, k
    assert float(r.amax_row.cpu()) == float(o["amax_row"])
    assert float(r.amax_col.cpu()) == float(o["amax_col"])
    # GEMM-ready copies hold the same bytes in the chunk layout
    assert mismatch(unswizzle_scales_ref(np_u8(r.scale_swz), M, Kd // 16), o["scale"][:M]) == 0
    mb = (M + 15) // 16
    assert mismatch(unswizzle_scales_ref(np_u8(r.scale_t_swz), Kd, mb), o["scale_t"][:Kd]) == 0


def test_nvfp4_quantize_matches_reference_fixtures(golden_nvfp4_quantize):
    g = golden_nvfp4_quantize
    n = 0
    for name in sorted({k.split("/")[0] for k in g.files}):
        x = from_bits(g[f"{name}/x"]).cuda()
        M, Kd = x.shape
        for mname, (tile, d2, rht) in MODES.items():
            if f"{name}/{mname}/data" not in g.files:
                continue
            r = K.quantize_nvfp4(x, tile=tile, with_2d=d2, with_rht=rht)
            o = {k: g[f"{name}/{mname}/{k}"] for k in ("data", "scale", "data_t", "scale_t")}
            o["amax_row"], o["amax_col"] = g[f"{name}/{mname}/amax_row"][0], g[f"{name}/{mname}/amax_col"][0]
            _check_nvfp4(r, o, M, Kd)
            n += 1
    assert n >= 40
    assert K.read_device_status() == 0


@pytest.mark.parametrize("shape", [(128, 128), (256, 512), (24, 32), (130, 272), (2, 16), (1024, 4096),
                                   (4096, 1024), (384, 14336)])
@pytest.mark.parametrize("mode", list(MODES))
def test_nvfp4_quantize_matches_oracle(shape, mode):
    tile, d2, rht = MODES[mode]
    if rht and shape[0] % 16:
        pytest.skip("the Hadamard transform needs rows % 16 == 0")
    t, x = seeded_bf16(shape, seed=1234 + shape[0], std=1.0 if mode != "w16" else 0.02)
    o = nvfp4.quantize(x, tile, d2, rht)
    r = K.quantize_nvfp4(t.cuda(), tile=tile, with_2d=d2, with_rht=rht)
    _check_nvfp4(r, o, *shape)
    assert K.read_device_status() == 0


def test_nvfp4_row_only_and_given_amax():
    t, x = seeded_bf16((256, 256), seed=7)
    o = nvfp4.quantize(x, return_transpose=False)
    r = K.quantize_nvfp4(t.cuda(), return_transpose=False)
    assert mismatch(np_u8(r.data), o["data"]) == 0 and mismatch(np_u8(r.scale), o["scale"]) == 0
    assert r.data_t is None
    # a caller-provided (e.g. all-reduced) abs-max larger than the local one changes the scales
    big = torch.tensor([float(o["amax_row"]) * 4], device="cuda")
    r2 = K.quantize_nvfp4(t.cuda(), return_transpose=False, amax_row=big)
    o2q, o2s = nvfp4.quantize_blockwise(x, np.float32(big.item()), False)
    assert mismatch(np_u8(r2.data), o2q) == 0 and mismatch(np_u8(r2.scale), o2s) == 0


def test_nvfp4_runs_are_deterministic():
    t, _ = seeded_bf16((512, 1024), seed=3)
    x = t.cuda()
    a = K.quantize_nvfp4(x, with_rht=True)
    b = K.quantize_nvfp4(x, with_rht=True)
    for k in ("data", "scale", "data_t", "scale_t", "scale_swz", "scale_t_swz"):
        assert torch.equal(getattr(a, k), getattr(b, k)), k


def test_nvfp4_full_size_properties():
    """Configuration-2 activation shape: checked through properties that need no CPU pass
    over the whole tensor: a seeded row slab and a column slab against the oracle, the
    transposed copy against an independent quantization of x^T, codes of -x = codes ^ 8."""
    M, Kd = 8192, 4096
    g = torch.Generator(device="cpu").manual_seed(99)
    t = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    x = t.cuda()
    r = K.quantize_nvfp4(x)
    amax = float(r.amax_row.cpu())
    assert amax == float(t.float().abs().max())
    rows = slice(4096 - 64, 4096 + 64)
    q, s = nvfp4.quantize_blockwise(t[rows].float().numpy(), np.float32(amax), False)
    assert mismatch(np_u8(r.data[rows]), q) == 0 and mismatch(np_u8(r.scale[rows]), s) == 0
    cols = slice(1024, 1024 + 128)
    qt, st = nvfp4.quantize_blockwise(np.ascontiguousarray(t[:, cols].float().numpy().T), np.float32(amax), False)
    assert mismatch(np_u8(r.data_t[cols]), qt) == 0 and mismatch(np_u8(r.scale_t[cols]), st) == 0
    # transposed copy == row-wise quantization of the materialised transpose
    rt = K.quantize_nvfp4(x.t().contiguous(), return_transpose=False, amax_row=r.amax_row)
    assert torch.equal(rt.data, r.data_t) and torch.equal(rt.scale, r.scale_t)
    # sign symmetry: quantizing -x keeps every magnitude code and every scale
    rn = K.quantize_nvfp4(-x, return_transpose=False)
    assert torch.equal(rn.data & 0x77, r.data & 0x77)
    assert torch.equal(rn.scale, r.scale)
    assert K.read_device_status() == 0


def test_nvfp4_rht_full_size_mismatch_rate():
    """Hadamard path at a larger size: the fp32 butterfly may differ from the oracle's exactly
    rounded sum only when a 16-term sum is inexact in fp32; bound the code mismatch rate."""
    t, x = seeded_bf16((2048, 2048), seed=5)
    o = nvfp4.quantize(x, (1, 16), False, True)
    r = K.quantize_nvfp4(t.cuda(), with_rht=True)
    assert mismatch(np_u8(r.data), o["data"]) == 0
    bad = mismatch(np_u8(r.data_t), o["data_t"]) + mismatch(np_u8(r.scale_t), o["scale_t"])
    assert bad <= 1e-6 * x.size, bad


def test_mxfp8_quantize_matches_fixtures(golden_mxfp8_quantize):
    g = golden_mxfp8_quantize
    for name in sorted({k.split("/")[0] for k in g.files}):
        x = from_bits(g[f"{name}/x"]).cuda()
        r = K.quantize_mxfp8(x)
        for k in ("data", "scale", "data_t", "scale_t"):
            assert mismatch(np_u8(getattr(r, k)), g[f"{name}/{k}"]) == 0, f"{name}/{k}"


@pytest.mark.parametrize("shape", [(128, 128), (256, 512), (24, 64), (130, 288), (1, 32), (1024, 4096), (4096, 768)])
@pytest.mark.parametrize("std", [1.0, 0.02, 1e-3])
def test_mxfp8_quantize_matches_oracle(shape, std):
    t, x = seeded_bf16(shape, seed=4321 + shape[1], std=std)
    o = mxfp8.quantize(x)
    r = K.quantize_mxfp8(t.cuda())
    for k in ("data", "scale", "data_t", "scale_t"):
        assert mismatch(np_u8(getattr(r, k)), o[k]) == 0, k
    M, Kd = shape
    assert mismatch(unswizzle_scales_ref(np_u8(r.scale_swz), M, Kd // 32), o["scale"]) == 0
    assert mismatch(unswizzle_scales_ref(np_u8(r.scale_t_swz), Kd, (M + 31) // 32), o["scale_t"]) == 0
    assert K.read_device_status() == 0


def test_mxfp8_edge_values():
    x = torch.zeros(64, 128, dtype=torch.bfloat16)
    x[0, :32] = 448.0          # scale exponent exactly 0
    x[1, :32] = 3.0e38         # near bf16 max
    x[2, :32] = 1e-38          # subnormal-range block
    x[3, 0] = -0.0
    x[4, :32] = torch.linspace(-500, 500, 32)
    o = mxfp8.quantize(x.float().numpy())
    r = K.quantize_mxfp8(x.cuda())
    for k in ("data", "scale", "data_t", "scale_t"):
        assert mismatch(np_u8(getattr(r, k)), o[k]) == 0, k


def test_swizzle_scales_kernel_matches_layout():
    rng = np.random.default_rng(0)
    for rows, kb in [(128, 4), (130, 17), (8192, 256), (5, 1)]:
        s = rng.integers(0, 255, size=(rows, kb), dtype=np.uint8)
        out = K.swizzle_scales(torch.from_numpy(s).cuda())
        assert mismatch(np_u8(out), swizzle_scales_ref(s, rows)) == 0


def test_empty_input_is_a_no_op():
    x = torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda")
    r = K.quantize_nvfp4(x)
    assert r.data.shape == (0, 32) and float(r.amax_row.cpu()) == 0.0
    r = K.quantize_mxfp8(x)
    assert r.data.shape == (0, 64)


def test_nvfp4_stochastic_rounding_is_unbiased_and_brackets_the_exact_value():
    """mt_quantize_nvfp4_sr (parity unpinned: the reference ships this path compiled out): scale
    bytes are those of the nearest-even cast; every code is one of the two E2M1 neighbours of the
    scaled element; averaged over seeds the dequantized value converges to the input (the
    nearest-even cast keeps a bias the average of stochastic casts must not have); one seed gives
    one result."""
    from oracle import formats as F
    M, Kd = 128, 256
    t, x = seeded_bf16((M, Kd), 77, 1e-3)
    xt = t.cuda()
    base = K.quantize_nvfp4(xt, with_rht=False)
    grid = np.sort(np.unique(np.abs(F.E2M1_VALUES)))                    # 0, 0.5, 1, 1.5, 2, 3, 4, 6
    sc = F.e4m3_decode(np_u8(base.scale)[:M])
    amax = float(base.amax_row.cpu())
    ges = np.float32(448.0 * 6.0) / np.float32(amax)
    scale_el = np.repeat(sc, 16, axis=1) / ges                          # decode factor of every element
    scaled = x / scale_el                                               # what the codes approximate, in E2M1 units
    acc = np.zeros_like(x, dtype=np.float64)
    acc_t = np.zeros((Kd, M), dtype=np.float64)
    n_seeds = 48
    clipped = np.minimum(np.abs(scaled), 6.0)
    lo = grid[np.searchsorted(grid, clipped, side="right") - 1]
    hi = grid[np.searchsorted(grid, clipped, side="left")]
    for seed in range(n_seeds):
        r = K.quantize_nvfp4(xt, with_rht=False, amax_row=base.amax_row, amax_col=base.amax_col, sr_seed=1000 + seed)
        assert torch.equal(r.scale, base.scale) and torch.equal(r.scale_t, base.scale_t)
        vals = F.unpack_e2m1(np_u8(r.data))
        mag = np.abs(vals)
        assert np.all((mag == lo) | (mag == hi)), "a code is not a neighbour of the exact value"
        assert np.all((np.sign(vals) == np.sign(scaled)) | (vals == 0))
        acc += vals * scale_el
        acc_t += F.unpack_e2m1(np_u8(r.data_t)).astype(np.float64)
    mean = acc / n_seeds
    rn = F.unpack_e2m1(np_u8(base.data)) * scale_el
    err_sr = np.abs(mean - x).mean()
    err_rn = np.abs(rn - x).mean()
    assert err_sr < 0.45 * err_rn, (err_sr, err_rn)                     # ~1/sqrt(48) of one rounding step
    assert np.abs(acc_t).sum() > 0                                      # the transposed copy is rounded too
    a = K.quantize_nvfp4(xt, with_rht=True, sr_seed=5)
    b = K.quantize_nvfp4(xt, with_rht=True, sr_seed=5)
    c = K.quantize_nvfp4(xt, with_rht=True, sr_seed=6)
    assert torch.equal(a.data, b.data) and torch.equal(a.data_t, b.data_t)
    assert not torch.equal(a.data, c.data) and not torch.equal(a.data_t, c.data_t)
    assert K.read_device_status() == 0


@pytest.mark.parametrize("rht", [True, False])
@pytest.mark.parametrize("shape", [(256, 384), (48, 72 * 8), (1024, 4096)])
def test_amax_pass_also_returns_column_sums(shape, rht):
    """mt_amax_colsum_bf16: the abs-max values are bit-identical to mt_amax_bf16 and the column sums
    equal the fp64 sums to fp32 accumulation accuracy (the bias gradient taken from the pass over dy)."""
    M, Kd = shape
    t, x = seeded_bf16((M, Kd), 7, 1e-3)
    xt = t.cuda()
    a0, c0 = K.amax_bf16(xt, with_rht=rht)
    col = torch.full((Kd,), 7.0, dtype=torch.float32, device="cuda")      # stale contents must be overwritten
    a1, c1 = K.amax_bf16(xt, with_rht=rht, col_sum=col)
    assert float(a0) == float(a1) and float(c0) == float(c1)
    want = x.astype(np.float64).sum(0)
    got = col.cpu().numpy().astype(np.float64)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(x).sum(0).max() + 1e-12
    assert K.read_device_status() == 0
