"""The numpy oracle must reproduce, bit for bit, the fixtures generated from the
reference's own PyTorch emulation (tests/golden/make_golden.py)."""
import numpy as np
import pytest

from conftest import bf16_bits_to_f32
from oracle import formats as F, gemm, linear, mxfp8, nvfp4

MODES = {"1d": ((1, 16), False, False), "1d_rht": ((1, 16), False, True),
         "w16": ((16, 16), False, False), "2d": ((16, 16), True, False)}


def _cases(npz):
    return sorted({k.split("/")[0] for k in npz.files})


def test_nvfp4_quantize_matches_reference(golden_nvfp4_quantize):
    g = golden_nvfp4_quantize
    checked = 0
    for name in _cases(g):
        x = bf16_bits_to_f32(g[f"{name}/x"])
        for mname, (tile, d2, rht) in MODES.items():
            if f"{name}/{mname}/data" not in g.files:
                continue
            o = nvfp4.quantize(x, tile, d2, rht)
            for k in ("data", "scale", "data_t", "scale_t"):
                np.testing.assert_array_equal(o[k], g[f"{name}/{mname}/{k}"], err_msg=f"{name}/{mname}/{k}")
            assert np.float32(g[f"{name}/{mname}/amax_row"][0]) == o["amax_row"]
            assert np.float32(g[f"{name}/{mname}/amax_col"][0]) == o["amax_col"]
            checked += 1
    assert checked >= 40


def test_nvfp4_gemm_and_linear_match_reference(golden_nvfp4_linear):
    g = golden_nvfp4_linear
    for tag in ("a", "b"):
        x, w, dy = (bf16_bits_to_f32(g[f"{tag}/{n}"]) for n in ("x", "w", "dy"))
        r = linear.nvfp4_linear_fwd_bwd(x, w, dy, with_rht=True)
        qx, qw = r["qx"], r["qw"]
        y = gemm.qgemm_nvfp4(qx["data"], qx["scale"], qx["amax_row"],
                             qw["data"], qw["scale"], qw["amax_row"])
        np.testing.assert_array_equal(F.f32_to_bf16_bits(y), g[f"{tag}/gemm_y"])
        acc = gemm.qgemm_nvfp4(qx["data"], qx["scale"], qx["amax_row"], qw["data"], qw["scale"],
                               qw["amax_row"], out_bf16=False, out=g[f"{tag}/acc_in"], accumulate=True)
        np.testing.assert_array_equal(acc, g[f"{tag}/acc_out"])
        np.testing.assert_array_equal(F.f32_to_bf16_bits(r["y"]), g[f"{tag}/lin_y"])
        np.testing.assert_array_equal(F.f32_to_bf16_bits(r["dx"]), g[f"{tag}/lin_dx"])
        # autograd hands the fp32 wgrad back in the parameter's dtype (bf16)
        np.testing.assert_array_equal(F.bf16_round(r["dw"]), g[f"{tag}/lin_dw"])
        # the single-sgemm variant only reorders the fp32 sum
        rf = linear.nvfp4_linear_fwd_bwd(x, w, dy, with_rht=True, fused=True)
        for k in ("y", "dx", "dw"):
            assert gemm.rel_frobenius(rf[k], r[k]) < 1e-5


def test_mxfp8_pieces_match_reference_helpers(golden_mxfp8_quantize):
    g = golden_mxfp8_quantize
    for name in _cases(g):
        x = bf16_bits_to_f32(g[f"{name}/x"])
        o = mxfp8.quantize(x)
        for k in ("data", "scale", "data_t", "scale_t"):
            np.testing.assert_array_equal(o[k], g[f"{name}/{k}"], err_msg=f"{name}/{k}")


def test_e4m3_roundtrip_and_ties():
    allb = np.arange(256, dtype=np.uint8)
    v = F.e4m3_decode(allb)
    ok = ~np.isnan(v)
    np.testing.assert_array_equal(F.e4m3_encode(v[ok]), allb[ok])
    # ties go to the even mantissa: 17 -> 16, 19 -> 20, 2^-10 -> 0
    np.testing.assert_array_equal(
        F.e4m3_decode(F.e4m3_encode(np.array([17.0, 19.0, 2.0 ** -10], np.float32))),
        np.array([16.0, 20.0, 0.0], np.float32))


def test_e2m1_edge_semantics():
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, -0.0, -0.1, -0.25, np.nan, 7.0],
                 np.float32)
    np.testing.assert_array_equal(
        F.e2m1_encode(x), np.array([0, 2, 2, 4, 4, 6, 6, 7, 0, 8, 8, 0, 7], np.uint8))


def test_e8m0_rule_spot_values():
    amax = np.array([448.0, 447.0, 896.0, 1.0, 0.0], np.float32)
    np.testing.assert_array_equal(mxfp8.e8m0_exponent(amax), np.array([0, 0, 1, -8, -127]))


def test_mxfp8_gemm_blockwise_vs_fused():
    rng = np.random.default_rng(0)
    x = F.bf16_round(rng.standard_normal((48, 128)).astype(np.float32))
    w = F.bf16_round((rng.standard_normal((40, 128)) * 0.02).astype(np.float32))
    qx, qw = mxfp8.quantize(x), mxfp8.quantize(w)
    a = gemm.qgemm_mxfp8(qx["data"], qx["scale"], qw["data"], qw["scale"], out_bf16=False)
    b = gemm.qgemm_mxfp8(qx["data"], qx["scale"], qw["data"], qw["scale"], out_bf16=False, fused=True)
    assert gemm.rel_frobenius(b, a) < 1e-5
    # quantization noise of E4M3 with 1x32 scales against the unquantized product
    assert gemm.rel_frobenius(a, x @ w.T) < 0.05
