"""Quantized Linear forward / dgrad / wgrad composed from the quantize and GEMM oracles.

TEST INFRASTRUCTURE ONLY: CPU checker; never imported by the shipped package.

Follows _QuantizedLinear.forward / .backward
(miniTransformer/module/linear.py:192-330, 332-461) for the single-rank case:
  y  = qgemm(q(x),      q(w))          x [M, K], w [N, K]
  dx = qgemm(q(dy),     q(w)^T copy)   contraction over N
  dw = qgemm(q(dy)^T copy, q(x)^T copy) contraction over M, fp32 output
with the recipe of miniTransformer/module/config.py:118-176: x and dy use 1x16 blocks
(Hadamard transform on their transposed copies when with_rht), w uses the (16,16) tile
without 2-D scaling.
"""
import numpy as np

from . import nvfp4, mxfp8, gemm


def nvfp4_linear_fwd_bwd(x, w, dy, with_rht=True, fused=False):
    """x [M,K], w [N,K], dy [M,N] float32 arrays holding bf16 values.
    Returns dict(y bf16-rounded, dx bf16-rounded, dw fp32)."""
    qx = nvfp4.quantize(x, (1, 16), False, with_rht)
    qw = nvfp4.quantize(w, (16, 16), False, False)
    qg = nvfp4.quantize(dy, (1, 16), False, with_rht)
    N, M = w.shape[0], x.shape[0]
    y = gemm.qgemm_nvfp4(qx["data"], qx["scale"], qx["amax_row"],
                         qw["data"], qw["scale"], qw["amax_row"], fused=fused)
    dx = gemm.qgemm_nvfp4(qg["data"], qg["scale"], qg["amax_row"],
                          qw["data_t"], qw["scale_t"], qw["amax_col"], fused=fused)
    dw = gemm.qgemm_nvfp4(qg["data_t"], qg["scale_t"], qg["amax_col"],
                          qx["data_t"], qx["scale_t"], qx["amax_col"], out_bf16=False, fused=fused)
    return {"y": y, "dx": dx, "dw": dw, "qx": qx, "qw": qw, "qg": qg}


def mxfp8_linear_fwd_bwd(x, w, dy, fused=False):
    qx = mxfp8.quantize(x)
    qw = mxfp8.quantize(w)
    qg = mxfp8.quantize(dy)
    y = gemm.qgemm_mxfp8(qx["data"], qx["scale"], qw["data"], qw["scale"], fused=fused)
    dx = gemm.qgemm_mxfp8(qg["data"], qg["scale"], qw["data_t"], qw["scale_t"], fused=fused)
    dw = gemm.qgemm_mxfp8(qg["data_t"], qg["scale_t"], qx["data_t"], qx["scale_t"],
                          out_bf16=False, fused=fused)
    return {"y": y, "dx": dx, "dw": dw, "qx": qx, "qw": qw, "qg": qg}


def mxfp8_grouped_fwd_bwd(x, ws, dy, m_splits, fused=True):
    """Grouped (per-expert) linear: rows of x / dy are split by m_splits, expert g uses
    ws[g] [N, K]. The wgrad of expert g contracts over that expert's rows zero-padded to a
    multiple of 32. API shape from miniTransformer/module/group_linear.py:44-264 (the
    arithmetic there is not runnable; parity unpinned)."""
    ys, dxs, dws = [], [], []
    off = 0
    for g, m in enumerate(m_splits):
        xs, gs = x[off:off + m], dy[off:off + m]
        off += m
        N, K = ws[g].shape
        if m == 0:
            ys.append(np.zeros((0, N), np.float32))
            dxs.append(np.zeros((0, K), np.float32))
            dws.append(np.zeros((N, K), np.float32))
            continue
        r = mxfp8_linear_fwd_bwd(xs, ws[g], gs, fused=fused)
        ys.append(r["y"]); dxs.append(r["dx"]); dws.append(r["dw"])
    return {"y": np.concatenate(ys), "dx": np.concatenate(dxs), "dw": dws}
