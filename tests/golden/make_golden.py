"""Regenerates the fixtures in this directory from the reference's own PyTorch emulation.

Run in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports Nvfp4TiledQuantizeRefOp and _QuantizedLinear from the reference (a stub module
named fp4_gemm satisfies their unused import), runs them on CPU on small seeded inputs
and stores inputs (bf16 bit patterns) and outputs as compressed .npz files. The MXFP8
fixture evaluates the reference's cast_to_e8 helper and clamp-then-cast idiom with
PyTorch, since the reference has no MXFP8 quantizer of its own.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.modules["fp4_gemm"] = types.ModuleType("fp4_gemm")
    from miniTransformer.ops.nvfp4_quantize_op_ref import Nvfp4TiledQuantizeRefOp, cast_to_e8
    from miniTransformer.ops.quantization import QParams, MMParams, QuantizeResultCache
    from miniTransformer.module.linear import _QuantizedLinear
    from miniTransformer.module.config import get_qlinear_params_from_predefined, QuantizeRecipe

    op = Nvfp4TiledQuantizeRefOp()

    def qparams(tile, d2, rht):
        return QParams(output_dtype=torch.uint8, scaling_dtype=torch.float8_e4m3fn,
                       quant_tile_shape=tile, with_2d_quantization=d2, with_rht=rht)

    def quant(x, tile, d2, rht):
        r = op.quantize(x, qparams(tile, d2, rht), return_transpose=True)
        return dict(data=r.data.numpy(), scale=r.scale.view(torch.uint8).numpy(),
                    data_t=r.data_t.numpy(), scale_t=r.scale_t.view(torch.uint8).numpy(),
                    amax_row=r.global_amax_row.numpy(), amax_col=r.global_amax_col.numpy())

    g = torch.Generator().manual_seed(1234)
    inputs = {}
    inputs["randn_64x128"] = torch.randn(64, 128, generator=g).to(torch.bfloat16)
    inputs["randn_128x256"] = torch.randn(128, 256, generator=g).to(torch.bfloat16)
    inputs["small_48x64"] = (torch.randn(48, 64, generator=g) * 0.02).to(torch.bfloat16)
    inputs["ragged_24x32"] = torch.randn(24, 32, generator=g).to(torch.bfloat16)
    inputs["zeros_32x64"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    x = torch.randn(32, 64, generator=g).to(torch.bfloat16); x[0, 0] = 3.3e38
    inputs["huge_32x64"] = x
    inputs["tiny_32x64"] = (torch.randn(32, 64, generator=g) * 1e-30).to(torch.bfloat16)
    x = torch.randn(32, 64, generator=g).to(torch.bfloat16)
    x[:, :16] *= 1e-20; x[3, 5] = -0.0; x[4, :16] = 0
    inputs["mixed_32x64"] = x
    x = torch.randn(32, 64, generator=g).to(torch.bfloat16); x[0, 0] = float("inf")
    inputs["inf_32x64"] = x
    inputs["ties_16x32"] = torch.tensor(
        [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5,
         -5.0, -6.0]).repeat(16, 2).to(torch.bfloat16)
    inputs["widerange_64x64"] = (torch.randn(64, 64, generator=g)
                                 * torch.exp(torch.randn(64, 64, generator=g) * 8)).to(torch.bfloat16)

    modes = {"1d": ((1, 16), False, False), "1d_rht": ((1, 16), False, True),
             "w16": ((16, 16), False, False), "2d": ((16, 16), True, False)}
    out = {}
    for name, x in inputs.items():
        out[f"{name}/x"] = bits(x)
        for mname, (tile, d2, rht) in modes.items():
            if rht and x.shape[0] % 16:
                continue
            for k, v in quant(x, tile, d2, rht).items():
                out[f"{name}/{mname}/{k}"] = v
    np.savez_compressed(os.path.join(HERE, "nvfp4_quantize.npz"), **out)

    # GEMM on quantized operands + Linear fwd/bwd through _QuantizedLinear.
    out = {}
    params = get_qlinear_params_from_predefined(QuantizeRecipe.FP4_SUB_CHANNEL_REF)
    for tag, (M, K, N) in {"a": (32, 64, 48), "b": (64, 128, 32)}.items():
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
        dy = (torch.randn(M, N, generator=g) * 1e-3).to(torch.bfloat16)
        out[f"{tag}/x"], out[f"{tag}/w"], out[f"{tag}/dy"] = bits(x), bits(w), bits(dy)
        rx = op.quantize(x, params.x_params, return_transpose=True)
        rw = op.quantize(w, params.w_params, return_transpose=True)
        y = op.qgemm(rx.data, rw.data, MMParams(), torch.bfloat16, rx.scale, rw.scale[:N],
                     global_amax_qx=rx.global_amax_row, global_amax_qw=rw.global_amax_row,
                     qparams_x=params.x_params, qparams_w=params.w_params)
        out[f"{tag}/gemm_y"] = bits(y)
        acc = torch.randn(M, N, generator=g)
        y2 = op.qgemm(rx.data, rw.data, MMParams(), torch.float32, rx.scale, rw.scale[:N],
                      out=acc, accumulate=True,
                      global_amax_qx=rx.global_amax_row, global_amax_qw=rw.global_amax_row,
                      qparams_x=params.x_params, qparams_w=params.w_params)
        out[f"{tag}/acc_in"], out[f"{tag}/acc_out"] = acc.numpy(), y2.numpy()
        xg = x.clone().requires_grad_(True)
        wg = w.clone().requires_grad_(True)
        yy = _QuantizedLinear.apply(xg, None, wg, QuantizeResultCache(), None, False, None, 1,
                                    None, params, torch.bfloat16, True, None, False)
        yy.backward(dy)
        out[f"{tag}/lin_y"] = bits(yy.detach())
        out[f"{tag}/lin_dx"] = bits(xg.grad)
        out[f"{tag}/lin_dw"] = wg.grad.float().numpy()
    np.savez_compressed(os.path.join(HERE, "nvfp4_linear.npz"), **out)

    # MXFP8 pieces.
    def torch_mx(x):
        m, n = x.shape
        xb = x.view(m, n // 32, 32)
        amax = torch.amax(torch.abs(xb), dim=-1, keepdim=True).to(torch.float32)
        dec = cast_to_e8(torch.div(amax, torch.tensor(448.0)))
        enc = torch.div(torch.tensor(1.0), dec)
        q = torch.clamp(xb.float() * enc, -448.0, 448.0).reshape(m, n).to(torch.float8_e4m3fn)
        sb = (torch.log2(dec).squeeze(-1) + 127).to(torch.uint8)
        return q.view(torch.uint8).numpy(), sb.numpy()

    out = {}
    mx_inputs = {
        "randn_64x256": torch.randn(64, 256, generator=g).to(torch.bfloat16),
        "small_64x128": (torch.randn(64, 128, generator=g) * 0.02).to(torch.bfloat16),
        "wide_64x128": (torch.randn(64, 128, generator=g)
                        * torch.exp(torch.randn(64, 128, generator=g) * 20)).to(torch.bfloat16),
        "zeros_32x64": torch.zeros(32, 64, dtype=torch.bfloat16),
        "pow2_32x64": torch.full((32, 64), 448.0).to(torch.bfloat16),
    }
    for name, x in mx_inputs.items():
        out[f"{name}/x"] = bits(x)
        out[f"{name}/data"], out[f"{name}/scale"] = torch_mx(x)
        out[f"{name}/data_t"], out[f"{name}/scale_t"] = torch_mx(x.t().contiguous())
    np.savez_compressed(os.path.join(HERE, "mxfp8_quantize.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
