"""Small, self-contained kernel workloads for `ncu` captures (one kernel family each, a few
launches, a few hundred MB on the device):

    python -m minitransformer_b200.profile_cases gemm        # NVFP4 pair GEMM 4096x9472x4096 (8 full waves), 3 launches
    python -m minitransformer_b200.profile_cases gemm_mxfp8  # MXFP8 pair GEMM, same shape
    python -m minitransformer_b200.profile_cases quant       # abs-max + NVFP4 cast/transpose (RHT) of 8192x14336
    python -m minitransformer_b200.profile_cases quant_mxfp8 # MXFP8 cast/transpose of 8192x14336
    python -m minitransformer_b200.profile_cases grouped     # MXFP8 GroupedLinear fc1+fc2 fwd+bwd, 128 experts, 2 steps

The quantize inputs (224 MiB) exceed the 126 MB L2, so their DRAM counters are meaningful.
"""
import sys

import torch

from . import kernels as K


def main(what: str) -> None:
    dev = "cuda"
    torch.manual_seed(0)
    if what in ("gemm", "gemm_mxfp8"):
        M, N, Kd = 4096, 9472, 4096   # 16 x 37 pair tiles = 8 x 74: no partial last wave
        x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, Kd, device=dev) * 0.02).to(torch.bfloat16)
        if what == "gemm":
            a, b = K.quantize_nvfp4(x, return_transpose=False), K.quantize_nvfp4(w, return_transpose=False)
            for _ in range(3):
                K.gemm_nvfp4(a.data, a.scale_swz, a.amax_row, b.data, b.scale_swz, b.amax_row)
        else:
            a, b = K.quantize_mxfp8(x, return_transpose=False), K.quantize_mxfp8(w, return_transpose=False)
            for _ in range(3):
                K.gemm_mxfp8(a.data, a.scale_swz, b.data, b.scale_swz)
    elif what == "quant":
        x = (torch.randn(8192, 14336, device=dev) * 1e-3).to(torch.bfloat16)
        for _ in range(3):
            K.quantize_nvfp4(x, with_rht=True)
    elif what == "quant_mxfp8":
        x = torch.randn(8192, 14336, device=dev).to(torch.bfloat16)
        for _ in range(3):
            K.quantize_mxfp8(x)
    elif what == "grouped":
        # GroupedLinear fc1 + fc2 forward+backward: 128 experts, 131072 rows, Zipf(1.1) group sizes
        import numpy as np
        from .module import config as mt_config
        from .module.group_linear import GroupedLinear
        params = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
        G, R, H, Fd = 128, 131072, 2048, 768
        rng = np.random.default_rng(1234)
        p = 1.0 / np.arange(1, G + 1) ** 1.1
        m_splits = np.bincount(rng.choice(G, size=R, p=p / p.sum()), minlength=G).tolist()
        kw = dict(bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                  fuse_wgrad_accumulation=True, init_method=lambda t: torch.nn.init.normal_(t, std=0.02))
        fc1, fc2 = GroupedLinear(G, H, Fd, **kw), GroupedLinear(G, Fd, H, **kw)
        for m in (fc1, fc2):
            block = torch.zeros(G, m.out_features, m.in_features, dtype=torch.float32, device=dev)
            for i in range(G):
                getattr(m, f"weight{i}").main_grad = block[i]
        x = torch.randn(R, H, device=dev).to(torch.bfloat16)
        dy = (torch.randn(R, H, device=dev) * 1e-3).to(torch.bfloat16)
        for _ in range(2):
            xd = x.detach().requires_grad_(True)
            fc2(fc1(xd, m_splits, is_first_microbatch=True), m_splits, is_first_microbatch=True).backward(dy)
    else:
        raise SystemExit(f"unknown case {what!r}")
    torch.cuda.synchronize()
    print("done, device status", K.read_device_status())


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm")
