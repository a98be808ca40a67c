"""Small, self-contained kernel workloads for `ncu` captures (one kernel family each, a few
launches, a few hundred MB on the device):

    python -m minitransformer_b200.profile_cases gemm        # NVFP4 pair GEMM 4096x9472x4096 (8 full waves), 3 launches
    python -m minitransformer_b200.profile_cases gemm_mxfp8  # MXFP8 pair GEMM, same shape
    python -m minitransformer_b200.profile_cases quant       # abs-max + NVFP4 cast/transpose (RHT) of 8192x14336
    python -m minitransformer_b200.profile_cases quant_mxfp8 # MXFP8 cast/transpose of 8192x14336

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
    else:
        raise SystemExit(f"unknown case {what!r}")
    torch.cuda.synchronize()
    print("done, device status", K.read_device_status())


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm")
