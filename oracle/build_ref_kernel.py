"""Builds the reference's own NVFP4 quantize extension (its only native kernel) from the sources
where they lie in a reference checkout, for head-to-head checks on the GPU:

    python oracle/build_ref_kernel.py /path/to/reference      # -> oracle/_ref/fp4_gemm.so

Test infrastructure only: nothing in the product imports the result. The reference's build
system is not used; two files are compiled directly (the pybind module and the kernel), for
sm_100a only. No reference source is copied: the compiler reads the files in place and only the
built module lands under oracle/_ref/ (git-ignored).
"""
import os
import subprocess
import sys
import sysconfig


def main(ref_root: str) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    here = os.path.dirname(os.path.abspath(__file__))
    out_dir = os.path.join(here, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    csrc = os.path.join(ref_root, "miniTransformer", "csrc")
    srcs = [os.path.join(csrc, "torch_bindings.cpp"),
            os.path.join(csrc, "ops", "fp4", "quantization", "quantize_transpose_nvfp4.cu")]
    incs = [csrc, sysconfig.get_paths()["include"], *ce.include_paths()]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    inc_flags = [f"-I{i}" for i in incs] + [f"-I{os.path.join(cuda_home, 'include')}"]
    defs = ["-DTORCH_EXTENSION_NAME=fp4_gemm", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    objs = []
    for src in srcs:
        obj = os.path.join(out_dir, os.path.basename(src) + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, "-c", src, "-o", obj, "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                   "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                   "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
                   "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
                   "--expt-relaxed-constexpr", "--expt-extended-lambda", "-diag-suppress=3189",
                   "-gencode", "arch=compute_100a,code=sm_100a", *defs, *inc_flags]
        else:
            cmd = ["g++", "-c", src, "-o", obj, "-O2", "-std=c++17", "-fPIC", *defs, *inc_flags]
        print(" ".join(cmd[:6]), "...", flush=True)
        subprocess.run(cmd, check=True)
        objs.append(obj)
    lib_dirs = ce.library_paths(device_type="cuda") if hasattr(ce, "library_paths") else []
    out = os.path.join(out_dir, "fp4_gemm.so")
    link = ["g++", "-shared", "-o", out, *objs, *[f"-L{d}" for d in lib_dirs],
            *[f"-Wl,-rpath,{d}" for d in lib_dirs], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", "-lcudart", "-lcuda"]
    subprocess.run(link, check=True)
    for o in objs:
        os.remove(o)
    return out


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/build_ref_kernel.py /path/to/reference")
    print(main(sys.argv[1]))
