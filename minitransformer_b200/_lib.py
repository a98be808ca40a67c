"""ctypes binding of libmt_b200.so, the C-ABI library of sm_100a kernels.

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmt_b200.so")
INCLUDE_DIR = os.path.join(os.path.dirname(_HERE), "include")
HEADER_PATHS = (os.path.join(INCLUDE_DIR, "mt_b200.h"), os.path.join(INCLUDE_DIR, "mt_b200_test.h"))

MT_BF16, MT_F32 = 0, 1
MT_Q_2D, MT_Q_RHT, MT_Q_ROWPAD16, MT_Q_AMAX_ZEROED = 1, 2, 4, 8
MT_MAX_PEERS, MT_PEER_CTRL_BYTES, MT_IPC_HANDLE_BYTES = 8, 4096, 64

_c = ctypes
_vp, _i64, _int = _c.c_void_p, _c.c_int64, _c.c_int


class GemmOpts(ctypes.Structure):
    """mt_gemm_opts of include/mt_b200.h."""
    _fields_ = [("sm_margin", _int), ("d_amax", _vp), ("n_dest", _int), ("my_rank", _int), ("dest", _vp * 8),
                ("dest_rows", _i64)]


_opts = _c.POINTER(GemmOpts)

_SIGNATURES = {
    "mt_version": (_int, []),
    "mt_set_launch_overlap": (_int, [_int]),
    "mt_last_error_string": (_c.c_char_p, []),
    "mt_swizzled_scale_bytes": (_i64, [_i64, _i64]),
    "mt_amax_bf16": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "mt_amax_colsum_bf16": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "mt_quantize_nvfp4": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp]),
    "mt_quantize_nvfp4_sr": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _c.c_uint64,
                                    _vp]),
    "mt_quantize_mxfp8": (_int, [_vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp]),
    "mt_swizzle_scales": (_int, [_vp, _i64, _i64, _i64, _vp, _vp]),
    "mt_gemm_nvfp4": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _i64, _vp, _int, _int, _opts, _vp]),
    "mt_gemm_mxfp8": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _i64, _vp, _int, _int, _opts, _vp]),
    "mt_gemm_nvfp4_kslab": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _int, _i64, _vp, _int,
                                   _int, _opts, _vp]),
    "mt_gemm_mxfp8_kslab": (_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _int, _i64, _vp, _int, _int,
                                   _opts, _vp]),
    "mt_test_bounded_wait": (_int, [_i64, _vp]),
    "mt_gemm_nvfp4_check": (_int, [_vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _vp, _int, _i64, _int, _vp]),
    "mt_gemm_mxfp8_check": (_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _int, _i64, _int, _vp]),
    "mt_grouped_plan_bytes": (_i64, [_i64, _i64]),
    "mt_grouped_plan_build": (_int, [_vp, _i64, _i64, _vp, _i64, _vp]),
    "mt_grouped_quantize_mxfp8": (_int, [_vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp]),
    "mt_grouped_transpose_quantize_mxfp8": (_int, [_vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp]),
    "mt_grouped_gemm_mxfp8": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                     _vp, _int, _i64, _vp]),
    "mt_grouped_gemm_mxfp8_static": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                            _vp, _int, _i64, _vp]),
    "mt_grouped_wgrad_mxfp8": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _int, _int, _vp]),
    "mt_ipc_export": (_int, [_vp, _vp, _c.POINTER(_i64)]),
    "mt_ipc_import": (_int, [_vp, _i64, _c.POINTER(_vp)]),
    "mt_ipc_close": (_int, [_vp, _i64]),
    "mt_peer_barrier": (_int, [_c.POINTER(_vp), _int, _int, _int, _vp]),
    "mt_peer_allreduce_max": (_int, [_c.POINTER(_vp), _int, _int, _int, _vp, _int, _vp]),
    "mt_peer_gather": (_int, [_c.POINTER(_vp), _int, _int, _c.POINTER(_i64), _c.POINTER(_vp), _c.POINTER(_i64), _int, _int,
                              _int, _vp]),
    "mt_peer_reduce_bf16": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _vp]),
    "mt_read_device_status": (_int, [_c.POINTER(_int), _vp]),
}

_lib = None


class MtError(RuntimeError):
    """A C-ABI call returned a negative status."""


def declared_symbols(header_paths=HEADER_PATHS):
    """Names of every function the headers under include/ declare."""
    names = set()
    for path in header_paths:
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names.update(re.findall(r"\b(mt_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def load():
    """Loads the shared library (once) and sets the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MtError(
            f"{LIB_PATH} is missing: build it with `python -m minitransformer_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = load().mt_last_error_string().decode(errors="replace")
        raise MtError(f"{what or 'libmt_b200'} failed with status {status}: {msg}")


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args), name)
