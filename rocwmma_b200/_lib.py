"""ctypes binding of the C ABI declared in include/rocwmma_b200.h.

The shared library is built in-tree (rocwmma_b200/lib/libb200wmma.so) by
`python -m rocwmma_b200.build`.  There is no fallback of any kind: if the
library is missing, loading raises; if no CUDA device is present, the compute
entry points return B200WMMA_ERR_CUDA and the wrappers in api.py raise.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200wmma.so")
TEST_LIB_PATH = os.path.join(_HERE, "lib", "libb200wmma_test.so")

# dtype / layout / status codes (enum b200wmma_dtype etc.)
F16, BF16, E4M3, I8, F32, XF32, F64, I32, E5M2 = range(9)
ROW_MAJOR, COL_MAJOR = 0, 1
OK = 0
ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_DEVICE_WAIT, ERR_TOO_LARGE = (
    -1, -2, -3, -4, -5, -6)

_u32, _i, _d, _p = C.c_uint32, C.c_int, C.c_double, C.c_void_p

# name -> (restype, argtypes); every symbol include/rocwmma_b200.h declares
SIGNATURES = {
    "b200wmma_version": (_i, []),
    "b200wmma_status_string": (C.c_char_p, [_i]),
    "b200wmma_gemm_simple": (_i, [_i, _i, _u32, _u32, _u32, _p, _p, _p, _p, _u32, _u32, _u32, _u32,
                                  _d, _d, _i, _i, _i, _i, _p]),
    "b200wmma_gemm_simple_ex": (_i, [_i, _i, _i, _u32, _u32, _u32, _p, _p, _p, _p, _u32, _u32, _u32,
                                     _u32, _d, _d, _i, _i, _i, _i, _i, _p]),
    "b200wmma_gemm": (_i, [_i, _i, _u32, _u32, _u32, _p, _p, _p, _p, _u32, _u32, _u32, _u32,
                           _d, _d, _i, _i, _p]),
    "b200wmma_gemm_host": (_i, [_i, _i, _u32, _u32, _u32, _p, _p, _p, _p, _u32, _u32, _u32, _u32,
                                _d, _d, _i, _i, _p]),
    "b200wmma_gemm_noalloc": (_i, [_i, _i, _u32, _u32, _u32, _p, _p, _p, _p, _u32, _u32, _u32, _u32,
                                   _d, _d, _i, _i, _p]),
    "b200wmma_gemv": (_i, [_i, _u32, _u32, _p, _p, _p, _p, _d, _d, _u32, _p]),
    "b200wmma_dlrm_fwd": (_i, [_i, _p, _p, _u32, _u32, _u32, _p]),
    "b200wmma_dlrm_bwd": (_i, [_i, _p, _p, _p, _p, _u32, _u32, _u32, _p]),
    "b200wmma_check_device": (_i, [_p, C.POINTER(_u32)]),
    "b200wmma_shutdown": (_i, []),
}

_lib = None


class B200WmmaError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().b200wmma_status_string(status).decode()
        super().__init__(f"{where}: {msg} (status {status})")


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m rocwmma_b200.build` "
                "(there is no fallback implementation)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # raises AttributeError when a declared symbol is absent
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        raise B200WmmaError(status, where)
