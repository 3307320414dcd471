"""CPU oracle bindings (ctypes) -- TEST INFRASTRUCTURE ONLY.

`liboracle.so` is this repository's restatement of rocWMMA's CPU reference
(GEMM, DLRM forward/backward, GEMV, error metric; see oracle.cpp for the
reference file:line each function follows).  `_ref/libref.so` is the
reference's own host code compiled from the mounted reference tree, when it
was available at build time.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# dtype codes shared with the C ABI of the CUDA library
F16, BF16, E4M3, I8, F32, XF32, F64, I32, E5M2 = range(9)
ROW, COL = 0, 1

_NP = {F16: np.float16, BF16: np.uint16, E4M3: np.uint8, I8: np.int8,
       F32: np.float32, XF32: np.float32, F64: np.float64, I32: np.int32, E5M2: np.uint8}


def np_dtype(code: int):
    return _NP[code]


def reference_dir() -> str:
    """Where the rocWMMA source tree is mounted (it need not exist).  The environment
    variable ROCWMMA_REFERENCE_DIR overrides the default location; the Makefile beside this
    file receives it as REF."""
    return os.environ.get("ROCWMMA_REFERENCE_DIR", "/root/reference")


def _have_reference() -> bool:
    return os.path.isdir(reference_dir())


def build(force: bool = False) -> None:
    """Compile liboracle.so (and _ref/libref.so where the reference tree is mounted)."""
    if force or not os.path.exists(os.path.join(_HERE, "liboracle.so")):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    if _have_reference() and (
            force or not os.path.exists(os.path.join(_HERE, "_ref", "libref.so"))):
        subprocess.run(["make", "-C", _HERE, "ref", "REF=" + reference_dir()], check=True,
                       stdout=subprocess.DEVNULL)
    if _have_reference() and (force or _ref_kernels_stale()):
        subprocess.run(["make", "-C", _HERE, "refkernels", "REF=" + reference_dir()],
                       check=True, stdout=subprocess.DEVNULL)


def _ref_kernels_stale() -> bool:
    """The reference's sample kernels are compiled against this repository's headers, so the
    library is stale when it is older than any of them (or than its own shim)."""
    target = os.path.join(_HERE, "_ref", "libref_kernels.so")
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = [os.path.join(_HERE, "ref_kernels.cu"), os.path.join(_HERE, "Makefile")]
    inc = os.path.join(os.path.dirname(_HERE), "include", "rocwmma")
    for root, _, files in os.walk(inc):
        deps += [os.path.join(root, f) for f in files]
    return any(os.path.getmtime(d) > t for d in deps)


_lib = None
_ref = None
_ref_kernels = None


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(os.path.join(_HERE, "liboracle.so"))
        L.oracle_gemm_ex.restype = C.c_int
        L.oracle_gemm_ex.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_uint32,
                                     C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                     C.c_double, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_dlrm_fwd.restype = C.c_int
        L.oracle_dlrm_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                      C.c_uint32]
        L.oracle_dlrm_bwd.restype = C.c_int
        L.oracle_dlrm_bwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_uint32, C.c_uint32, C.c_uint32]
        L.oracle_gemv.restype = C.c_int
        L.oracle_gemv.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_void_p, C.c_double, C.c_double, C.c_uint32]
        L.oracle_max_rel_err.restype = C.c_double
        L.oracle_max_rel_err.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint64]
        for name in ("oracle_encode_e5m2", "oracle_decode_e5m2"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        for name in ("oracle_encode_e4m3", "oracle_decode_e4m3", "oracle_encode_bf16",
                     "oracle_decode_bf16"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_num_threads.restype = None
        L.oracle_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def ref():
    """The reference's own compiled host code, or None when it was not built."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref.so")
        if not os.path.exists(path):
            if _have_reference():
                build()
            if not os.path.exists(path):
                return None
        L = C.CDLL(path)
        L.ref_gemm_ex.restype = C.c_int
        L.ref_gemm_ex.argtypes = [C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32,
                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_double,
                                  C.c_double, C.c_int, C.c_int]
        L.ref_dlrm_fwd.restype = C.c_int
        L.ref_dlrm_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                   C.c_uint32]
        L.ref_dlrm_bwd.restype = C.c_int
        L.ref_dlrm_bwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_uint32, C.c_uint32, C.c_uint32]
        L.ref_sgemv.restype = C.c_int
        L.ref_sgemv.argtypes = [C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_float, C.c_float]
        _ref = L
    return _ref


def ref_kernels():
    """The reference's own sample kernels compiled against this repository's headers
    (oracle/ref_kernels.cu), or None when the library was not built."""
    global _ref_kernels
    if _ref_kernels is None:
        path = os.path.join(_HERE, "_ref", "libref_kernels.so")
        if _have_reference():
            build()
        if not os.path.exists(path):
            return None
        L = C.CDLL(path)
        gemm = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_double, C.c_double, C.c_void_p]
        for name in ("refk_perf_hgemm", "refk_perf_sgemm", "refk_perf_dgemm", "refk_simple_hgemm",
                     "refk_simple_sgemm", "refk_simple_dgemm"):
            getattr(L, name).restype = C.c_int
            getattr(L, name).argtypes = gemm
        for name in ("refk_perf_hgemm_tile", "refk_perf_sgemm_tile", "refk_perf_dgemm_tile"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [C.POINTER(C.c_uint32)]
        for name in ("refk_simple_sgemv", "refk_simple_dgemv"):
            getattr(L, name).restype = C.c_int
            getattr(L, name).argtypes = [C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_double, C.c_double, C.c_void_p]
        L.refk_dlrm_fwd.restype = C.c_int
        L.refk_dlrm_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                    C.c_uint32, C.c_void_p]
        L.refk_dlrm_bwd.restype = C.c_int
        L.refk_dlrm_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]
        _ref_kernels = L
    return _ref_kernels


def num_threads() -> int:
    return lib().oracle_num_threads()


def host_cores() -> int:
    """Host cores this process may run on."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def set_num_threads(n: int) -> int:
    """OpenMP threads for the CPU routines of this module (restatement and reference build)
    from now on; returns the count in effect.  Needed where a launcher exported
    OMP_NUM_THREADS=1 (torch.distributed.run does): the CPU baseline states its core count
    and must really use it."""
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def _check(a, code, name):
    assert a.dtype == _NP[code], f"{name}: expected {_NP[code]}, got {a.dtype}"
    assert a.flags["C_CONTIGUOUS"], f"{name} must be contiguous"


def gemm(in_t, out_t, m, n, k, a, b, c, alpha, beta, layout_a=ROW, layout_b=COL,
         layout_c=ROW, layout_d=ROW, lda=None, ldb=None, ldc=None, ldd=None, literal=False,
         comp_t=None):
    """D = alpha*A*B + beta*C.  Arrays are flat storage in the stated layouts;
    leading dimensions default to the natural ones (test/reference_impl.hpp:53-56).
    comp_t: the compute type (rocWMMA's Tc); None = the usual one for the input type."""
    lda = lda or (k if layout_a == ROW else m)
    ldb = ldb or (n if layout_b == ROW else k)
    ldc = ldc or (n if layout_c == ROW else m)
    ldd = ldd or (n if layout_d == ROW else m)
    _check(a, in_t, "a"), _check(b, in_t, "b"), _check(c, out_t, "c")
    d = np.empty(m * ldd if layout_d == ROW else n * ldd, dtype=_NP[out_t])
    rc = lib().oracle_gemm_ex(in_t, out_t, -1 if comp_t is None else comp_t, int(literal), m, n,
                              k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc, ldd,
                              float(alpha), float(beta), layout_a, layout_b, layout_c, layout_d)
    if rc != 0:
        raise ValueError(f"oracle_gemm: unsupported type triple ({in_t},{out_t},{comp_t})")
    return d


def ref_gemm(in_t, out_t, m, n, k, a, b, c, alpha, beta, layout_a=ROW, layout_b=COL,
             comp_t=None):
    """The reference's gemm_CPU (natural leading dimensions, C/D row-major)."""
    R = ref()
    assert R is not None, "oracle/_ref/libref.so was not built"
    d = np.empty(m * n, dtype=_NP[out_t])
    rc = R.ref_gemm_ex(in_t, out_t, -1 if comp_t is None else comp_t, m, n, k, _ptr(a), _ptr(b),
                       _ptr(c), _ptr(d), float(alpha), float(beta), layout_a, layout_b)
    if rc != 0:
        raise ValueError("ref_gemm: unsupported type triple")
    return d


def dlrm_fwd(dt, x, m, k, batch, use_ref=False):
    out = np.empty(batch * (k + m * (m - 1) // 2), dtype=_NP[dt])
    fn = ref().ref_dlrm_fwd if use_ref else lib().oracle_dlrm_fwd
    assert fn(dt, _ptr(x), _ptr(out), m, k, batch) == 0
    return out


def dlrm_bwd(dt, x, up, m, k, batch, use_ref=False):
    mlp = np.empty(batch * k, dtype=_NP[dt])
    grad = np.empty(batch * m * k, dtype=_NP[dt])
    fn = ref().ref_dlrm_bwd if use_ref else lib().oracle_dlrm_bwd
    assert fn(dt, _ptr(x), _ptr(up), _ptr(mlp), _ptr(grad), m, k, batch) == 0
    return mlp, grad


def gemv(dt, m, k, a, x, y, alpha, beta, lda=None):
    out = np.empty(m, dtype=_NP[dt])
    assert lib().oracle_gemv(dt, m, k, _ptr(a), _ptr(x), _ptr(y), _ptr(out), float(alpha),
                             float(beta), lda or m) == 0
    return out


def ref_sgemv(m, k, a, x, y, alpha, beta):
    out = y.copy()
    assert ref().ref_sgemv(m, k, _ptr(a), _ptr(x), _ptr(out), alpha, beta) == 0
    return out


def max_rel_err(dt, a, b) -> float:
    """max |a-b| / (|a|+|b|+1); -1 if an infinity, -2 if a NaN was met
    (samples/common.hpp:345-416)."""
    a = np.ascontiguousarray(a).reshape(-1)
    b = np.ascontiguousarray(b).reshape(-1)
    assert a.size == b.size and a.dtype == _NP[dt] and b.dtype == _NP[dt]
    return float(lib().oracle_max_rel_err(dt, _ptr(a), _ptr(b), a.size))


def encode_e4m3(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_encode_e4m3(_ptr(x), _ptr(out), x.size)
    return out


def decode_e4m3(x):
    x = np.ascontiguousarray(x, dtype=np.uint8)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_decode_e4m3(_ptr(x), _ptr(out), x.size)
    return out


def encode_e5m2(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_encode_e5m2(_ptr(x), _ptr(out), x.size)
    return out


def decode_e5m2(x):
    x = np.ascontiguousarray(x, dtype=np.uint8)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_decode_e5m2(_ptr(x), _ptr(out), x.size)
    return out


def encode_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_encode_bf16(_ptr(x), _ptr(out), x.size)
    return out


def decode_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_decode_bf16(_ptr(x), _ptr(out), x.size)
    return out
