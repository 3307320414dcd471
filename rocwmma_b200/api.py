"""Host-side drivers over the C ABI, operating on torch CUDA tensors.

These mirror what the reference's host programs do around their kernels
(rocWMMA samples/simple_hgemm.cpp:141-290 `gemm_test`, samples/perf_hgemm.cpp:716-944,
samples/simple_sgemv.cpp:157-270, samples/simple_dlrm.cpp:443-700): pick leading
dimensions, launch, hand back the result.  PyTorch is used for device memory
and streams only; every computation happens in this library's own kernels.

Storage conventions: fp16 -> torch.float16, bf16 -> torch.bfloat16,
e4m3 -> torch.uint8 (raw bits) or torch.float8_e4m3fn, i8 -> torch.int8,
f32/xf32 -> torch.float32, f64 -> torch.float64, i32 -> torch.int32.
Matrices are passed as flat (or 2-D contiguous) storage in the stated layout.
"""
from __future__ import annotations

import torch

from . import _lib as L
from ._lib import (BF16, COL_MAJOR, E4M3, E5M2, F16, F32, F64, I8, I32, ROW_MAJOR, XF32,  # noqa: F401
                   B200WmmaError)

_TORCH = {F16: torch.float16, BF16: torch.bfloat16, E4M3: torch.uint8, I8: torch.int8,
          F32: torch.float32, XF32: torch.float32, F64: torch.float64, I32: torch.int32,
          E5M2: torch.uint8}


def torch_dtype(code: int):
    return _TORCH[code]


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("device tensors required (this library has no CPU path)")


def _natural_ld(layout, rows, cols):
    return cols if layout == ROW_MAJOR else rows


def gemm_simple(in_t, out_t, m, n, k, a, b, c, alpha, beta, layout_a=ROW_MAJOR,
                layout_b=COL_MAJOR, layout_cd=ROW_MAJOR, block=16, lda=None, ldb=None, ldc=None,
                ldd=None, out=None, stream=None, compute=None, block_k=0):
    """D = alpha*A*B + beta*C, one fragment tile per warp (the simple_*gemm samples).
    compute: rocWMMA's ComputeT as a dtype code (None = the usual one for the input type);
    block_k: K extent of the fragments (0 = the usual one)."""
    _require_cuda(a, b, c)
    lda = lda or _natural_ld(layout_a, m, k)
    ldb = ldb or _natural_ld(layout_b, k, n)
    ldc = ldc or _natural_ld(layout_cd, m, n)
    ldd = ldd or _natural_ld(layout_cd, m, n)
    d = out if out is not None else torch.empty(
        (m if layout_cd == ROW_MAJOR else n) * ldd, dtype=_TORCH[out_t], device=a.device)
    if compute is None and block_k == 0:
        rc = L.lib().b200wmma_gemm_simple(in_t, out_t, m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d),
                                          lda, ldb, ldc, ldd, float(alpha), float(beta), layout_a,
                                          layout_b, layout_cd, block, _stream(stream))
    else:
        rc = L.lib().b200wmma_gemm_simple_ex(in_t, out_t, -1 if compute is None else compute, m, n,
                                             k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb, ldc,
                                             ldd, float(alpha), float(beta), layout_a, layout_b,
                                             layout_cd, block, block_k, _stream(stream))
    L.check(rc, "b200wmma_gemm_simple")
    return d


def gemm(in_t, out_t, m, n, k, a, b, c, alpha, beta, layout_a=ROW_MAJOR, layout_b=COL_MAJOR,
         lda=None, ldb=None, ldc=None, ldd=None, out=None, stream=None):
    """D = alpha*A*B + beta*C through the block-cooperative tensor-core path; C/D row-major."""
    _require_cuda(a, b, c)
    lda = lda or _natural_ld(layout_a, m, k)
    ldb = ldb or _natural_ld(layout_b, k, n)
    ldc = ldc or n
    ldd = ldd or n
    d = out if out is not None else torch.empty(m * ldd, dtype=_TORCH[out_t], device=a.device)
    rc = L.lib().b200wmma_gemm(in_t, out_t, m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda, ldb,
                               ldc, ldd, float(alpha), float(beta), layout_a, layout_b,
                               _stream(stream))
    L.check(rc, "b200wmma_gemm")
    return d


def gemm_noalloc(in_t, out_t, m, n, k, a, b, c, alpha, beta, layout_a=ROW_MAJOR,
                 layout_b=COL_MAJOR, lda=None, ldb=None, ldc=None, ldd=None, out=None,
                 stream=None):
    """gemm() through the entry point that never allocates device memory: the scratch for
    transposed operand layouts is a fixed 8 MiB array inside the library.  `out` must be
    given by callers that cannot allocate; problems whose transposed operands exceed the
    array raise B200WmmaError (status -6).  Calls on one device must not overlap."""
    _require_cuda(a, b, c)
    lda = lda or _natural_ld(layout_a, m, k)
    ldb = ldb or _natural_ld(layout_b, k, n)
    ldc = ldc or n
    ldd = ldd or n
    d = out if out is not None else torch.empty(m * ldd, dtype=_TORCH[out_t], device=a.device)
    rc = L.lib().b200wmma_gemm_noalloc(in_t, out_t, m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d),
                                       lda, ldb, ldc, ldd, float(alpha), float(beta), layout_a,
                                       layout_b, _stream(stream))
    L.check(rc, "b200wmma_gemm_noalloc")
    return d


def gemm_host(in_t, out_t, m, n, k, a, b, c, d, alpha, beta, layout_a=ROW_MAJOR,
              layout_b=COL_MAJOR, stream=None):
    """Same with HOST tensors (ideally pinned): copies in, computes, copies D back, waits."""
    for t in (a, b, c, d):
        if t is not None and t.is_cuda:
            raise ValueError("gemm_host takes host tensors")
    lda = _natural_ld(layout_a, m, k)
    ldb = _natural_ld(layout_b, k, n)
    rc = L.lib().b200wmma_gemm_host(in_t, out_t, m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(d), lda,
                                    ldb, n, n, float(alpha), float(beta), layout_a, layout_b,
                                    _stream(stream))
    L.check(rc, "b200wmma_gemm_host")
    return d


def gemv(dtype, m, k, a, x, y, alpha, beta, lda=None, out=None, stream=None):
    """y_out = alpha*A*x + beta*y, A column-major (lda >= m)."""
    _require_cuda(a, x, y)
    out = out if out is not None else torch.empty_like(y)
    rc = L.lib().b200wmma_gemv(dtype, m, k, _ptr(a), _ptr(x), _ptr(y), _ptr(out), float(alpha),
                               float(beta), lda or m, _stream(stream))
    L.check(rc, "b200wmma_gemv")
    return out


def dlrm_fwd(x, m, k, batch, out=None, stream=None, dtype=F16):
    """[batch][m][k] -> [batch][k + m(m-1)/2]: row 0, then tril(X X^T, -1) row-major."""
    _require_cuda(x)
    out = out if out is not None else torch.empty(batch * (k + m * (m - 1) // 2),
                                                  dtype=_TORCH[dtype], device=x.device)
    rc = L.lib().b200wmma_dlrm_fwd(dtype, _ptr(x), _ptr(out), m, k, batch, _stream(stream))
    L.check(rc, "b200wmma_dlrm_fwd")
    return out


def dlrm_bwd(x, upstream, m, k, batch, grad=None, mlp_grad=None, stream=None, dtype=F16):
    """Returns (mlp_grad [batch][k], grad [batch][m][k])."""
    _require_cuda(x, upstream)
    grad = grad if grad is not None else torch.empty(batch * m * k, dtype=_TORCH[dtype],
                                                     device=x.device)
    mlp_grad = mlp_grad if mlp_grad is not None else torch.empty(batch * k, dtype=_TORCH[dtype],
                                                                 device=x.device)
    rc = L.lib().b200wmma_dlrm_bwd(dtype, _ptr(x), _ptr(upstream), _ptr(grad), _ptr(mlp_grad), m, k,
                                   batch, _stream(stream))
    L.check(rc, "b200wmma_dlrm_bwd")
    return mlp_grad, grad


def check_device(stream=None) -> None:
    """Waits for the stream; raises if a kernel gave up on a bounded device-side wait."""
    import ctypes as C
    detail = C.c_uint32(0)
    rc = L.lib().b200wmma_check_device(_stream(stream), C.byref(detail))
    if rc != L.OK:
        raise B200WmmaError(rc, f"b200wmma_check_device (wait code {detail.value})")


def shutdown() -> None:
    L.check(L.lib().b200wmma_shutdown(), "b200wmma_shutdown")
