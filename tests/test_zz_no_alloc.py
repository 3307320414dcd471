"""The allocation-free GEMM entry point (b200wmma_gemm_noalloc) against the regular one.

Some callers cannot let a library call cudaMalloc: a server or framework whose own pool
already owns the GPU's memory, or a latency-critical loop that cannot afford the
device-wide wait an allocation or free may cause.  For them the library offers a variant
whose transposition scratch is a fixed 8 MiB array inside the library image.  It runs the
same kernels as b200wmma_gemm, so its results must be identical, call after call, even
though the array still holds the previous call's data.

This file sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from rocwmma_b200 import _lib as L
from rocwmma_b200 import api
from tests.cases import TOLERANCE, gemm_inputs
from tests.gpu_util import to_device, to_host

ROW, COL = 0, 1


def _call(fn_name, case, out):
    """One call straight through the C ABI (no wrapper): device pointers and sizes only."""
    a, b, c = case["_dev"]
    m, n, k = case["m"], case["n"], case["k"]
    lda = k if case["la"] == ROW else m
    ldb = n if case["lb"] == ROW else k
    fn = getattr(L.lib(), fn_name)
    rc = fn(case["in_t"], case["out_t"], m, n, k, a.data_ptr(), b.data_ptr(), c.data_ptr(),
            out.data_ptr(), lda, ldb, n, n, float(case["alpha"]), float(case["beta"]), case["la"],
            case["lb"], torch.cuda.current_stream().cuda_stream)
    assert rc == L.OK, (fn_name, rc)


@pytest.mark.gpu
def test_noalloc_matches_regular_entry_point_on_consecutive_calls():
    cases = [
        # both operands need the scratch; the second call is smaller, so it runs on top of
        # stale data left by the first; the third uses other types and only one transpose
        dict(in_t=O.F16, out_t=O.F16, m=384, n=320, k=264, la=COL, lb=ROW, alpha=1.5, beta=0.5,
             seed=91),
        dict(in_t=O.F16, out_t=O.F16, m=200, n=136, k=72, la=COL, lb=ROW, alpha=2.0, beta=-1.0,
             seed=92),
        dict(in_t=O.I8, out_t=O.I32, m=256, n=256, k=160, la=ROW, lb=ROW, alpha=1, beta=1,
             seed=93),
        dict(in_t=O.E5M2, out_t=O.BF16, m=160, n=192, k=96, la=COL, lb=COL, alpha=1.0, beta=0.0,
             seed=94),
    ]
    for case in cases:
        a, b, c = gemm_inputs(case)
        case["_dev"] = (to_device(a, case["in_t"]), to_device(b, case["in_t"]),
                        to_device(c, case["out_t"]))
        m, n = case["m"], case["n"]
        dt = api.torch_dtype(case["out_t"])
        fill = -7 if case["out_t"] == O.I32 else float("nan")
        want_dev = torch.full((m * n,), fill, dtype=dt, device="cuda")
        got_dev = torch.full((m * n,), fill, dtype=dt, device="cuda")   # allocated by the caller
        _call("b200wmma_gemm", case, want_dev)
        _call("b200wmma_gemm_noalloc", case, got_dev)
        torch.cuda.synchronize()
        api.check_device()
        got, want = to_host(got_dev, case["out_t"]), to_host(want_dev, case["out_t"])
        err = O.max_rel_err(case["out_t"], got, want)
        assert 0 <= err <= TOLERANCE[case["in_t"]], (case["seed"], err)
        # same kernels, same order of operations: in fact bit-identical
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
        # and both agree with the CPU oracle
        ref = O.gemm(case["in_t"], case["out_t"], m, n, case["k"], a, b, c, case["alpha"],
                     case["beta"], case["la"], case["lb"])
        assert 0 <= O.max_rel_err(case["out_t"], got, ref) <= TOLERANCE[case["in_t"]]


def test_noalloc_rejects_sizes_beyond_its_scratch():
    """4096 x 4096 fp16 operands need 32 MiB of transposed copies each: refused up front,
    before anything touches the device (so this part needs no GPU)."""
    one = C.c_void_p(256)
    rc = L.lib().b200wmma_gemm_noalloc(L.F16, L.F16, 4096, 4096, 4096, one, one, None, one, 4096,
                                       4096, 4096, 4096, 1.0, 0.0, COL, ROW, None)
    assert rc == L.ERR_TOO_LARGE
    assert L.lib().b200wmma_gemm_noalloc(L.F64, L.F64, 64, 64, 64, one, one, None, one, 64, 64, 64,
                                         64, 1.0, 0.0, ROW, COL, None) == L.ERR_UNSUPPORTED
    assert L.lib().b200wmma_gemm_noalloc(L.F16, L.F16, 64, 64, 64, None, one, None, one, 64, 64, 64,
                                         64, 1.0, 0.0, ROW, COL, None) == L.ERR_INVALID_ARG
    # a leading dimension smaller than the extent it strides over is refused before the
    # transposition pass could read past the operand: column-major A needs lda >= m,
    # row-major B needs ldb >= n (the pointers are dummies; nothing is launched)
    assert L.lib().b200wmma_gemm_noalloc(L.F16, L.F16, 64, 64, 64, one, one, None, one, 56, 64, 64,
                                         64, 1.0, 0.0, COL, COL, None) == L.ERR_INVALID_ARG
    assert L.lib().b200wmma_gemm_noalloc(L.F16, L.F16, 64, 64, 64, one, one, None, one, 64, 56, 64,
                                         64, 1.0, 0.0, ROW, ROW, None) == L.ERR_INVALID_ARG
    assert L.lib().b200wmma_gemm_noalloc(L.F16, L.F16, 64, 64, 64, one, one, None, one, 64, 64, 64,
                                         56, 1.0, 0.0, COL, ROW, None) == L.ERR_INVALID_ARG
    # a misaligned output is refused before anything is launched as well
    assert L.lib().b200wmma_gemm_noalloc(L.F16, L.F16, 64, 64, 64, one, one, None,
                                         C.c_void_p(258), 64, 64, 64, 64, 1.0, 0.0, COL, ROW,
                                         None) == L.ERR_ALIGNMENT
