"""The C-ABI library loads without a GPU and exports every symbol its header declares."""
import ctypes as C
import os
import re

from rocwmma_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "rocwmma_b200.h")).read()
    return sorted(set(re.findall(r"B200WMMA_API\s+[\w\s\*]+?\b(b200wmma_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    names = _declared()
    assert len(names) >= 10
    lib = C.CDLL(L.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/rocwmma_b200.h but not exported"
    assert sorted(L.SIGNATURES) == names, "python binding table and header disagree"


def test_version_and_status_strings():
    lib = L.lib()
    assert lib.b200wmma_version() == 10700
    for code in range(0, -7, -1):
        assert lib.b200wmma_status_string(code)
    assert b"unknown" in lib.b200wmma_status_string(-99)


def test_argument_validation_needs_no_device():
    lib = L.lib()
    null = None
    one = C.c_void_p(16)
    # null pointers / zero sizes are rejected before anything touches CUDA
    assert lib.b200wmma_gemm(L.F16, L.F16, 128, 128, 128, null, one, null, one, 128, 128, 128, 128,
                             1.0, 0.0, 0, 1, None) == L.ERR_INVALID_ARG
    assert lib.b200wmma_gemm(L.F16, L.F16, 0, 128, 128, one, one, null, one, 128, 128, 128, 128,
                             1.0, 0.0, 0, 1, None) == L.ERR_INVALID_ARG
    # beta != 0 needs C
    assert lib.b200wmma_gemm(L.F16, L.F16, 128, 128, 128, one, one, null, one, 128, 128, 128, 128,
                             1.0, 0.5, 0, 1, None) == L.ERR_INVALID_ARG
    assert lib.b200wmma_gemm(L.F16, L.F16, 128, 128, 128, one, one, null, one, 128, 128, 128, 128,
                             1.0, 0.0, 7, 1, None) == L.ERR_INVALID_ARG
    # fp64 with transposed layouts: an undersized leading dimension is refused before the
    # transposition pass is enqueued (column-major A needs lda >= m, row-major B ldb >= n)
    assert lib.b200wmma_gemm(L.F64, L.F64, 64, 64, 64, one, one, null, one, 56, 64, 64, 64,
                             1.0, 0.0, 1, 1, None) == L.ERR_INVALID_ARG
    assert lib.b200wmma_gemm(L.F64, L.F64, 64, 64, 64, one, one, null, one, 64, 56, 64, 64,
                             1.0, 0.0, 0, 0, None) == L.ERR_INVALID_ARG
    assert lib.b200wmma_gemm_simple(L.F16, L.F32, 16, 16, 16, null, one, one, one, 16, 16, 16, 16,
                                    1.0, 0.0, 0, 1, 0, 16, None) == L.ERR_INVALID_ARG
    assert lib.b200wmma_gemv(L.F32, 16, 16, one, null, one, one, 1.0, 0.0, 16, None) \
        == L.ERR_INVALID_ARG
    assert lib.b200wmma_gemv(L.F32, 16, 16, one, one, one, one, 1.0, 0.0, 8, None) \
        == L.ERR_INVALID_ARG          # lda < m
    assert lib.b200wmma_gemv(L.F16, 16, 16, one, one, one, one, 1.0, 0.0, 16, None) \
        == L.ERR_UNSUPPORTED
    assert lib.b200wmma_dlrm_fwd(L.F16, null, one, 27, 128, 8, None) == L.ERR_INVALID_ARG
    assert lib.b200wmma_dlrm_fwd(L.F32, one, one, 27, 128, 8, None) == L.ERR_UNSUPPORTED
    assert lib.b200wmma_dlrm_fwd(L.F16, one, one, 40, 128, 8, None) == L.ERR_UNSUPPORTED
    assert lib.b200wmma_dlrm_fwd(L.F16, one, one, 27, 100, 8, None) == L.ERR_UNSUPPORTED
    assert lib.b200wmma_dlrm_bwd(L.F16, one, one, null, one, 27, 128, 8, None) \
        == L.ERR_INVALID_ARG
    assert lib.b200wmma_dlrm_fwd(L.F16, C.c_void_p(8), one, 27, 128, 8, None) == L.ERR_ALIGNMENT


def test_host_api_refuses_cpu_tensors():
    import pytest
    import torch
    from rocwmma_b200 import api
    t = torch.zeros(16)
    with pytest.raises(ValueError):
        api.gemv(L.F32, 4, 4, t, t, t, 1.0, 0.0)
