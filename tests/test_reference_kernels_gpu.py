"""Source-level drop-in check: the reference's OWN sample kernels -- their text unmodified --
compiled against this repository's include/rocwmma (oracle/ref_kernels.cu ->
oracle/_ref/libref_kernels.so, built where the reference tree is mounted), run on the GPU and
compared with the CPU oracle.

What this covers that the other tests do not: the macro-tile kernels of perf_hgemm / perf_sgemm /
perf_dgemm (samples/perf_hgemm.cpp:329-714) use the cooperative load -> applyDataLayout /
applyTranspose -> cooperative store -> shared memory -> load -> mma_sync chain, GetDataLayout_t /
GetIOShape_t address maps and fragments as large as 128 x 16, exactly as rocWMMA users write
them."""
import numpy as np
import pytest
import torch

import oracle as O
from rocwmma_b200 import synth
from tests.cases import TOLERANCE, dlrm_inputs, gemv_inputs
from tests.gpu_util import to_device, to_host

pytestmark = pytest.mark.gpu
ROW, COL = 0, 1


@pytest.fixture(scope="module")
def K():
    lib = O.ref_kernels()
    if lib is None:
        pytest.skip("oracle/_ref/libref_kernels.so was not built (needs the reference tree)")
    return lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _gemm_case(K, fn, dt, m, n, k, la, lb, alpha, beta, seed):
    a = synth.rows(seed, 1, dt, 0, m, k)
    bt = synth.rows(seed, 2, dt, 0, n, k)
    c = synth.rows(seed, 3, dt, 0, m, n).reshape(-1)
    a_st = (a if la == ROW else np.ascontiguousarray(a.T)).reshape(-1)
    b_st = (bt if lb == COL else np.ascontiguousarray(bt.T)).reshape(-1)
    lda = k if la == ROW else m
    ldb = n if lb == ROW else k
    want = O.gemm(dt, dt, m, n, k, a_st, b_st, c, alpha, beta, la, lb)
    da, db, dc = to_device(a_st, dt), to_device(b_st, dt), to_device(c, dt)
    dd = torch.full_like(dc, float("nan"))
    rc = getattr(K, fn)(m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr(), dd.data_ptr(), lda,
                        ldb, n, n, alpha, beta, _stream())
    assert rc == 0
    torch.cuda.synchronize()
    return to_host(dd, dt), want


@pytest.mark.parametrize("fn,dt", [("refk_perf_hgemm", O.F16), ("refk_perf_sgemm", O.F32),
                                   ("refk_perf_dgemm", O.F64)])
@pytest.mark.parametrize("mult", [(1, 1, 2), (3, 2, 9)])
def test_reference_macro_tile_kernels(K, fn, dt, mult):
    """perf_*gemm: A column-major, B row-major, C / D row-major, alpha = beta = 2
    (samples/perf_hgemm.cpp:264-271, 948)."""
    import ctypes as C
    tile = (C.c_uint32 * 4)()
    getattr(K, fn + "_tile")(tile)
    m, n, k = tile[0] * mult[0], tile[1] * mult[1], tile[2] * mult[2]
    got, want = _gemm_case(K, fn, dt, m, n, k, COL, ROW, 2.0, 2.0, seed=60 + dt)
    err = O.max_rel_err(dt, got, want)
    assert 0 <= err <= TOLERANCE[dt], err


@pytest.mark.parametrize("fn,dt", [("refk_simple_hgemm", O.F16), ("refk_simple_sgemm", O.F32),
                                   ("refk_simple_dgemm", O.F64)])
def test_reference_simple_kernels(K, fn, dt):
    """simple_*gemm: A row-major, B column-major, C / D row-major (samples/simple_hgemm.cpp:69-79)."""
    got, want = _gemm_case(K, fn, dt, 128, 192, 80, ROW, COL, 2.1, 2.1, seed=70 + dt)
    err = O.max_rel_err(dt, got, want)
    assert 0 <= err <= TOLERANCE[dt], err


@pytest.mark.parametrize("fn,dt", [("refk_simple_sgemv", O.F32), ("refk_simple_dgemv", O.F64)])
def test_reference_gemv_kernels(K, fn, dt):
    """simple_sgemv / simple_dgemv.  The sample kernel multiplies a 16-column B tile and loads /
    stores 16-column C / D tiles although only column 0 carries the vector
    (samples/simple_sgemv.cpp:139,145,153: ldb = k, ldc = ldd = m), so it touches 16 k elements
    from x and 16 m elements from y_in and y_out.  The buffers handed to it here are that
    large -- column 0 holds the vector, columns 1..15 are padding -- so that no access leaves
    an allocation; only column 0 of the result is compared."""
    m, k = 256, 192
    cols = 16
    a, x, y = gemv_inputs(m, k, seed=11)
    if dt == O.F64:
        a, x, y = a.astype(np.float64), x.astype(np.float64), y.astype(np.float64)
    want = O.gemv(dt, m, k, a, x, y, 2.1, 2.1)
    x_pad = np.zeros(cols * k, dtype=x.dtype)
    x_pad[:k] = x
    y_pad = np.zeros(cols * m, dtype=y.dtype)
    y_pad[:m] = y
    da, dx, dy = to_device(a, dt), to_device(x_pad, dt), to_device(y_pad, dt)
    out = torch.full_like(dy, float("nan"))
    assert dx.numel() == cols * k and dy.numel() == cols * m and out.numel() == cols * m
    rc = getattr(K, fn)(m, k, da.data_ptr(), dx.data_ptr(), dy.data_ptr(), out.data_ptr(), 2.1,
                        2.1, _stream())
    assert rc == 0
    torch.cuda.synchronize()
    got = to_host(out, dt)
    # the tensor-core tile sums a column block at a time, the host routine one product at a
    # time: same values, other rounding order
    err = O.max_rel_err(dt, np.ascontiguousarray(got[:m]), want)
    assert 0 <= err <= (1e-4 if dt == O.F32 else 1e-12), err
    # the padding columns were written by the kernel (beta * 0 + alpha * A * 0 = 0), nothing else
    assert np.all(got[m:] == 0)


def test_reference_dlrm_kernels(K):
    """simple_dlrm forward and backward (three kernels).  m = 64 fills all four warps of the
    sample's 128-thread block with a tile row each, so no warp leaves the kernel before the
    block-wide barriers the kernel executes inside its bounds check."""
    m, k, b = 64, 128, 6
    x, up = dlrm_inputs(m, k, b, seed=4)
    out_len = k + m * (m - 1) // 2
    dx, dup = to_device(x, O.F16), to_device(up, O.F16)
    out = torch.zeros(b * out_len, dtype=torch.float16, device="cuda")
    acc32 = torch.zeros(b * m * m, dtype=torch.float32, device="cuda")
    assert K.refk_dlrm_fwd(dx.data_ptr(), out.data_ptr(), acc32.data_ptr(), m, k, b, _stream()) == 0
    grad = torch.zeros(b * m * k, dtype=torch.float16, device="cuda")
    mlp = torch.zeros(b * k, dtype=torch.float16, device="cuda")
    acc16 = torch.zeros(b * m * m, dtype=torch.float16, device="cuda")
    assert K.refk_dlrm_bwd(dx.data_ptr(), dup.data_ptr(), grad.data_ptr(), mlp.data_ptr(),
                           acc16.data_ptr(), m, k, b, _stream()) == 0
    torch.cuda.synchronize()
    want_fwd = O.dlrm_fwd(O.F16, x, m, k, b)
    want_mlp, want_grad = O.dlrm_bwd(O.F16, x, up, m, k, b)
    assert O.max_rel_err(O.F16, to_host(out, O.F16), want_fwd) <= 2e-3
    assert np.array_equal(to_host(mlp, O.F16).view(np.uint16), want_mlp.view(np.uint16))
    assert O.max_rel_err(O.F16, to_host(grad, O.F16), want_grad) <= 2e-3
