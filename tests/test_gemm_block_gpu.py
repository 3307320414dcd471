"""Block-cooperative GEMM (TMA + tcgen05 + TMEM; fp64 on the warp-level path) through
the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle as O
from rocwmma_b200 import api, synth
from tests.cases import BLOCK_PAIRS, TOLERANCE, gemm_inputs, tolerance
from tests.gpu_util import to_device, to_host

pytestmark = pytest.mark.gpu
ROW, COL = 0, 1


ELEM = {O.F16: 2, O.BF16: 2, O.E4M3: 1, O.I8: 1, O.F32: 4, O.XF32: 4, O.F64: 8, O.I32: 4,
        O.E5M2: 1}


def _pad_ld(extent, dtype_code):
    """Smallest leading dimension >= extent whose byte size is a multiple of 16."""
    per16 = 16 // ELEM[dtype_code]
    return (extent + per16 - 1) // per16 * per16


def _run(case, with_c=True):
    """Runs the block GEMM with natural leading dimensions where they are 16-byte multiples,
    padded ones otherwise.  Output (and its padding) is prefilled with NaN / -7: anything
    the kernel fails to write, or writes outside m x n, shows up."""
    a, b, c = gemm_inputs(case)
    m, n, k = case["m"], case["n"], case["k"]
    it, ot = case["in_t"], case["out_t"]
    want = O.gemm(it, ot, m, n, k, a, b, c, case["alpha"], case["beta"], case["la"], case["lb"])

    def pad(flat, rows, cols, code):
        ld = _pad_ld(cols, code)
        if ld == cols:
            return flat, ld
        buf = np.zeros((rows, ld), dtype=flat.dtype)
        buf[:, :cols] = flat.reshape(rows, cols)
        return buf.reshape(-1), ld

    a_rows, a_cols = (m, k) if case["la"] == ROW else (k, m)
    b_rows, b_cols = (k, n) if case["lb"] == ROW else (n, k)
    a_p, lda = pad(a, a_rows, a_cols, it)
    b_p, ldb = pad(b, b_rows, b_cols, it)
    c_p, ldc = pad(c, m, n, ot)
    ldd = ldc
    fill = -7 if ot == O.I32 else float("nan")
    out = torch.full((m * ldd,), fill, dtype=api.torch_dtype(ot), device="cuda")
    api.gemm(it, ot, m, n, k, to_device(a_p, it), to_device(b_p, it),
             to_device(c_p, ot) if with_c else None, case["alpha"], case["beta"], case["la"],
             case["lb"], lda=lda, ldb=ldb, ldc=ldc, ldd=ldd, out=out)
    api.check_device()
    got = to_host(out, ot).reshape(m, ldd)
    if ldd != n:
        fill_bits = to_host(torch.full((1,), fill, dtype=api.torch_dtype(ot)), ot).view(np.uint8)
        pad_bits = np.ascontiguousarray(got[:, n:]).view(np.uint8).reshape(-1, fill_bits.size)
        assert (pad_bits == fill_bits).all(), "columns beyond n were overwritten"
    return np.ascontiguousarray(got[:, :n]).reshape(-1), want


def _ab(in_t):
    return (2, -1) if in_t == O.I8 else (2.0, -1.0)


@pytest.mark.parametrize("in_t,out_t", BLOCK_PAIRS)
def test_block_gemm_full_tiles(in_t, out_t):
    al, be = _ab(in_t)
    case = dict(in_t=in_t, out_t=out_t, m=256, n=512, k=512, la=ROW, lb=COL, alpha=al, beta=be,
                seed=40 + in_t)
    got, want = _run(case)
    err = O.max_rel_err(out_t, got, want)
    assert 0 <= err <= tolerance(in_t, out_t), err


@pytest.mark.parametrize("in_t,out_t", BLOCK_PAIRS)
@pytest.mark.parametrize("m,n,k", [(200, 136, 272), (1, 8, 16), (129, 257, 48), (384, 1000, 528),
                                   (130, 3, 7), (260, 264, 1040), (128, 1024, 272),
                                   (65, 777, 1040), (1, 512, 16)])
def test_block_gemm_ragged_edges(in_t, out_t, m, n, k):
    """Sizes that are not tile multiples: loads are zero-filled, stores masked.  The last three
    are skinny products (m <= 128, n >= 512), which run on the pair kernel with the second
    block of every pair entirely past the last row."""
    al, be = _ab(in_t)
    case = dict(in_t=in_t, out_t=out_t, m=m, n=n, k=k, la=ROW, lb=COL, alpha=al, beta=be,
                seed=50 + in_t)
    got, want = _run(case)
    err = O.max_rel_err(out_t, got, want)
    assert 0 <= err <= tolerance(in_t, out_t), err


@pytest.mark.parametrize("in_t,out_t", BLOCK_PAIRS)
@pytest.mark.parametrize("la,lb", [(COL, ROW), (ROW, ROW), (COL, COL)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 192), (300, 520, 264), (1024, 2048, 160),
                                   (100, 72, 40), (100, 520, 264)])
def test_block_gemm_other_layouts(in_t, out_t, la, lb, m, n, k):
    """Column-major A and row-major B are read in place as MN-major tensor-core operands
    (the layout of the reference's perf samples, samples/perf_hgemm.cpp:268-271)."""
    al, be = _ab(in_t)
    case = dict(in_t=in_t, out_t=out_t, m=m, n=n, k=k, la=la, lb=lb, alpha=al, beta=be,
                seed=60 + in_t)
    got, want = _run(case)
    assert 0 <= O.max_rel_err(out_t, got, want) <= tolerance(in_t, out_t)


@pytest.mark.parametrize("in_t,out_t", [(O.F16, O.F16), (O.BF16, O.F32), (O.XF32, O.F32)])
def test_two_width_tile_schedule(in_t, out_t, monkeypatch):
    """The pair kernel's optional schedule of wide tile columns followed by 128-wide ones
    (off by default, B200WMMA_GEMM_TAIL=1): for a 4096 x 4072 output on 74 pairs the launcher
    then picks 13 wide and 6 narrow columns, the last one ragged, so both widths, both tensor
    maps of B and the edge masks are exercised (K = 640 also makes xf32 accumulate in chunks)."""
    monkeypatch.setenv("B200WMMA_GEMM_TAIL", "1")
    m, n, k = 4096, 4072, 640
    case = dict(in_t=in_t, out_t=out_t, m=m, n=n, k=k, la=ROW, lb=COL, alpha=2.0, beta=-1.0,
                seed=77)
    a, b, c = gemm_inputs(case)
    want = O.gemm(in_t, out_t, m, n, k, a, b, c, 2.0, -1.0)
    got = api.gemm(in_t, out_t, m, n, k, to_device(a, in_t), to_device(b, in_t),
                   to_device(c, out_t), 2.0, -1.0)
    api.check_device()
    err = O.max_rel_err(out_t, to_host(got, out_t), want)
    assert 0 <= err <= tolerance(in_t, out_t), err


def test_beta_zero_never_reads_c():
    case = dict(in_t=O.F16, out_t=O.F16, m=256, n=256, k=128, la=ROW, lb=COL, alpha=1.0, beta=0.0,
                seed=70)
    got, want = _run(case, with_c=False)
    assert 0 <= O.max_rel_err(O.F16, got, want) <= 2e-3


def test_integer_pattern_inputs_are_exact():
    for in_t, out_t in BLOCK_PAIRS:
        case = dict(in_t=in_t, out_t=out_t, m=256, n=256, k=256, la=ROW, lb=COL, alpha=1, beta=1,
                    seed=5, dist="pattern")
        got, want = _run(case)
        assert O.max_rel_err(out_t, got, want) == 0.0, (in_t, out_t)


def test_padded_leading_dimensions_leave_padding_untouched():
    """Contamination check: D has ldd > n; the columns beyond n must keep their fill."""
    m, n, k = 256, 200, 128
    lda, ldb, ldd = k + 8, k + 16, n + 8
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    Bt = rng.uniform(-1, 1, (n, k)).astype(np.float16)
    a = np.zeros((m, lda), np.float16); a[:, :k] = A
    b = np.zeros((n, ldb), np.float16); b[:, :k] = Bt
    c = np.zeros(m * n, np.float16)
    want = O.gemm(O.F16, O.F16, m, n, k, A.reshape(-1), Bt.reshape(-1), c, 1.0, 0.0)
    out = torch.full((m * ldd,), 777.0, dtype=torch.float16, device="cuda")
    api.gemm(O.F16, O.F16, m, n, k, to_device(a.reshape(-1), O.F16), to_device(b.reshape(-1), O.F16),
             None, 1.0, 0.0, lda=lda, ldb=ldb, ldd=ldd, out=out)
    api.check_device()
    got = out.cpu().numpy().reshape(m, ldd)
    assert (got[:, n:] == 777.0).all()
    assert 0 <= O.max_rel_err(O.F16, np.ascontiguousarray(got[:, :n]).reshape(-1), want) <= 2e-3


@pytest.mark.parametrize("in_t,out_t", [(O.F16, O.F16), (O.BF16, O.F32), (O.I8, O.I32)])
def test_beta_with_c_in_place_and_own_leading_dimension(in_t, out_t):
    """beta != 0 over several tiles per block pair: once with C in a buffer of its own whose
    leading dimension differs from D's, once in place (C and D the same buffer).  Both must
    match the host routine; columns of D beyond n keep their fill."""
    m, n, k = 2100, 2600, 144  # 9 x 11 tiles: some block pairs get two
    al, be = _ab(in_t)
    case = dict(in_t=in_t, out_t=out_t, m=m, n=n, k=k, la=ROW, lb=COL, alpha=al, beta=be, seed=91)
    a, b, c = gemm_inputs(case)
    want = O.gemm(in_t, out_t, m, n, k, a, b, c, al, be, ROW, COL)
    ldc, ldd = n + 16, n + 32
    fill = -7 if out_t == O.I32 else 777.0
    cbuf = np.zeros((m, ldc), dtype=c.dtype); cbuf[:, :n] = c.reshape(m, n)
    da, db = to_device(a, in_t), to_device(b, in_t)
    out = torch.full((m * ldd,), fill, dtype=api.torch_dtype(out_t), device="cuda")
    api.gemm(in_t, out_t, m, n, k, da, db, to_device(cbuf.reshape(-1), out_t), al, be, ldc=ldc,
             ldd=ldd, out=out)
    api.check_device()
    got = to_host(out, out_t).reshape(m, ldd)
    assert (out.reshape(m, ldd)[:, n:] == fill).all(), "columns beyond n were overwritten"
    tol = 0.0 if out_t == O.I32 else 2e-3
    assert 0 <= O.max_rel_err(out_t, np.ascontiguousarray(got[:, :n]).reshape(-1), want) <= tol
    # in place
    dbuf = np.zeros((m, ldd), dtype=c.dtype); dbuf[:, :n] = c.reshape(m, n)
    inplace = to_device(dbuf.reshape(-1), out_t)
    api.gemm(in_t, out_t, m, n, k, da, db, inplace, al, be, ldc=ldd, ldd=ldd, out=inplace)
    api.check_device()
    got2 = to_host(inplace, out_t).reshape(m, ldd)
    assert np.array_equal(np.ascontiguousarray(got2[:, :n]).view(np.uint8),
                          np.ascontiguousarray(got[:, :n]).view(np.uint8))
    assert (np.ascontiguousarray(got2[:, n:]).view(np.uint8) == 0).all()


def test_misaligned_arguments_are_refused():
    t = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    with pytest.raises(api.B200WmmaError) as e:
        api.gemm(O.F16, O.F16, 128, 128, 100, t, t, None, 1, 0, lda=100, ldb=100)  # 200-byte rows
    assert e.value.status == -3
    with pytest.raises(api.B200WmmaError) as e:
        api.gemm(O.F16, O.F16, 128, 128, 128, t[1:], t, None, 1, 0)
    assert e.value.status == -3


def _rows_check(in_t, out_t, size, seed, alpha, beta, tol, nrows=24):
    """Full-size problem, validated on a sample of rows (the oracle needs ~minutes for all)."""
    m = n = k = size
    kw = {"dist": "int8"} if in_t == O.I8 else {}
    a = synth.rows(seed, 1, in_t, 0, m, k, **kw)
    bt = synth.rows(seed, 2, in_t, 0, n, k, **kw)
    d = api.gemm(in_t, out_t, m, n, k, to_device(a.reshape(-1), in_t),
                 to_device(bt.reshape(-1), in_t), None, alpha, beta)
    api.check_device()
    got = to_host(d, out_t).reshape(m, n)
    pick = np.unique(np.concatenate([[0, 127, 128, m - 1],
                                     np.random.default_rng(seed).integers(0, m, nrows)]))
    c0 = np.zeros(pick.size * n, dtype=O.np_dtype(out_t))
    want = O.gemm(in_t, out_t, pick.size, n, k, np.ascontiguousarray(a[pick]).reshape(-1),
                  bt.reshape(-1), c0, alpha, beta)
    err = O.max_rel_err(out_t, np.ascontiguousarray(got[pick]).reshape(-1), want)
    assert 0 <= err <= tol, err
    return got


def test_config_perf_hgemm_8192():
    """M=N=K=8192, fp16 A row / B col, fp32 accumulate, fp16 D, alpha=1, beta=0."""
    _rows_check(O.F16, O.F16, 8192, 1, 1.0, 0.0, 2e-3)


def test_config_int8_8192_bit_exact():
    _rows_check(O.I8, O.I32, 8192, 3, 1, 0, 0.0)


def test_linearity_at_full_size():
    """Size-independent property: gemm(A, B; alpha=2) == 2 * gemm(A, B; alpha=1) exactly
    (scaling by 2 commutes with fp16 rounding), on 4096^3."""
    m = n = k = 4096
    a = to_device(synth.matrix(2, 1, O.F16, m, k), O.F16)
    b = to_device(synth.matrix(2, 2, O.F16, n, k), O.F16)
    d1 = api.gemm(O.F16, O.F32, m, n, k, a, b, None, 1.0, 0.0)
    d2 = api.gemm(O.F16, O.F32, m, n, k, a, b, None, 2.0, 0.0)
    api.check_device()
    assert torch.equal(d2, 2 * d1)
    assert torch.isfinite(d1).all()


def _exact_rows(a_rows, bt, c_rows, alpha, beta, decode):
    """alpha * A B + beta * C for a few rows in float64 (the mathematically exact value up to
    double rounding), from the stored inputs."""
    return alpha * (decode(a_rows).astype(np.float64) @ decode(bt).astype(np.float64).T) \
        + beta * c_rows.astype(np.float64)


def _metric64(x, y):
    return float((np.abs(x - y) / (np.abs(x) + np.abs(y) + 1.0)).max())


@pytest.mark.parametrize("in_t,out_t", [(O.BF16, O.F32), (O.XF32, O.F32), (O.F32, O.F32),
                                        (O.F64, O.F64)])
def test_config_precision_sweep_4096(in_t, out_t):
    """M=N=K=4096, alpha=2, beta=-1, C nonzero; bf16 -> fp32, xf32 -> fp32, fp64 -- and full
    fp32 (three TF32 products over split operands), judged like xf32.

    Checked on a sample of rows against the oracle.  For xf32 the oracle's own fp32
    rounding (4096 products added one by one) already sits ~1.2e-4 away from the exact
    result in this metric, so no implementation that sums in another order can be within
    1e-4 of IT; what can be required, and is: the GPU result is within 1e-4 of the EXACT
    value, and no further from the oracle than the oracle is from exact, plus 1e-4."""
    m = n = k = 4096
    seed = 2
    a = synth.rows(seed, 1, in_t, 0, m, k)
    bt = synth.rows(seed, 2, in_t, 0, n, k)
    c = synth.rows(seed, 3, out_t, 0, m, n)
    d = api.gemm(in_t, out_t, m, n, k, to_device(a.reshape(-1), in_t),
                 to_device(bt.reshape(-1), in_t), to_device(c.reshape(-1), out_t), 2.0, -1.0)
    api.check_device()
    got = to_host(d, out_t).reshape(m, n)
    pick = np.unique(np.concatenate([[0, 127, 128, m - 1],
                                     np.random.default_rng(seed).integers(0, m, 28)]))
    want = O.gemm(in_t, out_t, pick.size, n, k, np.ascontiguousarray(a[pick]).reshape(-1),
                  bt.reshape(-1), np.ascontiguousarray(c[pick]).reshape(-1), 2.0, -1.0)
    g = np.ascontiguousarray(got[pick])
    err = O.max_rel_err(out_t, g.reshape(-1), want)
    if in_t in (O.XF32, O.F32):
        exact = _exact_rows(a[pick], bt, c[pick], 2.0, -1.0, lambda v: v)
        gpu_vs_exact = _metric64(g.astype(np.float64), exact)
        oracle_vs_exact = _metric64(want.reshape(pick.size, n).astype(np.float64), exact)
        assert gpu_vs_exact <= 1e-4, gpu_vs_exact
        assert 0 <= err <= oracle_vs_exact + 1e-4, (err, oracle_vs_exact)
    else:
        assert 0 <= err <= TOLERANCE[in_t], err


def test_config_fp8_8192_bf16_output():
    """e4m3 inputs (N(0,1) scaled to |x| <= 448), fp32 accumulate, bf16 D, 8192^3."""
    m = n = k = 8192
    seed = 3

    def gen(tid, rows):
        z = synth.rows(seed, tid, O.F32, 0, rows, k, dist="normal")
        return synth.f32_to_e4m3_bits(z * (448.0 / np.abs(z).max()))
    a, bt = gen(1, m), gen(2, n)
    # scale the product back into bf16 range through alpha
    alpha = 1.0 / 4096.0
    d = api.gemm(O.E4M3, O.BF16, m, n, k, to_device(a.reshape(-1), O.E4M3),
                 to_device(bt.reshape(-1), O.E4M3), None, alpha, 0.0)
    api.check_device()
    got = to_host(d, O.BF16).reshape(m, n)
    pick = np.unique(np.random.default_rng(seed).integers(0, m, 24))
    c0 = np.zeros(pick.size * n, dtype=np.uint16)
    want = O.gemm(O.E4M3, O.BF16, pick.size, n, k, np.ascontiguousarray(a[pick]).reshape(-1),
                  bt.reshape(-1), c0, alpha, 0.0)
    err = O.max_rel_err(O.BF16, np.ascontiguousarray(got[pick]).reshape(-1), want)
    assert 0 <= err <= 1e-2, err


@pytest.mark.parametrize("m,beta", [(2304, 0.5), (300, 0.0), (1024, -1.0)])
def test_host_buffer_entry_point(m, beta):
    """b200wmma_gemm_host: pinned host buffers in, host buffer out (slab-pipelined copies for
    m >= 1024, one-shot below)."""
    n, k = 512, 384
    case = dict(in_t=O.F16, out_t=O.F16, m=m, n=n, k=k, la=ROW, lb=COL, alpha=1.5, beta=beta,
                seed=80)
    a, b, c = gemm_inputs(case)
    want = O.gemm(O.F16, O.F16, m, n, k, a, b, c, 1.5, beta)
    ta, tb, tc = (torch.from_numpy(v).pin_memory() for v in (a, b, c))
    td = torch.full((m * n,), float("nan"), dtype=torch.float16).pin_memory()
    for _ in range(2):   # the second call reuses the cached staging buffers and streams
        td.fill_(float("nan"))
        api.gemm_host(O.F16, O.F16, m, n, k, ta, tb, tc if beta != 0 else None, td, 1.5, beta)
        assert 0 <= O.max_rel_err(O.F16, td.numpy(), want) <= 2e-3
    api.check_device()


@pytest.mark.parametrize("m", [1024, 2048])
def test_multi_gpu_shard_shapes(m):
    """The row shards of an 8- and 4-GPU run of the 8192^3 problem (reduced K): the launcher
    narrows the tile to 224 columns for these so the tiles fill whole waves."""
    case = dict(in_t=O.F16, out_t=O.F16, m=m, n=8192, k=256, la=ROW, lb=COL, alpha=1.0, beta=0.0,
                seed=75)
    got, want = _run(case, with_c=False)
    assert 0 <= O.max_rel_err(O.F16, got, want) <= 2e-3


@pytest.mark.parametrize("m", [64, 128, 1024])
def test_dependent_launches_keep_stream_order(m):
    """The block kernels are launched so that their set-up overlaps the previous kernel of the
    stream; everything after it must still see that kernel's results.  A chain X <- X . B of
    eight launches, each reading the previous launch's output as A (and once as C), issued
    back to back, must equal the same chain with a device synchronisation after every launch,
    bit for bit.  m = 64 / 128 take the skinny route, 1024 the ordinary pair kernel."""
    n = k = 1024
    a = to_device(synth.rows(91, 1, O.F16, 0, m, k).reshape(-1), O.F16)
    b = to_device((synth.rows(91, 2, O.F16, 0, n, k) / 16).astype(np.float16).reshape(-1), O.F16)

    def chain(sync):
        x = a.clone()
        for i in range(8):
            y = torch.empty_like(x)
            api.gemm(O.F16, O.F16, m, n, k, x, b, x if i == 3 else None, 1.0,
                     0.5 if i == 3 else 0.0, out=y)
            if sync:
                torch.cuda.synchronize()
            x = y
        torch.cuda.synchronize()
        return x.cpu().numpy().view(np.uint16)

    want = chain(True)
    for _ in range(3):
        assert np.array_equal(chain(False), want)
    api.check_device()
    assert np.isfinite(want.view(np.float16).astype(np.float32)).all()


@pytest.mark.parametrize("in_t,out_t,alpha,beta", [(O.F16, O.F16, 1.0, 0.0), (O.BF16, O.F32, 2.0, -1.0),
                                                   (O.I8, O.I32, 1, 1), (O.E4M3, O.BF16, 2.0 ** -8, 0.0)])
def test_split_last_wave(in_t, out_t, alpha, beta, monkeypatch):
    """A 4096 x 4096 output is 256 tiles on 74 CTA pairs: the 34 tiles of the last wave are cut
    in two along K and meet in a workspace (drainSplitPart).  The result must agree with the
    unsplit launch (bit for bit for int8, whose sums are exact in any order) and with the CPU
    oracle on a sample of rows; two launches in a row leave the arrival counters at zero."""
    m = n = 4096
    k = 1024
    seed = 9
    dist = "int8" if in_t == O.I8 else "uniform"
    a = synth.rows(seed, 1, in_t, 0, m, k, dist=dist)
    bt = synth.rows(seed, 2, in_t, 0, n, k, dist=dist)
    c = synth.rows(seed, 3, out_t, 0, m, n, dist="int32" if out_t == O.I32 else "uniform")
    da, db, dc = to_device(a.reshape(-1), in_t), to_device(bt.reshape(-1), in_t), \
        to_device(c.reshape(-1), out_t)
    cc = dc if beta != 0 else None
    monkeypatch.setenv("B200WMMA_GEMM_SPLIT", "0")
    whole = api.gemm(in_t, out_t, m, n, k, da, db, cc, alpha, beta)
    monkeypatch.setenv("B200WMMA_GEMM_SPLIT", "1")
    split1 = api.gemm(in_t, out_t, m, n, k, da, db, cc, alpha, beta)
    split2 = api.gemm(in_t, out_t, m, n, k, da, db, cc, alpha, beta)
    api.check_device()
    assert torch.equal(split1.view(torch.uint8), split2.view(torch.uint8))
    got = to_host(split1, out_t).reshape(m, n)
    ref = to_host(whole, out_t).reshape(m, n)
    if in_t == O.I8:
        assert np.array_equal(got, ref)
    pick = np.unique(np.concatenate([[0, 255, 256, m - 257, m - 1],
                                     np.random.default_rng(seed).integers(0, m, 16)]))
    c_rows = np.ascontiguousarray(c[pick]).reshape(-1)
    want = O.gemm(in_t, out_t, pick.size, n, k, np.ascontiguousarray(a[pick]).reshape(-1),
                  bt.reshape(-1), c_rows, alpha, beta)
    for res in (got, ref):
        err = O.max_rel_err(out_t, np.ascontiguousarray(res[pick]).reshape(-1), want)
        assert 0 <= err <= tolerance(in_t, out_t), err
