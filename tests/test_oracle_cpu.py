"""CPU checks of the oracle itself: it must reproduce the reference's stored vectors
and the outputs of the reference's own host code before any GPU result is trusted."""
import os

import numpy as np
import pytest
import torch

import oracle as O
from rocwmma_b200 import synth
from tests.cases import (GEMM_GOLDEN_CASES, TOLERANCE, dlrm_inputs, gemm_inputs, gemv_inputs)

M, K = 27, 128
OUT = K + M * (M - 1) // 2


def _ulps_fp16(a, b):
    def key(x):
        i = x.view(np.int16).astype(np.int32)
        return np.where(i < 0, -(i & 0x7FFF), i)
    return np.abs(key(a) - key(b)).max()


def test_dlrm_fwd_matches_reference_fixture(golden_dir):
    f = np.load(os.path.join(golden_dir, "dlrm_reference_fixture.npz"))
    x, want = f["input_fp16"], f["output_fp16"]
    b = x.size // (M * K)
    got = O.dlrm_fwd(O.F16, x, M, K, b)
    # the stored vectors were produced on a GPU: sums differ in order, at most 1 fp16 ulp
    assert _ulps_fp16(got, want) <= 1
    assert (got.view(np.uint16) == want.view(np.uint16)).mean() > 0.99
    x32, want32 = f["input_fp32"], f["output_fp32"]
    got32 = O.dlrm_fwd(O.F32, x32, M, K, x32.size // (M * K))
    assert O.max_rel_err(O.F32, got32, want32) < 1e-5


def test_dlrm_bwd_matches_reference_fixture(golden_dir):
    f = np.load(os.path.join(golden_dir, "dlrm_reference_fixture.npz"))
    x, up = f["input_fp16"], f["input_grad_fp16"]
    b = x.size // (M * K)
    mlp, grad = O.dlrm_bwd(O.F16, x, up, M, K, b)
    assert np.array_equal(mlp.view(np.uint16), f["output_mlp_input_grad_fp16"].view(np.uint16))
    assert O.max_rel_err(O.F16, grad, f["output_input_grad_fp16"]) <= 2e-3
    x32, up32 = f["input_fp32"], f["input_grad_fp32"]
    mlp32, grad32 = O.dlrm_bwd(O.F32, x32, up32, M, K, x32.size // (M * K))
    assert np.array_equal(mlp32, f["output_mlp_input_grad_fp32"])
    assert O.max_rel_err(O.F32, grad32, f["output_input_grad_fp32"]) < 1e-5


@pytest.mark.parametrize("name", sorted(GEMM_GOLDEN_CASES))
def test_gemm_matches_reference_host_code(name, golden_dir):
    """Bit-for-bit against outputs of the reference's gemm_CPU (stored golden vectors)."""
    case = GEMM_GOLDEN_CASES[name]
    want = np.load(os.path.join(golden_dir, "gemm_ref_outputs.npz"))[name]
    a, b, c = gemm_inputs(case)
    for literal in (False, True):
        got = O.gemm(case["in_t"], case["out_t"], case["m"], case["n"], case["k"], a, b, c,
                     case["alpha"], case["beta"], case["la"], case["lb"], literal=literal,
                     comp_t=case.get("comp_t"))
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (name, literal)


def test_gemv_matches_reference_host_code(golden_dir):
    want = np.load(os.path.join(golden_dir, "gemv_ref_outputs.npz"))["y"]
    a, x, y = gemv_inputs(256, 192, seed=11)
    got = O.gemv(O.F32, 256, 192, a, x, y, 2.1, 2.1)
    assert np.array_equal(got, want)


def test_dlrm_matches_reference_host_code(golden_dir):
    g = np.load(os.path.join(golden_dir, "dlrm_ref_outputs.npz"))
    x, up = dlrm_inputs(27, 128, 9, seed=4)
    assert np.array_equal(O.dlrm_fwd(O.F16, x, 27, 128, 9).view(np.uint16), g["fwd"].view(np.uint16))
    mlp, grad = O.dlrm_bwd(O.F16, x, up, 27, 128, 9)
    assert np.array_equal(mlp.view(np.uint16), g["mlp"].view(np.uint16))
    assert np.array_equal(grad.view(np.uint16), g["grad"].view(np.uint16))


@pytest.mark.skipif(not os.path.isdir(O.reference_dir()), reason="reference tree not mounted")
def test_live_reference_build_agrees():
    """Where the reference tree is mounted, its freshly compiled host code must agree too."""
    assert O.ref() is not None
    rng = np.random.default_rng(5)
    m, n, k = 40, 24, 56
    a = rng.uniform(-1, 1, m * k).astype(np.float16)
    b = rng.uniform(-1, 1, k * n).astype(np.float16)
    c = rng.uniform(-1, 1, m * n).astype(np.float32)
    got = O.gemm(O.F16, O.F32, m, n, k, a, b, c, 1.5, 0.5)
    want = O.ref_gemm(O.F16, O.F32, m, n, k, a, b, c, 1.5, 0.5)
    assert np.array_equal(got, want)


@pytest.mark.skipif(not os.path.isdir(O.reference_dir()), reason="reference tree not mounted")
@pytest.mark.parametrize("triple", [(O.F16, O.F16, O.F16), (O.I8, O.I8, O.I32),
                                    (O.E4M3, O.F32, O.F32), (O.E5M2, O.F32, O.F32)])
def test_live_reference_build_agrees_on_other_type_triples(triple):
    it, ot, ct = triple
    rng = np.random.default_rng(9)
    m, n, k = 24, 40, 96

    def draw(dt, count):
        if dt == O.I8:
            return rng.integers(-128, 128, count).astype(np.int8)
        v = rng.standard_normal(count).astype(np.float32)
        return {O.F16: lambda: v.astype(np.float16), O.F32: lambda: v,
                O.E4M3: lambda: O.encode_e4m3(v), O.E5M2: lambda: O.encode_e5m2(v)}[dt]()

    a, b, c = draw(it, m * k), draw(it, k * n), draw(ot, m * n)
    alpha, beta = (3, -2) if it == O.I8 else (2.0, -1.0)
    want = O.ref_gemm(it, ot, m, n, k, a, b, c, alpha, beta, comp_t=ct)
    for literal in (False, True):
        got = O.gemm(it, ot, m, n, k, a, b, c, alpha, beta, comp_t=ct, literal=literal)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (triple, literal)


@pytest.mark.skipif(not os.path.isdir(O.reference_dir()), reason="reference tree not mounted")
def test_reference_sample_kernels_compile_unmodified():
    """Source-level drop-in: the kernel text of the reference's perf_*gemm, simple_*gemm,
    simple_*gemv and simple_dlrm samples compiles, unmodified, against include/rocwmma
    (oracle/ref_kernels.cu; nvcc cross-compiles without a GPU).  The GPU tests run them."""
    lib = O.ref_kernels()
    assert lib is not None
    import ctypes as C
    tile = (C.c_uint32 * 4)()
    lib.refk_perf_hgemm_tile(tile)
    # the sample's parameters for 32-lane hardware: 16 x 16 x 16 fragments, 4 x 2 per warp,
    # 2 x 4 warps -> 128 x 128 macro tile, 256 threads (samples/perf_hgemm.cpp:239-252)
    assert list(tile) == [128, 128, 16, 256]


def test_e5m2_codec():
    """e5m2 is the upper byte of binary16; the encoder rounds to nearest even, saturates to
    +-57344 and agrees with the input generators' numpy encoder."""
    from rocwmma_b200 import synth
    codes = np.arange(256, dtype=np.uint8)
    dec = O.decode_e5m2(codes)
    via16 = (codes.astype(np.uint16) << 8).view(np.float16).astype(np.float32)
    assert np.array_equal(np.isnan(dec), np.isnan(via16))
    assert np.array_equal(dec[~np.isnan(dec)], via16[~np.isnan(via16)])
    fin = np.isfinite(dec) & (dec != 0)
    assert np.array_equal(O.encode_e5m2(dec[fin]), codes[fin])
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(50000) * np.exp(rng.uniform(-14, 12, 50000))).astype(np.float32)
    x[:6] = [0.0, 57344.0, 61000.0, -1e9, 2.0 ** -17, 1.5 * 2.0 ** -16]
    enc = O.encode_e5m2(x)
    assert np.array_equal(enc, synth.f32_to_e5m2_bits(x))
    assert enc[1] == 0x7B and enc[2] == 0x7B and enc[3] == 0xFB and enc[4] == 0
    assert enc[5] == 2  # tie between 1 and 2 units of 2^-16: to even


def test_bf16_compute_type_rounds_every_operation():
    """BF16 / BF16 / BF16: blocked and literal forms agree; 64 products rounded one by one
    to 8 significant bits leave visible noise against fp32 compute, but only noise."""
    rng = np.random.default_rng(4)
    m, n, k = 16, 24, 64
    a, b, c = (O.encode_bf16(rng.standard_normal(s)) for s in (m * k, k * n, m * n))
    d16 = O.gemm(O.BF16, O.BF16, m, n, k, a, b, c, 2.0, -1.0, comp_t=O.BF16)
    lit = O.gemm(O.BF16, O.BF16, m, n, k, a, b, c, 2.0, -1.0, comp_t=O.BF16, literal=True)
    d32 = O.gemm(O.BF16, O.BF16, m, n, k, a, b, c, 2.0, -1.0)
    assert np.array_equal(d16, lit)
    assert 0 < O.max_rel_err(O.BF16, d16, d32) < 0.3


def test_leading_dimensions_and_cd_layouts():
    """Padded leading dimensions and column-major C/D against a float64 numpy product."""
    rng = np.random.default_rng(7)
    m, n, k = 20, 12, 28
    lda, ldb, ldc, ldd = k + 3, k + 5, m + 2, m + 4
    A = rng.integers(-4, 5, (m, k)).astype(np.float32)
    B = rng.integers(-4, 5, (k, n)).astype(np.float32)
    Cm = rng.integers(-4, 5, (m, n)).astype(np.float32)
    a = np.zeros(m * lda, np.float32); a.reshape(m, lda)[:, :k] = A          # row-major
    b = np.zeros(n * ldb, np.float32); b.reshape(n, ldb)[:, :k] = B.T        # col-major
    c = np.zeros(n * ldc, np.float32); c.reshape(n, ldc)[:, :m] = Cm.T       # col-major
    d = O.gemm(O.F32, O.F32, m, n, k, a, b, c, 2, -1, O.ROW, O.COL, O.COL, O.COL,
               lda=lda, ldb=ldb, ldc=ldc, ldd=ldd)
    want = 2 * (A @ B) - Cm
    assert np.array_equal(d.reshape(n, ldd)[:, :m].T, want)


def test_error_metric():
    a = np.array([1.0, 2.0, -3.0], np.float32)
    b = np.array([1.0, 2.5, -3.0], np.float32)
    assert abs(O.max_rel_err(O.F32, a, b) - 0.5 / 5.5) < 1e-12
    assert O.max_rel_err(O.F32, a, np.array([1.0, np.inf, 0], np.float32)) == -1.0
    assert O.max_rel_err(O.F32, a, np.array([1.0, np.nan, 0], np.float32)) == -2.0
    assert O.max_rel_err(O.I32, np.array([5], np.int32), np.array([5], np.int32)) == 0.0


def test_encoders_agree_with_torch_and_numpy():
    x = np.random.default_rng(1).standard_normal(100000).astype(np.float32) * 60
    x[:8] = [0, 2.0 ** -10, 2.0 ** -9, 1.5 * 2.0 ** -9, 447.9, 448, 1e4, -1e-3]
    mine = O.encode_e4m3(x)
    assert np.array_equal(mine, synth.f32_to_e4m3_bits(x))
    t = torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, t)
    allbits = np.arange(256, dtype=np.uint8)
    assert np.array_equal(O.decode_e4m3(allbits), synth.e4m3_bits_to_f32(allbits), equal_nan=True)
    tb = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.encode_bf16(x), tb)
    assert np.array_equal(O.encode_bf16(x), synth.f32_to_bf16_bits(x))


def test_integer_pattern_is_exact_for_every_type():
    """The reference's small-integer fill makes every GEMM exact: all type pairs agree."""
    base = None
    for it, ot in [(O.F16, O.F32), (O.BF16, O.F32), (O.E4M3, O.F32), (O.F32, O.F32),
                   (O.F64, O.F64), (O.I8, O.I32)]:
        case = dict(in_t=it, out_t=ot, m=32, n=16, k=48, la=0, lb=1, alpha=1, beta=1, seed=3,
                    dist="pattern")
        a, b, c = gemm_inputs(case)
        d = O.gemm(it, ot, 32, 16, 48, a, b, c, 1, 1).astype(np.float64)
        base = d if base is None else base
        assert np.array_equal(d, base), (it, ot)
