"""Per-warp fragment API, end to end: the one-tile-per-warp GEMM (simple_*gemm samples)
through the C ABI against the CPU oracle and the stored reference outputs."""
import os

import numpy as np
import pytest

import oracle as O
from rocwmma_b200 import api
from tests.cases import (EXTRA_TRIPLES, GEMM_GOLDEN_CASES, SIMPLE_PAIRS, TOLERANCE, gemm_inputs,
                         tolerance, triple_tolerance)
from tests.gpu_util import to_device, to_host

pytestmark = pytest.mark.gpu
ROW, COL = 0, 1


def _run_simple(case, layout_cd=ROW, block=16, compute=None, block_k=0):
    a, b, c = gemm_inputs(case)
    m, n, k = case["m"], case["n"], case["k"]
    if layout_cd == COL:
        c = np.ascontiguousarray(c.reshape(m, n).T).reshape(-1)
    want = O.gemm(case["in_t"], case["out_t"], m, n, k, a, b, c, case["alpha"], case["beta"],
                  case["la"], case["lb"], layout_cd, layout_cd, comp_t=compute)
    got = api.gemm_simple(case["in_t"], case["out_t"], m, n, k, to_device(a, case["in_t"]),
                          to_device(b, case["in_t"]), to_device(c, case["out_t"]), case["alpha"],
                          case["beta"], case["la"], case["lb"], layout_cd, block, compute=compute,
                          block_k=block_k)
    return to_host(got, case["out_t"]), want


def _host_rounding_noise(case, comp_t, want):
    """With a 16-bit compute type the host reference rounds to 11 (fp16) or 8 (bf16)
    significant bits after every one of the K products and additions; the device rounds
    once per tensor-core instruction (fp16) or keeps fp32 inside a BlockK step (bf16).  The
    host result's own distance from fp32 compute is therefore part of what separates the
    two, and is added to the tolerance.  Zero for the other compute types."""
    if comp_t not in (O.F16, O.BF16):
        return 0.0
    a, b, c = gemm_inputs(case)
    fine = O.gemm(case["in_t"], case["out_t"], case["m"], case["n"], case["k"], a, b, c,
                  case["alpha"], case["beta"], case["la"], case["lb"])
    return O.max_rel_err(case["out_t"], want, fine)


@pytest.mark.parametrize("in_t,out_t", SIMPLE_PAIRS)
@pytest.mark.parametrize("la,lb", [(ROW, COL), (COL, ROW), (ROW, ROW), (COL, COL)])
@pytest.mark.parametrize("block", [16, 32])
def test_simple_gemm_types_layouts_blocks(in_t, out_t, la, lb, block):
    if block == 32 and in_t == O.F64:
        pytest.skip("64-bit fragments are 16x16 only, as in the reference")
    alpha, beta = (2, -1) if in_t == O.I8 else (2.0, -1.0)
    case = dict(in_t=in_t, out_t=out_t, m=96, n=64, k=64, la=la, lb=lb, alpha=alpha, beta=beta,
                seed=20 + in_t)
    got, want = _run_simple(case, ROW, block)
    err = O.max_rel_err(out_t, got, want)
    assert 0 <= err <= tolerance(in_t, out_t), (err, tolerance(in_t, out_t))


@pytest.mark.parametrize("in_t,out_t,comp_t", EXTRA_TRIPLES)
@pytest.mark.parametrize("la,lb", [(ROW, COL), (COL, ROW)])
@pytest.mark.parametrize("block", [16, 32])
def test_simple_gemm_other_type_triples(in_t, out_t, comp_t, la, lb, block):
    """fp16 / bf16 compute types, int8 outputs, e5m2 inputs (Ti / To / Tc of the reference's
    extended test set, test/gemm/gemm_common_test_params.hpp:51-121)."""
    alpha, beta = (2, -1) if in_t == O.I8 else (2.0, -1.0)
    case = dict(in_t=in_t, out_t=out_t, m=96, n=64, k=64, la=la, lb=lb, alpha=alpha, beta=beta,
                seed=40 + in_t)
    got, want = _run_simple(case, ROW, block, compute=comp_t)
    err = O.max_rel_err(out_t, got, want)
    tol = triple_tolerance(in_t, out_t, comp_t) + _host_rounding_noise(case, comp_t, want)
    assert 0 <= err <= tol, (err, tol)


def test_other_type_triples_are_exact_on_integer_pattern_inputs():
    """Small-integer inputs and K = 16 keep every partial sum exactly representable even in
    bf16, so the 16-bit compute types must then match the oracle bit for bit."""
    for in_t, out_t, comp_t in EXTRA_TRIPLES:
        case = dict(in_t=in_t, out_t=out_t, m=32, n=32, k=16, la=ROW, lb=COL, alpha=1, beta=1,
                    seed=6, dist="pattern")
        got, want = _run_simple(case, compute=comp_t)
        assert O.max_rel_err(out_t, got, want) == 0.0, (in_t, out_t, comp_t)


def test_int8_output_wraps_like_the_host_cast():
    """I8 / I8 / I32: the int32 result is narrowed to int8 by a plain cast on both sides."""
    case = dict(in_t=O.I8, out_t=O.I8, m=64, n=64, k=128, la=ROW, lb=COL, alpha=3, beta=-2,
                seed=44)
    got, want = _run_simple(case, compute=O.I32)
    assert np.array_equal(got, want)


BLOCK_K_CASES = [(O.F16, O.F32, 16, 32), (O.F16, O.F32, 16, 64), (O.F16, O.F32, 32, 32),
                 (O.F16, O.F32, 32, 64), (O.BF16, O.BF16, 32, 64), (O.E4M3, O.F32, 16, 32),
                 (O.E4M3, O.F32, 32, 16), (O.E4M3, O.F32, 32, 64), (O.E5M2, O.F32, 16, 64),
                 (O.I8, O.I32, 16, 32), (O.I8, O.I32, 32, 16), (O.I8, O.I32, 32, 64),
                 (O.F32, O.F32, 16, 8), (O.F32, O.F32, 32, 32), (O.XF32, O.F32, 16, 8),
                 (O.XF32, O.F32, 32, 8), (O.XF32, O.F32, 32, 32), (O.F64, O.F64, 16, 4),
                 (O.F64, O.F64, 16, 8), (O.F16, O.F32, 16, 128), (O.BF16, O.F32, 16, 128),
                 (O.E4M3, O.F32, 16, 128), (O.I8, O.I32, 16, 128),
                 # below the K extent of the full-depth tensor-core instruction: the reference's
                 # minima for 32 x 32 blocks (test/gemm/gemm_predicates_base.hpp:137-209)
                 (O.F16, O.F32, 32, 8), (O.F16, O.F16, 32, 8), (O.BF16, O.F32, 32, 8),
                 (O.BF16, O.BF16, 32, 8), (O.F16, O.F32, 16, 8), (O.XF32, O.F32, 32, 4),
                 (O.XF32, O.F32, 16, 4), (O.F32, O.F32, 32, 4)]


@pytest.mark.parametrize("in_t,out_t,block,block_k", BLOCK_K_CASES)
def test_simple_gemm_other_fragment_k_extents(in_t, out_t, block, block_k):
    """BlockK away from the usual 16 (reference: from the per-type minimum up to 128,
    test/gemm/gemm_common_test_params.hpp:51-121)."""
    alpha, beta = (2, -1) if in_t == O.I8 else (2.0, -1.0)
    case = dict(in_t=in_t, out_t=out_t, m=64, n=96, k=128, la=ROW, lb=COL, alpha=alpha,
                beta=beta, seed=50 + in_t)
    got, want = _run_simple(case, ROW, block, block_k=block_k)
    err = O.max_rel_err(out_t, got, want)
    assert 0 <= err <= tolerance(in_t, out_t), err


def test_half_depth_fragments_with_16_bit_accumulation():
    """f16 / f16 / f16 with BlockK = 8 (m16n8k8 with fp16 accumulators) on the reference's
    small-integer fill, where every product and sum is exact in any order; bf16 / bf16 / bf16
    (rounded to bf16 per BlockK step) within the reference's pass mark for that type."""
    case = dict(in_t=O.F16, out_t=O.F16, m=64, n=64, k=64, la=ROW, lb=COL, alpha=1.0, beta=1.0,
                seed=77, dist="pattern")
    got, want = _run_simple(case, ROW, 32, compute=O.F16, block_k=8)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    case = dict(in_t=O.BF16, out_t=O.BF16, m=64, n=64, k=64, la=ROW, lb=COL, alpha=1.0, beta=1.0,
                seed=78)
    got, want = _run_simple(case, ROW, 32, compute=O.BF16, block_k=8)
    err = O.max_rel_err(O.BF16, got, want)
    assert 0 <= err <= triple_tolerance(O.BF16, O.BF16, O.BF16) + _host_rounding_noise(
        case, O.BF16, want), err


def test_unbuilt_fragment_k_extent_is_refused():
    case = dict(in_t=O.F16, out_t=O.F32, m=64, n=64, k=128, la=ROW, lb=COL, alpha=1.0, beta=0.0,
                seed=1)
    with pytest.raises(Exception):
        _run_simple(case, ROW, 32, block_k=128)


@pytest.mark.parametrize("in_t,out_t", [(O.F16, O.F32), (O.I8, O.I32), (O.F64, O.F64)])
def test_simple_gemm_col_major_cd(in_t, out_t):
    alpha, beta = (1, 1) if in_t == O.I8 else (1.5, 0.5)
    case = dict(in_t=in_t, out_t=out_t, m=64, n=96, k=48, la=ROW, lb=COL, alpha=alpha, beta=beta,
                seed=31)
    got, want = _run_simple(case, COL, 16)
    assert 0 <= O.max_rel_err(out_t, got, want) <= TOLERANCE[in_t]


@pytest.mark.parametrize("name", sorted(GEMM_GOLDEN_CASES))
def test_simple_gemm_against_stored_reference_outputs(name, golden_dir):
    case = GEMM_GOLDEN_CASES[name]
    want = np.load(os.path.join(golden_dir, "gemm_ref_outputs.npz"))[name]
    got, _ = _run_simple(case, ROW, 16, compute=case.get("comp_t"))
    err = O.max_rel_err(case["out_t"], got, want)
    tol = triple_tolerance(case["in_t"], case["out_t"], case.get("comp_t"))
    assert 0 <= err <= tol + _host_rounding_noise(case, case.get("comp_t"), want)


def test_integer_pattern_inputs_are_exact():
    """With the reference's small-integer fill every type must match the oracle exactly."""
    for in_t, out_t in SIMPLE_PAIRS:
        case = dict(in_t=in_t, out_t=out_t, m=64, n=64, k=64, la=ROW, lb=COL, alpha=1, beta=1,
                    seed=5, dist="pattern")
        got, want = _run_simple(case)
        assert O.max_rel_err(out_t, got, want) == 0.0, (in_t, out_t)


def test_config_simple_hgemm_1024():
    """D = 1.5 A B + 0.5 C, 1024^3, fp16 A row / B col, fp32 C/D row, 16x16x16, seed 0."""
    case = dict(in_t=O.F16, out_t=O.F32, m=1024, n=1024, k=1024, la=ROW, lb=COL, alpha=1.5,
                beta=0.5, seed=0)
    got, want = _run_simple(case)
    err = O.max_rel_err(O.F32, got, want)
    assert 0 <= err <= 2e-3


def test_size_must_be_a_multiple_of_the_fragment():
    import torch
    t = torch.zeros(64 * 64, dtype=torch.float16, device="cuda")
    c = torch.zeros(64 * 64, dtype=torch.float32, device="cuda")
    with pytest.raises(api.B200WmmaError) as e:
        api.gemm_simple(O.F16, O.F32, 40, 64, 64, t, t, c, 1, 0)
    assert e.value.status == -1
