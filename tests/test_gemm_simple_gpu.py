"""Per-warp fragment API, end to end: the one-tile-per-warp GEMM (simple_*gemm samples)
through the C ABI against the CPU oracle and the stored reference outputs."""
import os

import numpy as np
import pytest

import oracle as O
from rocwmma_b200 import api
from tests.cases import (GEMM_GOLDEN_CASES, SIMPLE_PAIRS, TOLERANCE, gemm_inputs, tolerance)
from tests.gpu_util import to_device, to_host

pytestmark = pytest.mark.gpu
ROW, COL = 0, 1


def _run_simple(case, layout_cd=ROW, block=16):
    a, b, c = gemm_inputs(case)
    m, n, k = case["m"], case["n"], case["k"]
    if layout_cd == COL:
        c = np.ascontiguousarray(c.reshape(m, n).T).reshape(-1)
    want = O.gemm(case["in_t"], case["out_t"], m, n, k, a, b, c, case["alpha"], case["beta"],
                  case["la"], case["lb"], layout_cd, layout_cd)
    got = api.gemm_simple(case["in_t"], case["out_t"], m, n, k, to_device(a, case["in_t"]),
                          to_device(b, case["in_t"]), to_device(c, case["out_t"]), case["alpha"],
                          case["beta"], case["la"], case["lb"], layout_cd, block)
    return to_host(got, case["out_t"]), want


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
    got, _ = _run_simple(case, ROW, 16)
    err = O.max_rel_err(case["out_t"], got, want)
    assert 0 <= err <= TOLERANCE[case["in_t"]]


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
