"""Shared test cases and seeded input builders (host side, numpy)."""
from __future__ import annotations

import numpy as np

from rocwmma_b200 import synth
from rocwmma_b200.synth import BF16, E4M3, E5M2, F16, F32, F64, I8, I32, XF32

ROW, COL = 0, 1

# Tolerances on max |a-b| / (|a|+|b|+1) per input type: bit-exact for i8 -> i32.
TOLERANCE = {F16: 2e-3, BF16: 2e-3, E4M3: 1e-2, E5M2: 1e-2, I8: 0.0, F32: 1e-4, XF32: 1e-4,
             F64: 1e-12}

# An output stored in bf16 carries 8 significant bits: results that differ only in the
# fp32 summation order can round to neighbouring bf16 values, 2^-8 apart relative to the
# value, which the metric sees as up to 2^-8 / (2 + 1/|v|) ~ 3.9e-3.  fp16 outputs
# (11 bits) stay inside the 2e-3 of their input type.
BF16_OUTPUT_TOLERANCE = 4e-3


def tolerance(in_t, out_t):
    tol = TOLERANCE[in_t]
    return max(tol, BF16_OUTPUT_TOLERANCE) if out_t == BF16 else tol


# (input type, output type) pairs of the simple (per-warp) GEMM
SIMPLE_PAIRS = [(F16, F32), (F16, F16), (BF16, F32), (BF16, BF16), (E4M3, F32), (I8, I32),
                (F32, F32), (XF32, F32), (F64, F64)]
# pairs of the block-cooperative GEMM
BLOCK_PAIRS = [(F16, F16), (F16, F32), (BF16, F32), (BF16, BF16), (XF32, F32), (F32, F32),
               (I8, I32),
               (E4M3, BF16), (E4M3, F32), (E5M2, BF16), (E5M2, F32), (F64, F64)]

# (input, output, compute) triples of the simple GEMM beyond SIMPLE_PAIRS' usual compute
# types (rocWMMA docs/api-reference/api-reference-guide.rst:80-153).
EXTRA_TRIPLES = [(F16, F16, F16), (BF16, BF16, BF16), (I8, I8, I32), (E5M2, F32, F32)]

# With a 16-bit COMPUTE type the CPU reference rounds after every product and every
# addition while the tensor core rounds once per instruction (fp16) or once per BlockK
# step (bf16, carried through fp32 as rocWMMA does), so the two legitimately differ by
# rounding noise that grows with K.  The reference's own pass mark for these triples is
# 10 * eps of the type (samples/common.hpp:410); it is used here unchanged.
COMPUTE_TOLERANCE = {F16: 10 * 2.0 ** -10, BF16: 10 * 2.0 ** -7}


def triple_tolerance(in_t, out_t, comp_t):
    return COMPUTE_TOLERANCE.get(comp_t, tolerance(in_t, out_t))


def _dist(dt):
    return {"dist": "int8"} if dt == I8 else ({"dist": "int32"} if dt == I32 else
                                              {"dist": "uniform"})


def gemm_inputs(case):
    """A (m x k), B (k x n), C (m x n) as flat storage in the case's layouts.

    The generator produces logical rows; a column-major operand is the
    transposed storage of the same logical matrix."""
    m, n, k, seed = case["m"], case["n"], case["k"], case["seed"]
    it, ot = case["in_t"], case["out_t"]
    dist = case.get("dist")
    kw_in = {"dist": dist} if dist else _dist(it)
    kw_out = {"dist": dist} if dist else _dist(ot)
    a = synth.rows(seed, 1, it, 0, m, k, **kw_in)            # logical m x k
    bt = synth.rows(seed, 2, it, 0, n, k, **kw_in)           # logical B^T: n x k
    c = synth.rows(seed, 3, ot, 0, m, n, **kw_out)
    a_st = a if case["la"] == ROW else np.ascontiguousarray(a.T)
    b_st = bt if case["lb"] == COL else np.ascontiguousarray(bt.T)
    return a_st.reshape(-1), b_st.reshape(-1), c.reshape(-1)


def _case(in_t, out_t, m, n, k, la, lb, alpha, beta, seed, **kw):
    d = dict(in_t=in_t, out_t=out_t, m=m, n=n, k=k, la=la, lb=lb, alpha=alpha, beta=beta,
             seed=seed)
    d.update(kw)
    return d


# Cases whose outputs are stored in tests/golden/gemm_ref_outputs.npz (made by the
# reference's own gemm_CPU).  bf16 OUTPUT and bf16 compute are absent: the reference's
# host code for float -> bf16 lives in a HIP header outside its tree.  (8-bit float INPUTS
# only need the format-defined decoding.)
GEMM_GOLDEN_CASES = {}
for _it, _ot in [(F16, F32), (F16, F16), (BF16, F32), (I8, I32), (F32, F32), (XF32, F32),
                 (F64, F64)]:
    for _la, _lb in [(ROW, COL), (COL, ROW), (ROW, ROW), (COL, COL)]:
        _ab = (1, 1) if _it == I8 else (2.0, -1.0)
        GEMM_GOLDEN_CASES[f"t{_it}_{_ot}_l{_la}{_lb}"] = _case(_it, _ot, 48, 32, 64, _la, _lb,
                                                            _ab[0], _ab[1], seed=100 + _it)


for _it, _ot, _ct in [(F16, F16, F16), (I8, I8, I32), (E4M3, F32, F32), (E5M2, F32, F32)]:
    for _la, _lb in [(ROW, COL), (COL, ROW)]:
        _ab = (3, -2) if _it == I8 else (2.0, -1.0)
        GEMM_GOLDEN_CASES[f"t{_it}_{_ot}_c{_ct}_l{_la}{_lb}"] = _case(
            _it, _ot, 48, 32, 64, _la, _lb, _ab[0], _ab[1], seed=120 + _it, comp_t=_ct)


def gemv_inputs(m, k, seed):
    a = synth.rows(seed, 1, F32, 0, k, m).reshape(-1)   # column-major m x k = k rows of m
    x = synth.rows(seed, 2, F32, 0, 1, k).reshape(-1)
    y = synth.rows(seed, 3, F32, 0, 1, m).reshape(-1)
    return a, x, y


def dlrm_inputs(m, k, batch, seed):
    x = synth.rows(seed, 1, F16, 0, batch, m * k, dist="normal").reshape(-1)
    up = synth.rows(seed, 2, F16, 0, batch, k + m * (m - 1) // 2, dist="normal").reshape(-1)
    return x, up
