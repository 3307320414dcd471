#!/usr/bin/env python
"""Throughput, roofline fraction and parity of every benchmark configuration other than the
headline one (which bench.py itself times): one result per kernel and configuration, the
way rocWMMA's GEMM test programs print one row per kernel (test/gemm/gemm_kernel_base_impl.hpp:441-523).

    python bench_configs.py [--only NAME[,NAME...]] [--iters N] [--small] [--no-check] [--csv FILE]
    python -m torch.distributed.run --nproc-per-node N ... bench_configs.py ...

bench.py imports run_all() and attaches its results to its JSON line as `extras`.

Configurations
    simple_hgemm   1024^3 fp16 -> fp32, 16x16x16 fragments, alpha 1.5, beta 0.5   (seed 0)
    hgemm          8192^3 fp16 -> fp16, alpha 1, beta 0 (stand-alone runs only)   (seed 1)
    bf16 xf32 f32 f64   4096^3, alpha 2, beta -1, C nonzero                       (seed 2)
    i8 fp8 bf8     8192^3 int8 -> int32 and e4m3 / e5m2 -> bf16                   (seed 3)
    dlrm_fwd dlrm_bwd   batch 65536, 27 x 128 fp16;  sgemv 16384^2 fp32           (seed 4)

Inputs come from the seeded host generator (rocwmma_b200.synth), so the CPU side checks
exactly the values the GPU computed on: after timing, a sample of each rank's own rows (or
DLRM samples; all rows for GEMV) is recomputed by the CPU oracle -- the reference's own
host routine where it was built -- and the largest relative error (the reference's metric)
is reported next to the tolerance.  GEMMs report TFLOP/s = 2 M N K / time against the measured
dense bf16 tensor peak scaled per type; GEMV and DLRM report algorithmic bytes / time against
the measured copy bandwidth.  Timing: CUDA events over `iters` back-to-back launches after
warm-ups; when a configuration's working set fits in the 126 MB L2 (the 1024^3 sample, a
shard of a many-GPU run) the launches rotate through enough copies of its buffers that every
launch reads its operands from DRAM.

Under torchrun every configuration is split over the ranks as rocwmma_b200.shard says (GEMM
by rows of A / C / D with B replicated, DLRM by batch, GEMV by rows; no collective in a
timed region); figures are whole-job totals over the slowest rank's time and the parity
figure is the worst over the ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from rocwmma_b200 import api, shard, synth  # noqa: E402
from rocwmma_b200._lib import (BF16, COL_MAJOR, E4M3, E5M2, F16, F32, F64, I8, I32,  # noqa: E402
                               ROW_MAJOR, XF32)

WORLD = int(os.environ.get("WORLD_SIZE", "1"))
RANK = int(os.environ.get("RANK", "0"))
# How many ranks the problem is cut for.  Normally the process group's size; --as-shard-of N
# makes a single process run (and time) rank 0's share of an N-rank job, which is how the
# profiler captures of shard-sized launches are taken on one GPU.
SHARD_WORLD = WORLD

# north_star tolerances on max |a-b| / (|a|+|b|+1), per input type
TOLERANCE = {F16: 2e-3, BF16: 2e-3, E4M3: 1e-2, E5M2: 1e-2, I8: 0.0, F32: 1e-4, XF32: 1e-4,
             F64: 1e-12}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def _barrier():
    if WORLD > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(v: float) -> float:
    return shard.max_over_ranks(float(v), device="cuda")


def gen_threads() -> int:
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    return max(1, min(16, cores // max(1, WORLD)))


L2_BYTES = 126 << 20


def copies_needed(working_set: int) -> int:
    """How many copies of a configuration's device buffers a timed loop rotates through so that
    no launch finds its operands in L2: 1 when the working set exceeds the L2 by itself, else
    enough copies for 2.5 x the L2 between two uses of the same copy."""
    if working_set > L2_BYTES:
        return 1
    return min(64, max(2, -(-int(2.5 * L2_BYTES) // max(1, working_set))))


def replicate(count, *tensors):
    """`count` sets of the given device tensors (set 0 = the originals; None stays None)."""
    sets = [tensors]
    for _ in range(count - 1):
        sets.append(tuple(None if t is None else t.clone() for t in tensors))
    return sets


def timed(fn, iters, copies=1):
    """Per-launch time in ms, the slowest rank's: `iters` back-to-back launches between two
    device events (after 3 warm-ups per copy in use).  fn(i) launches on buffer set
    i % copies; with a working set smaller than the L2 the sets rotate (copies_needed), so
    that every launch reads its operands from DRAM like the first one would -- and the
    launches still run back to back, as they would in a pipeline that feeds the kernel new
    data each time.  Returns (ms, copies)."""
    iters = max(iters, copies) if copies > 1 else iters
    for i in range(max(3, copies)):
        fn(i)
    _barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    _barrier()
    total = e0.elapsed_time(e1)
    api.check_device()
    return _max_over_ranks(total) / iters, copies


def l2_note(copies):
    return ("working set exceeds L2" if copies == 1
            else f"{copies} copies of the buffers in rotation (2.5 x L2 between reuses)")


def to_device(a: np.ndarray, code: int) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a).reshape(-1))
    if code == BF16:
        return t.view(torch.int16).cuda().view(torch.bfloat16)
    return t.cuda()


def to_host(t: torch.Tensor, code: int) -> np.ndarray:
    if code == BF16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def _dist(code):
    return "int8" if code == I8 else "int32" if code == I32 else "uniform"


def _fp8_matrix(seed, tid, code, row0, nrows, ncols, total_rows):
    """N(0,1) values scaled so that the largest magnitude of the WHOLE matrix maps to the
    format's maximum, then rounded to nearest even.  A rank holding a row range needs the
    matrix-wide maximum: it is reduced over the ranks (outside any timed region)."""
    z = synth.rows(seed, tid, F32, row0, nrows, ncols, dist="normal", threads=gen_threads())
    peak = float(np.abs(z).max()) if z.size else 0.0
    if nrows != total_rows and WORLD > 1:
        t = torch.tensor([peak], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        peak = float(t.item())
    top = 448.0 if code == E4M3 else 57344.0
    z *= np.float32(top / peak)
    tz = torch.from_numpy(z)
    # torch's conversions are bit-identical to synth.f32_to_e4m3_bits / f32_to_e5m2_bits for
    # finite values inside the range (the test-suite checks that) and run on all cores
    bits = tz.to(torch.float8_e4m3fn if code == E4M3 else torch.float8_e5m2).view(torch.uint8)
    return bits.numpy()


def _checker_threads():
    import oracle as O
    return O.set_num_threads(max(1, O.host_cores() // max(1, WORLD)))


def _pick_rows(m_local, count, seed):
    if m_local <= count:
        return np.arange(m_local)
    fixed = [r for r in (0, 1, 127, 128, m_local - 2, m_local - 1) if 0 <= r < m_local]
    rnd = np.random.default_rng(seed * 1000 + RANK).integers(0, m_local, count)
    return np.unique(np.concatenate([fixed, rnd]).astype(np.int64))


def _metric64(x, y):
    return float((np.abs(x - y) / (np.abs(x) + np.abs(y) + 1.0)).max())


# rocWMMA's spellings of the element types in its result tables (dataTypeToString).
_TYPE_NAME = {F16: "f16", BF16: "bf16", E4M3: "f8", E5M2: "bf8", I8: "i8", I32: "i32",
              F32: "f32", XF32: "xf32", F64: "f64"}
_ELEM_BYTES = {F16: 2, BF16: 2, E4M3: 1, E5M2: 1, I8: 1, I32: 4, F32: 4, XF32: 4, F64: 8}

CSV_HEADER = ("TBlkX, TBlkY, BlkM, BlkN, BlkK, MatM, MatN, MatK, alpha, lda, ldb, beta, ldc, ldd, "
              "LytA_LytB_LytC_LytD, Ti_To_Tc, elapsedMs, Problem Size(GFlops), TFlops/s, "
              "Efficiency(%), Result")


def csv_row(r):
    g = r["gemm"]
    comp = I32 if g["in_t"] == I8 else F64 if g["in_t"] == F64 else F32
    if g["simple"]:
        tile = (128, 4, 16, 16, 16)       # thread block and fragment of the per-warp kernel
    elif g["in_t"] == F64:
        tile = (256, 1, 128, 128, 16)     # block tile of the double-precision kernel
    else:
        tile = (192, 1, 256, 256, 128 // _ELEM_BYTES[g["in_t"]])  # CTA-pair tile, one ring slot
    n = g["size"]
    result = "BENCH" if r.get("parity") is None else ("PASSED" if r["parity"] else "FAILED")
    fields = [*tile, n, n, n, g["alpha"], n, n, g["beta"], n, n, "row_col_row_row",
              f"{_TYPE_NAME[g['in_t']]}_{_TYPE_NAME[g['out_t']]}_{_TYPE_NAME[comp]}",
              f"{r['ms']:.6f}", f"{2.0 * n ** 3 / 1e9:.3f}", f"{r['value']:.3f}",
              f"{100.0 * r['roofline']['frac']:.2f}", result]
    return ", ".join(str(f) for f in fields)


def gemm_case(name, in_t, out_t, size, alpha, beta, seed, peak_scale, simple=False, iters=20,
              check=True, check_rows=16):
    """One GEMM configuration: this rank's rows of A / C / D, all of B."""
    n = k = size
    row0, m = shard.gemm_shard(size, SHARD_WORLD, RANK)
    th = gen_threads()
    if in_t in (E4M3, E5M2):
        a = _fp8_matrix(seed, 1, in_t, row0, m, k, size)
        bt = _fp8_matrix(seed, 2, in_t, 0, n, k, n)
        # Inputs reach the format's maximum, so the products sum to ~1e6 (e4m3) or ~1e10
        # (e5m2).  The reference's metric |a-b| / (|a|+|b|+1) is a relative measure only for
        # values of order 1 and above whose ABSOLUTE error is small against 1; alpha brings
        # the results back to O(100) so that it measures what the tolerance is about.
        alpha = 2.0 ** -12 if in_t == E4M3 else 2.0 ** -26
    else:
        a = synth.rows(seed, 1, in_t, row0, m, k, dist=_dist(in_t), threads=th)
        bt = synth.rows(seed, 2, in_t, 0, n, k, dist=_dist(in_t), threads=th)
    c = synth.rows(seed, 3, out_t, row0, m, n, dist=_dist(out_t), threads=th) if beta != 0 else None
    da, db = to_device(a, in_t), to_device(bt, in_t)
    dc = to_device(c, out_t) if c is not None else None
    dd = torch.empty(m * n, dtype=api.torch_dtype(out_t), device="cuda")
    ws = (m * k + k * n) * _ELEM_BYTES[in_t] + m * n * _ELEM_BYTES[out_t] * (2 if c is not None else 1)
    sets = replicate(copies_needed(ws), da, db, dc, dd)
    if simple:
        def fn(i):
            xa, xb, xc, xd = sets[i % len(sets)]
            api.gemm_simple(in_t, out_t, m, n, k, xa, xb, xc, alpha, beta, ROW_MAJOR, COL_MAJOR,
                            ROW_MAJOR, 16, out=xd)
    else:
        def fn(i):
            xa, xb, xc, xd = sets[i % len(sets)]
            api.gemm(in_t, out_t, m, n, k, xa, xb, xc, alpha, beta, out=xd)
    ms, copies = timed(fn, iters, len(sets))
    work_rows = size if SHARD_WORLD == WORLD else m     # a lone shard counts its own rows only
    tf = 2.0 * work_rows * n * k / ms / 1e9
    peak_bf16, _, src = peaks()
    peak = (peak_bf16 * peak_scale if peak_scale else 40.0) * WORLD
    res = {"config": name, "n_gpus": WORLD, "ms": ms, "value": tf, "unit": "TFLOP/s",
           "partition": f"M-split x{WORLD}, B replicated", "seed": seed,
           "l2": l2_note(copies),
           "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s",
                        "frac": tf / peak, "algorithmic_flops": 2.0 * size * n * k,
                        "peak_source": (f"{src} bf16 tensor peak x {peak_scale} x {WORLD} GPU(s)"
                                        + ("" if peak_scale == 1.0 else " (derived)")
                                        if peak_scale else
                                        f"nominal fp64 tensor 40 TFLOP/s x {WORLD} GPU(s)")},
           "gemm": {"in_t": in_t, "out_t": out_t, "size": size, "alpha": alpha, "beta": beta,
                    "simple": simple}}
    if check:
        import oracle as O
        threads = _checker_threads()
        pick = _pick_rows(m, check_rows, seed)
        a_s = np.ascontiguousarray(a[pick]).reshape(-1)
        c_s = (np.ascontiguousarray(c[pick]).reshape(-1) if c is not None
               else np.zeros(pick.size * n, dtype=O.np_dtype(out_t)))
        # bf16 OUTPUTS are encoded by a routine outside the reference tree, so the reference
        # build has no such pair: those go to the restatement
        use_ref = O.ref() is not None and out_t != BF16
        want = (O.ref_gemm if use_ref else O.gemm)(in_t, out_t, pick.size, n, k, a_s,
                                                   bt.reshape(-1), c_s, alpha, beta)
        got = to_host(dd, out_t).reshape(m, n)[pick]
        err = O.max_rel_err(out_t, np.ascontiguousarray(got).reshape(-1), want)
        tol = TOLERANCE[in_t]
        ok = 0 <= err <= tol
        res["checker"] = ("rocWMMA gemm_CPU" if use_ref else "oracle port") + \
            f", {pick.size} rows per rank, {threads} threads"
        if in_t in (XF32, F32):
            # the host routine's own sequential fp32 rounding over K = 4096 is further than
            # 1e-4 from the exact value, so the result is judged against the exact (fp64)
            # value, and against the host routine with that routine's own distance added
            exact = alpha * (a[pick].astype(np.float64) @ bt.astype(np.float64).T) \
                + beta * c[pick].astype(np.float64)
            e_gpu = _metric64(got.astype(np.float64), exact)
            e_cpu = _metric64(want.reshape(pick.size, n).astype(np.float64), exact)
            res["max_rel_err_vs_exact"] = _max_over_ranks(e_gpu)
            res["checker_vs_exact"] = _max_over_ranks(e_cpu)
            ok = e_gpu <= tol and 0 <= err <= e_cpu + tol
        worst = _max_over_ranks(err if err >= 0 else 1e30)
        res["max_rel_err"] = worst
        res["tolerance"] = tol
        res["parity"] = bool(_max_over_ranks(0.0 if ok else 1.0) == 0.0)
    return res


def gemv_case(size, seed=4, iters=50, check=True):
    k = size
    row0, m = shard.gemv_shard(size, SHARD_WORLD, RANK)   # this rank's rows: its own column-major block
    th = gen_threads()
    # column-major m x k with lda = m: k rows of m values; every row shard is its own tensor
    a = synth.rows(seed, 16 + row0 // 64, F32, 0, k, m, threads=th)
    x = synth.rows(seed, 10, F32, 0, 1, k).reshape(-1)
    y = synth.rows(seed, 11, F32, 0, (size + 127) // 128 * 128, 1).reshape(-1)[row0:row0 + m]
    y = np.ascontiguousarray(y)
    da, dx, dy = to_device(a, F32), to_device(x, F32), to_device(y, F32)
    out = torch.empty_like(dy)
    sets = replicate(copies_needed(m * k * 4), da, dx, dy, out)

    def fn(i):
        xa, xx, xy, xo = sets[i % len(sets)]
        api.gemv(F32, m, k, xa, xx, xy, 2.1, 2.1, out=xo)
    ms, copies = timed(fn, iters, len(sets))
    nbytes = size * k * 4 + WORLD * k * 4 + 2 * size * 4
    _, hbm, src = peaks()
    hbm *= WORLD
    gbs = nbytes / ms / 1e6
    res = {"config": f"sgemv {size}^2 fp32 col-major, alpha=beta=2.1", "n_gpus": WORLD, "ms": ms,
           "value": gbs, "unit": "GB/s", "partition": f"row split x{WORLD}, x replicated",
           "seed": seed, "l2": l2_note(copies),
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s",
                        "frac": gbs / hbm, "algorithmic_bytes": nbytes,
                        "peak_source": f"{src} copy bandwidth x {WORLD} GPU(s)"}}
    if check:
        import oracle as O
        threads = _checker_threads()
        want = O.gemv(F32, m, k, a.reshape(-1), x, y, 2.1, 2.1)
        got = out.cpu().numpy()
        same = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        err = O.max_rel_err(F32, got, want)
        res["checker"] = f"host routine order (oracle), all {m} rows per rank, {threads} threads"
        res["max_rel_err"] = _max_over_ranks(err if err >= 0 else 1e30)
        res["tolerance"] = 0.0
        res["bit_identical"] = bool(_max_over_ranks(0.0 if same else 1.0) == 0.0)
        res["parity"] = res["bit_identical"]
    return res


def dlrm_cases(total_batch, seed=4, iters=20, check=True, which=("fwd", "bwd")):
    m, k = 27, 128
    out_len = k + m * (m - 1) // 2
    first, batch = shard.dlrm_shard(total_batch, SHARD_WORLD, RANK)   # this rank's samples
    assert first % synth.CHUNK_ROWS == 0
    th = gen_threads()
    x = synth.rows(seed, 1, F16, first, batch, m * k, dist="normal", threads=th)
    up = synth.rows(seed, 2, F16, first, batch, out_len, dist="normal", threads=th)
    dx, dup = to_device(x, F16), to_device(up, F16)
    out = torch.empty(batch * out_len, device="cuda", dtype=torch.float16)
    grad = torch.empty(batch * m * k, device="cuda", dtype=torch.float16)
    mlp = torch.empty(batch * k, device="cuda", dtype=torch.float16)
    _, hbm, src = peaks()
    hbm *= WORLD
    res = []
    pick = np.unique(np.concatenate([np.arange(min(128, batch)),
                                     np.arange(max(0, batch - 128), batch)]))

    def entry(name, ms, copies, nb):
        gbs = nb / ms / 1e6
        return {"config": name, "n_gpus": WORLD, "ms": ms, "value": gbs, "unit": "GB/s",
                "partition": f"batch split x{WORLD}", "seed": seed,
                "l2": l2_note(copies),
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s",
                             "frac": gbs / hbm, "algorithmic_bytes": nb,
                             "peak_source": f"{src} copy bandwidth x {WORLD} GPU(s)"}}

    def record_parity(r, err, exact_ok=True):
        r["max_rel_err"] = _max_over_ranks(err if err >= 0 else 1e30)
        r["tolerance"] = 2e-3
        r["parity"] = bool(_max_over_ranks(0.0 if (0 <= err <= 2e-3 and exact_ok) else 1.0) == 0.0)

    if "fwd" in which:
        sets = replicate(copies_needed(batch * (m * k + out_len) * 2), dx, out)

        def fwd(i):
            xx, xo = sets[i % len(sets)]
            api.dlrm_fwd(xx, m, k, batch, out=xo)
        ms, copies = timed(fwd, iters, len(sets))
        del sets
        r = entry(f"dlrm fwd b={total_batch} 27x128 fp16", ms, copies,
                  total_batch * (m * k + out_len) * 2)
        if check:
            import oracle as O
            threads = _checker_threads()
            xs = np.ascontiguousarray(x[pick]).reshape(-1)
            want = O.dlrm_fwd(F16, xs, m, k, pick.size, use_ref=O.ref() is not None)
            got = out.view(batch, out_len)[torch.from_numpy(pick).cuda()].cpu().numpy().reshape(-1)
            r["checker"] = ("rocWMMA dlrm_fwd_CPU" if O.ref() is not None else "oracle port") + \
                f", {pick.size} samples per rank, {threads} threads"
            record_parity(r, O.max_rel_err(F16, got, want))
        res.append(r)
    if "bwd" in which:
        sets = replicate(copies_needed(batch * (2 * m * k + out_len + k) * 2), dx, dup, grad, mlp)

        def bwd(i):
            xx, xu, xg, xm = sets[i % len(sets)]
            api.dlrm_bwd(xx, xu, m, k, batch, grad=xg, mlp_grad=xm)
        ms, copies = timed(bwd, iters, len(sets))
        del sets
        r = entry(f"dlrm bwd b={total_batch} 27x128 fp16", ms, copies,
                  total_batch * (m * k + out_len + m * k + k) * 2)
        if check:
            import oracle as O
            threads = _checker_threads()
            xs = np.ascontiguousarray(x[pick]).reshape(-1)
            ups = np.ascontiguousarray(up[pick]).reshape(-1)
            wmlp, wgrad = O.dlrm_bwd(F16, xs, ups, m, k, pick.size, use_ref=O.ref() is not None)
            sel = torch.from_numpy(pick).cuda()
            ggrad = grad.view(batch, m * k)[sel].cpu().numpy().reshape(-1)
            gmlp = mlp.view(batch, k)[sel].cpu().numpy().reshape(-1)
            r["checker"] = ("rocWMMA dlrm_bwd_CPU" if O.ref() is not None else "oracle port") + \
                f", {pick.size} samples per rank, {threads} threads"
            record_parity(r, O.max_rel_err(F16, ggrad, wgrad),
                    bool(np.array_equal(gmlp.view(np.uint16), wmlp.view(np.uint16))))
        res.append(r)
    return res


def case_table(small=False, iters=0, check=True):
    big, mid = (2048, 2048) if small else (8192, 4096)
    it = (lambda d: iters or d)
    return {
        "simple_hgemm": lambda: gemm_case("simple_hgemm 1024^3 f16->f32 16x16x16, alpha=1.5 beta=0.5",
                                          F16, F32, 1024, 1.5, 0.5, 0, 1.0, simple=True,
                                          iters=it(20), check=check),
        "hgemm": lambda: gemm_case(f"perf_hgemm {big}^3 f16->f16, alpha=1 beta=0", F16, F16, big,
                                   1.0, 0.0, 1, 1.0, iters=it(20), check=check),
        "bf16": lambda: gemm_case(f"gemm {mid}^3 bf16->f32, alpha=2 beta=-1", BF16, F32, mid, 2.0,
                                  -1.0, 2, 1.0, iters=it(20), check=check),
        "xf32": lambda: gemm_case(f"gemm {mid}^3 xf32->f32, alpha=2 beta=-1", XF32, F32, mid, 2.0,
                                  -1.0, 2, 0.5, iters=it(20), check=check),
        "f32": lambda: gemm_case(f"gemm {mid}^3 f32->f32 (3 x TF32), alpha=2 beta=-1", F32, F32,
                                 mid, 2.0, -1.0, 2, 0.5 / 3, iters=it(10), check=check),
        "f64": lambda: gemm_case(f"gemm {mid}^3 f64 (DMMA), alpha=2 beta=-1", F64, F64, mid, 2.0,
                                 -1.0, 2, None, iters=it(5), check=check),
        "i8": lambda: gemm_case(f"gemm {big}^3 i8->i32", I8, I32, big, 1, 0, 3, 2.0, iters=it(20),
                                check=check),
        "fp8": lambda: gemm_case(f"gemm {big}^3 e4m3->bf16", E4M3, BF16, big, 1.0, 0.0, 3, 2.0,
                                 iters=it(20), check=check),
        "bf8": lambda: gemm_case(f"gemm {big}^3 e5m2->bf16", E5M2, BF16, big, 1.0, 0.0, 3, 2.0,
                                 iters=it(20), check=check),
        "sgemv": lambda: gemv_case(8192 if small else 16384, iters=it(50), check=check),
        "dlrm_fwd": lambda: dlrm_cases(8192 if small else 65536, iters=it(20), check=check,
                                       which=("fwd",)),
        "dlrm_bwd": lambda: dlrm_cases(8192 if small else 65536, iters=it(20), check=check,
                                       which=("bwd",)),
    }


# what bench.py attaches to its line: everything but the headline configuration
EXTRAS = ["simple_hgemm", "bf16", "xf32", "f32", "f64", "i8", "fp8", "bf8", "dlrm_fwd", "dlrm_bwd",
          "sgemv"]


def run_all(names=None, small=False, iters=0, check=True, keep_gemm=False):
    """Runs the named configurations (default: EXTRAS) on the current device / rank and returns
    their result dictionaries (identical on every rank)."""
    table = case_table(small, iters, check)
    out = []
    for name in (names or EXTRAS):
        res = table[name]()
        for r in (res if isinstance(res, list) else [res]):
            if not keep_gemm:
                r = {k: v for k, v in r.items() if k != "gemm"}
            out.append(r)
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=0)
    ap.add_argument("--csv", default="", help="also write the GEMM results as a rocWMMA-style table")
    ap.add_argument("--no-check", action="store_true", help="timing only (no CPU parity check)")
    ap.add_argument("--as-shard-of", type=int, default=0,
                    help="run rank 0's share of an N-rank job in this single process (GEMM "
                         "figures then count the shard's rows only)")
    ap.add_argument("--small", action="store_true",
                    help="reduced sizes (for profiler captures): GEMMs 2048^3, DLRM b=8192, "
                         "GEMV 8192^2")
    args = ap.parse_args()
    if args.as_shard_of > 1:
        assert WORLD == 1, "--as-shard-of is for single-process runs"
        global SHARD_WORLD
        SHARD_WORLD = args.as_shard_of
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if WORLD > 1:
        torch.distributed.init_process_group("nccl")
    only = []
    for name in filter(None, args.only.split(",")):
        only += ["dlrm_fwd", "dlrm_bwd"] if name == "dlrm" else [name]
    names = only or (["hgemm"] + EXTRAS)
    rows = []
    for r in run_all(names, args.small, args.iters, not args.no_check, keep_gemm=True):
        if "gemm" in r:
            rows.append(csv_row(r))
            r = {k: v for k, v in r.items() if k != "gemm"}
        if RANK == 0:
            print(json.dumps(r), flush=True)
    if args.csv and RANK == 0:
        with open(args.csv, "w") as f:
            f.write(CSV_HEADER + "\n" + "\n".join(rows) + "\n")
    if WORLD > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
