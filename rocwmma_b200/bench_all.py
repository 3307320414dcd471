"""Per-configuration throughput of every kernel in the library, one JSON line each.

    python -m rocwmma_b200.bench_all [--only NAME[,NAME...]] [--iters N] [--small] [--csv FILE]

Covers the configurations the headline benchmark (bench.py at the repository root) does
not: the simple one-tile-per-warp GEMM, the precision sweep, the quantised GEMMs, GEMV
and the DLRM passes.  GEMMs report TFLOP/s = 2*M*N*K / time against the measured dense
bf16 peak scaled per type; GEMV and DLRM report algorithmic bytes / time against the
measured HBM copy bandwidth.  Inputs are random device tensors (timing only; parity is
the test-suite's job).  Timed with CUDA events over `iters` back-to-back launches after
3 warm-ups; working sets that do not exceed the 126 MB L2 are timed launch by launch with an
L2 flush (a 256 MiB read) in between.

Under torchrun (python -m torch.distributed.run --nproc-per-node N -m rocwmma_b200.bench_all)
every configuration is split over the N GPUs the way rocwmma_b200.shard says -- GEMM by rows
of A / C / D with B replicated, GEMV by rows, DLRM by batch; no collective in the timed region --
and the figures are whole-job totals over the slowest rank's time.

--csv FILE also writes the GEMM results as the table rocWMMA's GEMM test programs print
(header and row format: test/gemm/gemm_kernel_base_impl.hpp:441-523), which its plotting
script test/bin/GenBenchmarkPlots.py reads.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import api, shard
from ._lib import BF16, COL_MAJOR, E4M3, E5M2, F16, F32, F64, I8, I32, ROW_MAJOR, XF32

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


WORLD = int(os.environ.get("WORLD_SIZE", "1"))
RANK = int(os.environ.get("RANK", "0"))


def _barrier():
    if WORLD > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


L2_BYTES = 126 << 20
_flush = None


def timed(fn, iters, working_set=None):
    """Per-launch time in ms, the slowest rank's.  A working set larger than the L2 is timed
    as `iters` back-to-back launches between two device events; a smaller one (the 1024^3
    sample, a shard of a many-GPU run) would be served from L2, so every launch is then
    timed on its own with a 256 MiB buffer read in between."""
    global _flush
    for _ in range(3):
        fn()
    _barrier()
    if working_set is None or working_set > L2_BYTES:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        _barrier()
        total = e0.elapsed_time(e1)
    else:
        if _flush is None:
            _flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")   # 256 MiB
        pairs = []
        for i in range(iters):
            # evict by READING twice the L2's size: a written buffer would leave the L2 full
            # of dirty lines whose write-back the timed kernel then pays for
            _flush.sum()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            pairs.append((e0, e1))
        _barrier()
        total = sum(a.elapsed_time(b) for a, b in pairs)
    api.check_device()
    return shard.max_over_ranks(total, device="cuda") / iters


def rand(n, code):
    dev = "cuda"
    if code in (F16, BF16, F32, XF32, F64):
        t = torch.rand(n, device=dev, dtype=torch.float32) * 2 - 1
        if code == XF32:
            return (t.view(torch.int32) & -8192).view(torch.float32)
        return t.to(api.torch_dtype(code))
    if code == I8:
        return torch.randint(-128, 128, (n,), device=dev, dtype=torch.int8)
    if code == I32:
        return torch.randint(-100, 100, (n,), device=dev, dtype=torch.int32)
    if code == E4M3:
        return (torch.randn(n, device=dev) * 80).clamp(-448, 448).to(torch.float8_e4m3fn).view(
            torch.uint8)
    if code == E5M2:
        return (torch.randn(n, device=dev) * 80).to(torch.float8_e5m2).view(torch.uint8)
    raise ValueError(code)


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
    fields = [*tile, n, n, n, g["alpha"], n, n, g["beta"], n, n, "row_col_row_row",
              f"{_TYPE_NAME[g['in_t']]}_{_TYPE_NAME[g['out_t']]}_{_TYPE_NAME[comp]}",
              f"{r['ms']:.6f}", f"{2.0 * n ** 3 / 1e9:.3f}", f"{r['value']:.3f}",
              f"{100.0 * r['frac']:.2f}", "BENCH"]
    return ", ".join(str(f) for f in fields)


def gemm_case(name, in_t, out_t, size, alpha, beta, peak_scale, simple=False, iters=20):
    n = k = size
    _, m = shard.gemm_shard(size, WORLD, RANK)   # this rank's rows of A, C, D
    a, b = rand(m * k, in_t), rand(k * n, in_t)
    c = rand(m * n, out_t) if beta != 0 else None
    d = torch.empty(m * n, dtype=api.torch_dtype(out_t), device="cuda")
    if simple:
        fn = lambda: api.gemm_simple(in_t, out_t, m, n, k, a, b, c, alpha, beta, ROW_MAJOR,  # noqa
                                     COL_MAJOR, ROW_MAJOR, 16, out=d)
    else:
        fn = lambda: api.gemm(in_t, out_t, m, n, k, a, b, c, alpha, beta, out=d)  # noqa: E731
    ms = timed(fn, iters, (m * k + k * n) * a.element_size() + m * n * d.element_size())
    tf = 2.0 * size * n * k / ms / 1e9
    peak_bf16, _, src = peaks()
    peak = (peak_bf16 * peak_scale if peak_scale else 40.0) * WORLD
    return {"config": name, "n_gpus": WORLD, "ms": ms, "value": tf, "unit": "TFLOP/s",
            "bound": "tensor", "peak": peak, "frac": tf / peak,
            "gemm": {"in_t": in_t, "out_t": out_t, "size": size, "alpha": alpha, "beta": beta,
                     "simple": simple},
            "peak_source": (f"{src} bf16 peak x {peak_scale}" if peak_scale
                            else "nominal fp64 tensor 40 TFLOP/s")}


def gemv_case(size, iters=50):
    k = size
    _, m = shard.gemv_shard(size, WORLD, RANK)   # this rank's rows: its own column-major block
    a, x, y = rand(m * k, F32), rand(k, F32), rand(m, F32)
    out = torch.empty_like(y)
    ms = timed(lambda: api.gemv(F32, m, k, a, x, y, 2.1, 2.1, out=out), iters, m * k * 4)
    nbytes = size * k * 4 + WORLD * k * 4 + 2 * size * 4
    _, hbm, src = peaks()
    hbm *= WORLD
    gbs = nbytes / ms / 1e6
    return {"config": f"sgemv {size}^2 fp32 col-major", "n_gpus": WORLD, "ms": ms, "value": gbs,
            "unit": "GB/s",
            "bound": "hbm", "algorithmic_bytes": nbytes, "peak": hbm, "frac": gbs / hbm,
            "peak_source": f"{src} copy bandwidth"}


def dlrm_cases(total_batch, iters=20):
    m, k = 27, 128
    out_len = k + m * (m - 1) // 2
    _, batch = shard.dlrm_shard(total_batch, WORLD, RANK)   # this rank's samples
    x = torch.randn(batch * m * k, device="cuda").half()
    up = torch.randn(batch * out_len, device="cuda").half()
    out = torch.empty(batch * out_len, device="cuda", dtype=torch.float16)
    grad = torch.empty(batch * m * k, device="cuda", dtype=torch.float16)
    mlp = torch.empty(batch * k, device="cuda", dtype=torch.float16)
    _, hbm, src = peaks()
    hbm *= WORLD
    res = []
    ms = timed(lambda: api.dlrm_fwd(x, m, k, batch, out=out), iters, batch * m * k * 2)
    nb = total_batch * (m * k + out_len) * 2
    res.append({"config": f"dlrm fwd b={total_batch} 27x128 fp16", "n_gpus": WORLD, "ms": ms,
                "value": nb / ms / 1e6,
                "unit": "GB/s", "bound": "hbm", "algorithmic_bytes": nb, "peak": hbm,
                "frac": nb / ms / 1e6 / hbm, "peak_source": f"{src} copy bandwidth"})
    ms = timed(lambda: api.dlrm_bwd(x, up, m, k, batch, grad=grad, mlp_grad=mlp), iters,
               batch * m * k * 4)
    nb = total_batch * (m * k + out_len + m * k + k) * 2
    res.append({"config": f"dlrm bwd b={total_batch} 27x128 fp16", "n_gpus": WORLD, "ms": ms,
                "value": nb / ms / 1e6,
                "unit": "GB/s", "bound": "hbm", "algorithmic_bytes": nb, "peak": hbm,
                "frac": nb / ms / 1e6 / hbm, "peak_source": f"{src} copy bandwidth"})
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=0)
    ap.add_argument("--csv", default="", help="also write the GEMM results as a rocWMMA-style table")
    ap.add_argument("--small", action="store_true",
                    help="reduced sizes (for profiler captures): GEMMs 2048^3, DLRM b=8192, "
                         "GEMV 8192^2")
    args = ap.parse_args()
    if WORLD > 1:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        torch.distributed.init_process_group("nccl")
    only = set(filter(None, args.only.split(",")))
    big, mid = (2048, 2048) if args.small else (8192, 4096)
    it = (lambda d: args.iters or d)

    cases = {
        "simple_hgemm": lambda: gemm_case("simple_hgemm 1024^3 f16->f32 16x16x16", F16, F32, 1024,
                                          1.5, 0.5, 1.0, simple=True, iters=it(20)),
        "hgemm": lambda: gemm_case(f"perf_hgemm {big}^3 f16->f16", F16, F16, big, 1.0, 0.0, 1.0,
                                   iters=it(20)),
        "bf16": lambda: gemm_case(f"gemm {mid}^3 bf16->f32", BF16, F32, mid, 2.0, -1.0, 1.0,
                                  iters=it(20)),
        "xf32": lambda: gemm_case(f"gemm {mid}^3 xf32->f32", XF32, F32, mid, 2.0, -1.0, 0.5,
                                  iters=it(20)),
        "f32": lambda: gemm_case(f"gemm {mid}^3 f32 (3 x TF32)", F32, F32, mid, 2.0, -1.0, 0.5 / 3,
                                 iters=it(10)),
        "f64": lambda: gemm_case(f"gemm {mid}^3 f64", F64, F64, mid, 2.0, -1.0, None,
                                 iters=it(5)),
        "i8": lambda: gemm_case(f"gemm {big}^3 i8->i32", I8, I32, big, 1, 0, 2.0, iters=it(20)),
        "fp8": lambda: gemm_case(f"gemm {big}^3 e4m3->bf16", E4M3, BF16, big, 1.0, 0.0, 2.0,
                                 iters=it(20)),
        "bf8": lambda: gemm_case(f"gemm {big}^3 e5m2->bf16", E5M2, BF16, big, 1.0, 0.0, 2.0,
                                 iters=it(20)),
        "sgemv": lambda: gemv_case(8192 if args.small else 16384, iters=it(50)),
        "dlrm": lambda: dlrm_cases(8192 if args.small else 65536, iters=it(20)),
    }
    rows = []
    for name, fn in cases.items():
        if only and name not in only:
            continue
        res = fn()
        for r in (res if isinstance(res, list) else [res]):
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
