#!/usr/bin/env python
"""Headline benchmark: hgemm 8192^3 (fp16 A row-major, fp16 B col-major, fp32 accumulate,
fp16 D, alpha = 1, beta = 0) in TFLOP/s on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the block-cooperative GEMM over the whole problem.  With N > 1 the
rows of A and D are split evenly over the ranks (B replicated, no collective in the timed
region), so the total work is fixed: strong scaling.  Prints ONE JSON line on rank 0.

`value`    device-resident throughput: 2*M*N*K*K_steps / time of the K launches (CUDA events
           on the launching stream, max over ranks).  The K-step region is timed REGIONS
           times, each bracketed by a barrier and a device synchronisation; the line
           reports the median region (all of them are listed under `regions_ms_per_step`):
           at N = 8 a region lasts 2 ms, too short to stand alone.
`e2e`      the same metric with HOST buffers: at N = 1 through the C ABI's host-buffer entry
           point (b200wmma_gemm_host: pinned A, B -> device, kernel, D -> host); at N > 1
           through rocwmma_b200.shard.ShardedHostGemm: every rank uploads its rows of A and
           1/N of B, the B slabs are exchanged GPU to GPU (one NCCL all-gather over NVLink,
           inside this timed region, never inside the `value` region), kernel, rows of D ->
           host.
`roofline` tensor-bound: achieved TFLOP/s of the kernel against the measured dense bf16/fp16
           peak of this pool (MEASURED_PEAKS.json, burst figure: the kernel is timed alone).
`parity`   after timing, every rank recomputes a sample of ITS OWN rows of D on the CPU with
           the reference's host GEMM (oracle/_ref, else the oracle port) and compares; the
           line carries the worst relative error over the ranks, at every N.  A result out
           of tolerance makes the benchmark exit non-zero.
`cpu_baseline`  (N = 1) that host GEMM timed on a bounded sample of rows of the same
           problem, on all host cores (count stated).
`extras`   every other benchmark configuration (bench_configs.py): throughput, roofline
           fraction and parity per kernel, sharded the same way at N > 1.

--impl reference times only that CPU implementation, on the same config and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 8192
SEED = 1
WORKLOAD = ("perf_hgemm 8192^3: fp16 A row-major, fp16 B col-major, fp32 accumulate, fp16 D, "
            "alpha=1, beta=0")
METRIC = "hgemm 8192^3 TFLOP/s"
FALLBACK_PEAK_TFLOPS = 1590.0
REGIONS = 5          # timed regions of K steps each; the median one is reported
TOLERANCE = 2e-3     # fp16 inputs, fp32 accumulate: max |a-b| / (|a|+|b|+1)
# DRAM bytes per launch of the GEMM kernel (dram__bytes_read.sum + dram__bytes_write.sum of one
# profiler capture of the current kernel at that launch shape), keyed by the rows of A per
# launch.  Quoted in roofline.traffic -- a benchmark run does not measure it -- together with
# where it came from; launch shapes without a capture report null.
PROFILED_TRAFFIC = {
    # B's tiles are fetched "evict first": a lone cold launch re-reads them from DRAM (1.22 GB
    # without the mark) and is slower for it, launches back to back are 1.7 % faster
    8192: 1.968e9,   # 1.857 GB read + 0.110 GB written (algorithmic: 0.403 GB)
    1024: 0.160e9,   # 155.2 MB read + 4.7 MB written inside the kernel (algorithmic: 0.168 GB)
}
TRAFFIC_SOURCE = ("one ncu capture (--set full, --clock-control none) of a launch of this shape, "
                  "cold L2; quoted from the committed profiler summary, not measured by this run")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)", p
    except Exception:
        return FALLBACK_PEAK_TFLOPS, "fallback (no MEASURED_PEAKS.json)", {}


# The B200s this runs on are power-capped: a dense GEMM holds its top clock for roughly the
# first 100 ms and then settles 10-15 % lower, for the vendor library as for this kernel,
# which is why the measured peaks come as a burst and a sustained figure.  A timed region
# shorter than this is compared with the burst peak, a longer one with the sustained peak;
# both fractions are reported either way.
BURST_REGION_MS = 100.0


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs
    (read-only NVML queries)."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nvml
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)
        med = None
        if self.samples:
            s = sorted(self.samples)
            med = s[len(s) // 2]
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            pass
    return local_rank


def make_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "seed": SEED,
            "partition": f"M-split x{world}, B replicated", "rows_per_gpu": M // world,
            "l2": "per-GPU inputs (A rows + all of B >= 144 MiB) exceed the 126 MB L2; no flush",
            "timing": f"median of {REGIONS} regions of K steps, each between barrier + "
                      "synchronize; CUDA events on the launching stream, max over ranks"}


def cpu_reference_sample(rows_budget_s: float, a_rows_fn, bt, want_rows=None):
    """Times the reference's host GEMM on a sample of rows of the 8192^3 problem, on all
    host cores.  Returns (tflops, info, rows_idx, d_rows)."""
    import numpy as np

    import oracle as O
    use_ref = O.ref() is not None
    kind = "reference" if use_ref else "port"
    # all host cores, whatever OMP_NUM_THREADS this process inherited (torch.distributed.run
    # exports 1 to its workers)
    O.set_num_threads(O.host_cores())

    def run(a_rows):
        nrows = a_rows.shape[0]
        c0 = np.zeros(nrows * N, dtype=np.float16)
        t0 = time.perf_counter()
        if use_ref:
            d = O.ref_gemm(O.F16, O.F16, nrows, N, K, np.ascontiguousarray(a_rows).reshape(-1), bt,
                           c0, 1.0, 0.0)
        else:
            d = O.gemm(O.F16, O.F16, nrows, N, K, np.ascontiguousarray(a_rows).reshape(-1), bt, c0,
                       1.0, 0.0)
        return d, time.perf_counter() - t0

    threads = O.num_threads()
    probe_rows = max(threads, 8)
    _, t_probe = run(a_rows_fn(probe_rows))
    rate = probe_rows / max(t_probe, 1e-6)  # rows per second
    nrows = int(max(probe_rows, min(2048, rate * rows_budget_s)))
    nrows = max(threads, nrows // threads * threads)
    a_rows = a_rows_fn(nrows)
    d, t = run(a_rows)
    tflops = 2.0 * nrows * N * K / t / 1e12
    info = {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": f"first {nrows} rows of A x all of B ({nrows}x{N}x{K}), "
                      f"{t:.1f} s of {'rocWMMA gemm_CPU (OpenMP)' if use_ref else 'the oracle port'}"}
    return tflops, info, nrows, d


def run_reference_arm(args, rank, world):
    """--impl reference: the reference's own CPU GEMM for this path on the host cores."""
    if rank != 0:
        return
    import numpy as np

    from rocwmma_b200 import synth
    bt = synth.matrix(SEED, 2, synth.F16, N, K)
    a_cache = {}

    def a_rows(n):
        if n not in a_cache:
            a_cache[n] = synth.rows(SEED, 1, synth.F16, 0, (n + 127) // 128 * 128, K)[:n]
        return a_cache[n]

    # each step is a bounded sample; the whole run stays within a few minutes
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    budget = min(10.0, 120.0 / (steps + warmup))
    vals, info, rows = [], None, 0
    for i in range(warmup + steps):
        tf, info, rows, _ = cpu_reference_sample(budget, a_rows, bt)
        if i >= warmup:
            vals.append(tf)
    value = sum(vals) / len(vals)
    ms = 2.0 * rows * N * K / (value * 1e12) * 1e3
    info["value"] = value
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": make_config(max(1, args.gpus)),
            "cpu_baseline": info,
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def shard_parity(a_host, b_host, d_dev, d_host, m_local, world, rows_budget=24):
    """This rank recomputes a sample of its own rows of D with the reference's host GEMM and
    compares the device-resident result and the end-to-end (host-buffer) result with it.
    Returns (err_device, err_e2e, rows)."""
    import numpy as np

    import oracle as O
    O.set_num_threads(max(1, O.host_cores() // world))
    rng = np.random.default_rng(SEED * 100 + int(os.environ.get("RANK", "0")))
    pick = np.unique(np.concatenate([[0, 127, 128, m_local - 1],
                                     rng.integers(0, m_local, rows_budget)]))
    a_np = a_host.numpy()[pick]
    c0 = np.zeros(pick.size * N, dtype=np.float16)
    fn = O.ref_gemm if O.ref() is not None else O.gemm
    want = fn(O.F16, O.F16, pick.size, N, K, np.ascontiguousarray(a_np).reshape(-1),
              b_host.numpy().reshape(-1), c0, 1.0, 0.0)
    import torch
    sel = torch.from_numpy(pick).cuda()
    got = d_dev.view(m_local, N)[sel].cpu().numpy().reshape(-1)
    err_dev = O.max_rel_err(O.F16, got, want)
    err_e2e = O.max_rel_err(O.F16, np.ascontiguousarray(d_host.numpy()[pick]).reshape(-1), want)
    return err_dev, err_e2e, int(pick.size)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=None,
                    help="steps of the host-buffer measurement (default: min(steps, 10))")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations (bench_configs.py)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    from rocwmma_b200 import api, shard, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"
    assert M % (world * synth.CHUNK_ROWS) == 0 and N % world == 0

    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    row0, m_local = shard.gemm_shard(M, world, rank)
    try:
        gen_threads = max(1, min(16, len(os.sched_getaffinity(0)) // world))
    except AttributeError:
        gen_threads = 1

    # ---- synthetic inputs (seeded; every rank regenerates its own rows of A, all of B) ----
    a_host = torch.from_numpy(synth.rows(SEED, 1, synth.F16, row0, m_local, K,
                                         threads=gen_threads)).pin_memory()
    b_host = torch.from_numpy(synth.rows(SEED, 2, synth.F16, 0, N, K,
                                         threads=gen_threads)).pin_memory()
    d_host = torch.empty((m_local, N), dtype=torch.float16).pin_memory()
    a_dev = a_host.cuda(non_blocking=True)
    b_dev = b_host.cuda(non_blocking=True)
    d_dev = torch.empty(m_local * N, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        api.gemm(api.F16, api.F16, m_local, N, K, a_dev, b_dev, None, 1.0, 0.0, out=d_dev)

    stream = torch.cuda.current_stream()

    # ---- device-resident measurement: REGIONS regions of exactly `steps` launches ----
    for _ in range(warmup):
        step()
    api.check_device()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    region_ms, own_ms = [], []
    sampler.start()
    for _ in range(REGIONS):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        barrier()
        mine = e0.elapsed_time(e1)
        own_ms.append(mine)
        region_ms.append(shard.max_over_ranks(mine, device="cuda"))
    clocks = sampler.stop()
    api.check_device()
    ms_total = sorted(region_ms)[len(region_ms) // 2]
    # every rank's own median region, for the record (the figure above is the slowest rank's)
    per_rank = [sorted(own_ms)[len(own_ms) // 2] / steps]
    if world > 1:
        t = torch.tensor(per_rank, dtype=torch.float64, device="cuda")
        allr = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allr, t)
        per_rank = [float(x.item()) for x in allr]

    # ---- end to end with host buffers ----
    e2e_steps = args.e2e_steps if args.e2e_steps is not None else min(steps, 10)
    host_gemm = shard.ShardedHostGemm(api.F16, api.F16, M, N, K)
    if world == 1:
        b_part = b_host
    else:
        slab = N // world
        b_part = b_host[rank * slab:(rank + 1) * slab]      # a view of the pinned buffer

    def e2e_step():
        host_gemm(a_host, b_part, None, d_host, 1.0, 0.0)

    for _ in range(2):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    f1.record(stream)
    barrier()
    e2e_ms_total = shard.max_over_ranks(f0.elapsed_time(f1), device="cuda")

    flops = 2.0 * M * N * K
    ms_per_step = ms_total / steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    e2e_ms = e2e_ms_total / e2e_steps
    e2e_value = flops / (e2e_ms * 1e-3) / 1e12

    # ---- roofline of the dominant (only) kernel: this rank's launch ----
    peak, peak_src, peaks_json = measured_peaks()
    kernel_tflops = 2.0 * m_local * N * K / (ms_per_step * 1e-3) / 1e12
    burst_peak = peak
    sustained_peak = float(peaks_json.get("bf16_tflops_sustained", 0.0)) or None
    if sustained_peak and ms_total > BURST_REGION_MS:
        peak = sustained_peak
        peak_src = ("measured (MEASURED_PEAKS.json bf16_tflops_sustained: the timed region of "
                    f"{ms_total:.0f} ms is past the ~{BURST_REGION_MS:.0f} ms the power cap allows "
                    "at top clock)")
    roofline = {"bound": "tensor", "achieved": kernel_tflops, "peak": peak, "unit": "TFLOP/s",
                "frac": kernel_tflops / peak,
                "frac_of_burst_peak": kernel_tflops / burst_peak,
                "frac_of_sustained_peak": (kernel_tflops / sustained_peak
                                           if sustained_peak else None),
                "timed_region_ms": ms_total,
                "traffic": PROFILED_TRAFFIC.get(m_local),
                "traffic_source": (TRAFFIC_SOURCE if m_local in PROFILED_TRAFFIC
                                   else "not captured for this launch shape"),
                "peak_source": peak_src, "kernel": "gemm_tcgen05_pair_kernel<half,half,float>",
                "algorithmic_flops_per_launch": 2.0 * m_local * N * K}

    # ---- parity of every rank's shard (both results), worst over the ranks ----
    err_dev, err_e2e, rows_checked = shard_parity(a_host, b_host, d_dev, d_host, m_local, world)
    bad = 1e30
    worst_dev = shard.max_over_ranks(err_dev if err_dev >= 0 else bad, device="cuda")
    worst_e2e = shard.max_over_ranks(err_e2e if err_e2e >= 0 else bad, device="cuda")
    parity_ok = worst_dev <= TOLERANCE and worst_e2e <= TOLERANCE
    parity = {"max_rel_err": worst_dev, "e2e_max_rel_err": worst_e2e, "tolerance": TOLERANCE,
              "within_tolerance": bool(parity_ok), "rows_checked_per_rank": rows_checked,
              "ranks": world,
              "checker": "rocWMMA gemm_CPU on each rank's own rows (per-shard validation)"}

    # ---- CPU baseline (rank 0, N = 1 only) ----
    cpu_info = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        a_np, b_np = a_host.numpy(), b_host.numpy().reshape(-1)
        _, cpu_info, nrows, d_cpu = cpu_reference_sample(10.0, lambda n: a_np[:n], b_np)
        import oracle as O
        d_gpu = d_dev.view(m_local, N)[:nrows].cpu().numpy().reshape(-1)
        err = O.max_rel_err(O.F16, d_gpu, d_cpu)
        cpu_info["gpu_rows_checked"] = nrows
        cpu_info["gpu_max_rel_err"] = err
        cpu_info["gpu_within_tolerance_2e-3"] = bool(0 <= err <= TOLERANCE)
        cpu_info["e2e_rows_max_rel_err"] = O.max_rel_err(
            O.F16, d_host[:nrows].numpy().reshape(-1), d_cpu)
        parity_ok = parity_ok and 0 <= err <= TOLERANCE

    # ---- every other configuration ----
    extras = None
    if not args.no_extras:
        torch.cuda.empty_cache()
        import bench_configs
        extras = bench_configs.run_all()
        parity_ok = parity_ok and all(e.get("parity", True) for e in extras)

    if rank == 0:
        h2d = (a_host.numel() * 2 + b_part.numel() * 2)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": make_config(world),
            "regions_ms_per_step": [r / steps for r in region_ms],
            "per_rank_ms_per_step": per_rank,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "steps": e2e_steps,
                    "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d_host.numel() * 2),
                    "bytes_are": "per rank",
                    "call": ("b200wmma_gemm_host (pinned host buffers)" if world == 1 else
                             "rocwmma_b200.shard.ShardedHostGemm: rows of A + 1/N of B per rank "
                             "over PCIe, NCCL all-gather of the B slabs over NVLink inside this "
                             "region (not inside the `value` region), b200wmma_gemm, rows of D "
                             "back")},
            "gpu_launches": steps,
            "roofline": roofline,
            "parity": parity,
        }
        if cpu_info is not None:
            line["cpu_baseline"] = cpu_info
        if extras is not None:
            line["extras"] = extras
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit("bench.py: a result is out of tolerance against the CPU reference")


if __name__ == "__main__":
    main()
