"""The C++ test-and-bench driver (tests/harness/bench_harness.cpp) drives every kernel family of
the library through its C ABI, the way the reference's host programs drive their kernels
(samples/perf_hgemm.cpp:716-944, simple_sgemv.cpp:157-270, simple_dlrm.cpp:443-680): built with
g++ against include/rocwmma_b200.h, linked to libb200wmma.so and (for validation) liboracle.so;
it prints the reference's result table (test/gemm/gemm_kernel_base_impl.hpp:441-523) and
PASSED / FAILED."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "harness", "bench_harness.cpp")
OUT = os.path.join(ROOT, "tests", "harness", "_build", "bench_harness")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    if os.path.exists(OUT) and os.path.getmtime(OUT) > os.path.getmtime(SRC):
        return
    lib = os.path.join(ROOT, "rocwmma_b200", "lib")
    ora = os.path.join(ROOT, "oracle")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", SRC, "-o", OUT, f"-I{ROOT}/include",
           f"-I{CUDA}/include", f"-L{lib}", f"-L{ora}", f"-L{CUDA}/lib64", "-lb200wmma",
           "-loracle", "-lcudart", f"-Wl,-rpath,{lib}", f"-Wl,-rpath,{ora}",
           f"-Wl,-rpath,{CUDA}/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_harness_builds():
    """Compiles and links without a GPU: the header is plain C and self-contained."""
    _build()
    assert os.path.exists(OUT)


def test_harness_refuses_unknown_input_without_a_gpu():
    _build()
    assert subprocess.run([OUT], capture_output=True).returncode == 2
    assert subprocess.run([OUT, "gemm", "--in", "f4"], capture_output=True).returncode == 2


def _run(args):
    _build()
    r = subprocess.run([OUT, *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASSED" in r.stdout
    lines = r.stdout.strip().split("\n")
    return lines, json.loads(lines[-1])


GEMM_RUNS = [
    ["--m", "1024", "--n", "1024", "--k", "1024"],                                  # f16 -> f16
    ["--m", "7168", "--n", "7168", "--k", "512", "--check-rows", "256"],            # the sample's size
    ["--m", "300", "--n", "200", "--k", "136", "--alpha", "1.5", "--beta", "0"],    # ragged
    ["--layout-a", "col", "--layout-b", "row", "--m", "512", "--n", "384", "--k", "256"],
    ["--in", "bf16", "--out", "f32", "--m", "512", "--n", "512", "--k", "512", "--beta", "-1"],
    ["--in", "xf32", "--m", "512", "--n", "256", "--k", "384", "--beta", "-1"],
    ["--in", "f32", "--m", "256", "--n", "256", "--k", "256"],
    ["--in", "f64", "--m", "256", "--n", "384", "--k", "128", "--beta", "-1"],
    ["--in", "i8", "--m", "512", "--n", "512", "--k", "1024"],
    ["--in", "f8", "--out", "bf16", "--m", "512", "--n", "512", "--k", "1024", "--beta", "0"],
    ["--in", "bf8", "--out", "f32", "--m", "256", "--n", "512", "--k", "512", "--beta", "0"],
    ["--simple", "--in", "f16", "--out", "f32", "--m", "256", "--n", "256", "--k", "256",
     "--alpha", "1.5", "--beta", "0.5"],
    ["--simple", "--block", "32", "--block-k", "8", "--in", "bf16", "--out", "f32", "--m", "128",
     "--n", "128", "--k", "64"],
]


@pytest.mark.gpu
@pytest.mark.parametrize("args", GEMM_RUNS, ids=[" ".join(a) for a in GEMM_RUNS])
def test_harness_gemm(args):
    lines, summary = _run(["gemm", *args])
    header = [c.strip() for c in lines[0].split(",")]
    row = [c.strip() for c in lines[1].split(",")]
    assert header[:5] == ["TBlkX", "TBlkY", "BlkM", "BlkN", "BlkK"] and header[-1] == "Result"
    assert len(row) == len(header) and row[-1] == "PASSED"
    assert summary["kernel"] == "gemm" and 0 <= summary["max_rel_err"] <= summary["tolerance"]


@pytest.mark.gpu
@pytest.mark.parametrize("args", [["--m", "4096", "--k", "4096"], ["--m", "1000", "--k", "777"],
                                  ["--type", "f64", "--m", "512", "--k", "640"]])
def test_harness_gemv(args):
    _, summary = _run(["gemv", *args])
    assert summary["kernel"] == "gemv" and summary["bit_identical"] is True


@pytest.mark.gpu
@pytest.mark.parametrize("args", [["--batch", "1024"], ["--bwd", "--batch", "1024"],
                                  ["--m", "32", "--k", "64", "--batch", "100"],
                                  ["--bwd", "--batch", "4096", "--check-samples", "512"]])
def test_harness_dlrm(args):
    _, summary = _run(["dlrm", *args])
    assert summary["kernel"].startswith("dlrm_") and 0 <= summary["max_rel_err"] <= 2e-3
