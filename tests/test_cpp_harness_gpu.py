"""A C++ host program drives the library through its C ABI, the way the reference's sample
drivers drive their kernels (samples/perf_hgemm.cpp:716-944): built with g++ against
include/rocwmma_b200.h, linked to libb200wmma.so and (for validation) liboracle.so."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "harness", "gemm_harness.cpp")
OUT = os.path.join(ROOT, "tests", "harness", "_build", "gemm_harness")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    lib = os.path.join(ROOT, "rocwmma_b200", "lib")
    ora = os.path.join(ROOT, "oracle")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", SRC, "-o", OUT, f"-I{ROOT}/include",
           f"-I{CUDA}/include", f"-L{lib}", f"-L{ora}", f"-L{CUDA}/lib64", "-lb200wmma",
           "-loracle", "-lcudart", f"-Wl,-rpath,{lib}", f"-Wl,-rpath,{ora}",
           f"-Wl,-rpath,{CUDA}/lib64"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)


def test_harness_builds():
    """Compiles and links without a GPU: the header is plain C and self-contained."""
    _build()
    assert os.path.exists(OUT)


@pytest.mark.gpu
@pytest.mark.parametrize("args", [["1024", "1024", "1024", "2", "2"], ["7168", "7168", "512", "2", "2"],
                                  ["300", "200", "136", "1.5", "0"]])
def test_harness_runs_and_validates(args):
    _build()
    r = subprocess.run([OUT, *args], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASSED" in r.stdout
