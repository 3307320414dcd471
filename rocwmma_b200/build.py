"""In-tree build of the CUDA libraries for sm_100a (nvcc, no JIT cache).

    python -m rocwmma_b200.build [--force]

Produces, next to this file:
    lib/libb200wmma.so        the product: kernels + C ABI (include/rocwmma_b200.h)
    lib/libb200wmma_test.so   device-API unit-test kernels used only by tests/
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "lib")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
         "-I", os.path.join(ROOT, "include"), "-I", CSRC]

PRODUCT = ["runtime.cu", "simple_gemm.cu", "simple_gemm_blockk.cu", "gemm_tcgen05.cu", "gemm_f64.cu", "gemv.cu", "dlrm.cu"]
TESTLIB = ["test_kernels.cu"]


def _deps():
    out = []
    for base, _, files in os.walk(os.path.join(ROOT, "include")):
        out += [os.path.join(base, f) for f in files]
    out += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    return out


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _compile(src, force, extra=()):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if force or _stale(obj, [path] + _deps()):
        cmd = [NVCC, *FLAGS, *extra, "-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def _link(objs, name, force):
    so = os.path.join(LIB, name)
    if force or _stale(so, objs):
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", so, *objs,
               "-Xcompiler", "-fPIC", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed for {name}:\n{r.stdout}\n{r.stderr}")
    return so


def build(force: bool = False, verbose: bool = False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    srcs = [s for s in PRODUCT + TESTLIB if os.path.exists(os.path.join(CSRC, s))]
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = dict(zip(srcs, ex.map(lambda s: _compile(s, force), srcs)))
    prod = _link([objs[s] for s in PRODUCT if s in objs], "libb200wmma.so", force)
    test = None
    if all(s in objs for s in TESTLIB):
        test = _link([objs[s] for s in TESTLIB], "libb200wmma_test.so", force)
    if verbose:
        print("built", prod, test)
    return prod, test


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
