"""Regenerates the golden vectors in this directory.  Needs the rocWMMA source tree
(oracle.reference_dir(): the environment variable ROCWMMA_REFERENCE_DIR or the default
mount point); the tree is NOT needed to run the tests.

    python tests/golden/make_golden.py

1. dlrm_reference_fixture.npz -- a prefix of the reference's own stored
   known-answer vectors for the DLRM dot interaction (rocWMMA test/dlrm/data/*:
   m = 27, k = 128, batch = 64, raw little-endian arrays): the first 4 samples of
   the fp16 set and the first 2 of the fp32 set.
2. gemm_ref_outputs.npz / gemv_ref_outputs.npz / dlrm_ref_outputs.npz -- outputs
   of the reference's own host functions (gemm_CPU, sgemv_cpu_h, dlrm_*_CPU,
   compiled from the reference sources into oracle/_ref/libref.so) on this
   repository's seeded synthetic inputs.  Only outputs are stored; the tests
   regenerate the inputs from the same seeds.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle as O  # noqa: E402
from rocwmma_b200 import synth  # noqa: E402
from tests.cases import GEMM_GOLDEN_CASES, gemm_inputs, gemv_inputs, dlrm_inputs  # noqa: E402

REF_DATA = os.path.join(O.reference_dir(), "test", "dlrm", "data")
M, K, B = 27, 128, 64
OUT = K + M * (M - 1) // 2


def dlrm_fixture():
    keep = {"fp16": (np.float16, 4), "fp32": (np.float32, 2)}
    out = {}
    for tag, (dt, nb) in keep.items():
        def rd(name, per):
            a = np.fromfile(os.path.join(REF_DATA, f"{name}_{tag}"), dtype=dt)
            assert a.size == B * per, (name, a.size)
            return a[: nb * per].copy()
        out[f"input_{tag}"] = rd("input", M * K)
        out[f"output_{tag}"] = rd("output", OUT)
        out[f"input_grad_{tag}"] = rd("input_grad", OUT)
        out[f"output_input_grad_{tag}"] = rd("output_input_grad", M * K)
        out[f"output_mlp_input_grad_{tag}"] = rd("output_mlp_input_grad", K)
    np.savez_compressed(os.path.join(HERE, "dlrm_reference_fixture.npz"), **out)


def gemm_outputs():
    assert O.ref() is not None, "oracle/_ref/libref.so missing (make -C oracle ref)"
    out = {}
    for name, case in GEMM_GOLDEN_CASES.items():
        a, b, c = gemm_inputs(case)
        d = O.ref_gemm(case["in_t"], case["out_t"], case["m"], case["n"], case["k"], a, b, c,
                       case["alpha"], case["beta"], case["la"], case["lb"],
                       comp_t=case.get("comp_t"))
        out[name] = d
    np.savez_compressed(os.path.join(HERE, "gemm_ref_outputs.npz"), **out)


def gemv_outputs():
    m, k = 256, 192
    a, x, y = gemv_inputs(m, k, seed=11)
    np.savez_compressed(os.path.join(HERE, "gemv_ref_outputs.npz"),
                        y=O.ref_sgemv(m, k, a, x, y, 2.1, 2.1))


def dlrm_outputs():
    m, k, b = 27, 128, 9
    x, up = dlrm_inputs(m, k, b, seed=4)
    fwd = O.dlrm_fwd(O.F16, x, m, k, b, use_ref=True)
    mlp, grad = O.dlrm_bwd(O.F16, x, up, m, k, b, use_ref=True)
    np.savez_compressed(os.path.join(HERE, "dlrm_ref_outputs.npz"), fwd=fwd, mlp=mlp, grad=grad)


if __name__ == "__main__":
    dlrm_fixture()
    gemm_outputs()
    gemv_outputs()
    dlrm_outputs()
    print("golden vectors written to", HERE)
