"""GEMV through the C ABI against the oracle and the stored reference output.

The kernel adds each row's products in the host routine's order with the same two
roundings per term, so fp32 and fp64 results are required to be bit-identical."""
import os

import numpy as np
import pytest

import oracle as O
from rocwmma_b200 import api, synth
from tests.cases import gemv_inputs
from tests.gpu_util import to_device

pytestmark = pytest.mark.gpu


def test_gemv_against_stored_reference_output(golden_dir):
    want = np.load(os.path.join(golden_dir, "gemv_ref_outputs.npz"))["y"]
    a, x, y = gemv_inputs(256, 192, seed=11)
    got = api.gemv(O.F32, 256, 192, to_device(a, O.F32), to_device(x, O.F32), to_device(y, O.F32),
                   2.1, 2.1).cpu().numpy()
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,k", [(256, 256), (1000, 333), (4096, 4096), (3, 5), (8192, 100),
                                 (64, 1), (65, 33), (1026, 2050)])
def test_sgemv_sizes(m, k):
    a, x, y = gemv_inputs(m, k, seed=12)
    want = O.gemv(O.F32, m, k, a, x, y, 2.1, 2.1)
    got = api.gemv(O.F32, m, k, to_device(a, O.F32), to_device(x, O.F32), to_device(y, O.F32), 2.1,
                   2.1).cpu().numpy()
    api.check_device()
    assert np.array_equal(got, want)


def test_dgemv_and_padded_lda():
    m, k, lda = 500, 300, 512
    rng = np.random.default_rng(2)
    A = rng.uniform(-1, 1, (k, m))
    a = np.zeros((k, lda)); a[:, :m] = A
    x = rng.uniform(-1, 1, k); y = rng.uniform(-1, 1, m)
    want = O.gemv(O.F64, m, k, a.reshape(-1), x, y, 2.1, -0.5, lda=lda)
    got = api.gemv(O.F64, m, k, to_device(a.reshape(-1), O.F64), to_device(x, O.F64),
                   to_device(y, O.F64), 2.1, -0.5, lda=lda).cpu().numpy()
    assert np.array_equal(got, want)


def test_config_sgemv_16384():
    m = k = 16384
    a, x, y = gemv_inputs(m, k, seed=4)
    want = O.gemv(O.F32, m, k, a, x, y, 2.1, 2.1)
    got = api.gemv(O.F32, m, k, to_device(a, O.F32), to_device(x, O.F32), to_device(y, O.F32), 2.1,
                   2.1).cpu().numpy()
    api.check_device()
    assert np.array_equal(got, want)


@pytest.mark.parametrize("form", ["chain", "single"])
@pytest.mark.parametrize("m,k", [(2048, 4100), (6144, 2048), (9472, 1024), (12000, 515)])
def test_sgemv_both_forms_at_every_block_count(form, m, k, monkeypatch):
    """The two fp32 forms (adding warp fed by multiplier warps / one warp doing everything) are
    picked by the number of 32-row blocks; B200WMMA_GEMV_FORM forces one.  Forced, each must
    stay bit-identical to the host routine also where the other would run: one block per SM,
    two blocks per SM (a shallower ring), 64-row blocks -- on the first launch of each shape,
    when the copies of a ring land least in order."""
    monkeypatch.setenv("B200WMMA_GEMV_FORM", form)
    a, x, y = gemv_inputs(m, k, seed=13)
    want = O.gemv(O.F32, m, k, a, x, y, 2.1, 2.1)
    da, dx, dy = to_device(a, O.F32), to_device(x, O.F32), to_device(y, O.F32)
    for _ in range(3):
        got = api.gemv(O.F32, m, k, da, dx, dy, 2.1, 2.1).cpu().numpy()
        api.check_device()
        assert np.array_equal(got, want)
