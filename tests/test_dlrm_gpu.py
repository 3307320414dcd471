"""Fused DLRM dot-interaction forward/backward through the C ABI against the reference's
stored known-answer vectors, stored reference outputs and the oracle."""
import os

import numpy as np
import pytest
import torch

import oracle as O
from rocwmma_b200 import api, synth
from tests.cases import dlrm_inputs
from tests.gpu_util import to_device

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _fwd(x, m, k, b):
    return api.dlrm_fwd(to_device(x, O.F16), m, k, b).cpu().numpy()


def _bwd(x, up, m, k, b):
    mlp, grad = api.dlrm_bwd(to_device(x, O.F16), to_device(up, O.F16), m, k, b)
    return mlp.cpu().numpy(), grad.cpu().numpy()


def test_reference_known_answer_vectors(golden_dir):
    f = np.load(os.path.join(golden_dir, "dlrm_reference_fixture.npz"))
    x, up = f["input_fp16"], f["input_grad_fp16"]
    b = x.size // (27 * 128)
    out = _fwd(x, 27, 128, b)
    assert 0 <= O.max_rel_err(O.F16, out, f["output_fp16"]) <= TOL
    mlp, grad = _bwd(x, up, 27, 128, b)
    assert np.array_equal(mlp.view(np.uint16), f["output_mlp_input_grad_fp16"].view(np.uint16))
    assert 0 <= O.max_rel_err(O.F16, grad, f["output_input_grad_fp16"]) <= TOL


def test_stored_reference_outputs(golden_dir):
    g = np.load(os.path.join(golden_dir, "dlrm_ref_outputs.npz"))
    x, up = dlrm_inputs(27, 128, 9, seed=4)       # 9 = one full group of 8 + a tail of 1
    assert 0 <= O.max_rel_err(O.F16, _fwd(x, 27, 128, 9), g["fwd"]) <= TOL
    mlp, grad = _bwd(x, up, 27, 128, 9)
    assert np.array_equal(mlp.view(np.uint16), g["mlp"].view(np.uint16))
    assert 0 <= O.max_rel_err(O.F16, grad, g["grad"]) <= TOL


@pytest.mark.parametrize("m,k,b", [(27, 128, 1), (27, 128, 7), (27, 128, 64), (27, 128, 1003),
                                   (32, 128, 64), (16, 64, 40), (5, 16, 17), (32, 256, 24),
                                   (2, 32, 8)])
def test_shapes_against_oracle(m, k, b):
    x, up = dlrm_inputs(m, k, b, seed=7)
    want = O.dlrm_fwd(O.F16, x, m, k, b)
    assert 0 <= O.max_rel_err(O.F16, _fwd(x, m, k, b), want) <= TOL
    wmlp, wgrad = O.dlrm_bwd(O.F16, x, up, m, k, b)
    mlp, grad = _bwd(x, up, m, k, b)
    assert np.array_equal(mlp.view(np.uint16), wmlp.view(np.uint16))
    assert 0 <= O.max_rel_err(O.F16, grad, wgrad) <= TOL


def test_config_batch_65536():
    """Full configuration: batch 65536, 27 x 128, inputs from the seeded host generator
    (seed 4: the values the CPU side regenerates for any range of samples).  Exact copies
    are checked everywhere, the products on 384 samples spread over the batch -- whole
    128-sample chunks at the start, in the middle and at the end, which also cover the
    first and last work groups of the launch."""
    m, k, b = 27, 128, 65536
    out_len = k + m * (m - 1) // 2
    x_host = synth.rows(4, 1, synth.F16, 0, b, m * k, dist="normal")
    up_host = synth.rows(4, 2, synth.F16, 0, b, out_len, dist="normal")
    x = torch.from_numpy(x_host).cuda().view(-1)
    up = torch.from_numpy(up_host).cuda().view(-1)
    out = api.dlrm_fwd(x, m, k, b)
    mlp, grad = api.dlrm_bwd(x, up, m, k, b)
    torch.cuda.synchronize()
    api.check_device()
    assert torch.equal(out.view(b, out_len)[:, :k], x.view(b, m, k)[:, 0, :])
    assert torch.equal(mlp.view(b, k), up.view(b, out_len)[:, :k])
    for first in (0, 32768 - 64, b - 128):
        n = 128
        xs = np.ascontiguousarray(x_host[first:first + n]).reshape(-1)
        ups = np.ascontiguousarray(up_host[first:first + n]).reshape(-1)
        want = O.dlrm_fwd(O.F16, xs, m, k, n)
        got = out.view(b, out_len)[first:first + n].cpu().numpy().reshape(-1)
        assert 0 <= O.max_rel_err(O.F16, got, want) <= TOL, first
        _, wgrad = O.dlrm_bwd(O.F16, xs, ups, m, k, n)
        ggrad = grad.view(b, m * k)[first:first + n].cpu().numpy().reshape(-1)
        assert 0 <= O.max_rel_err(O.F16, ggrad, wgrad) <= TOL, first
    assert torch.isfinite(out.float()).all() and torch.isfinite(grad.float()).all()


def test_many_launches_back_to_back():
    """The kernels of one stream share one work counter and leave it at zero themselves
    (nothing clears it between launches), and consecutive launches overlap their set-up with
    the previous kernel's tail: 150 forward / backward launches back to back on one stream,
    alternating two batch sizes (so the number of tickets drawn per launch changes), must all
    give the oracle's result."""
    m, k = 27, 128
    cases = []
    for b, seed in ((1003, 21), (72, 22)):
        x, up = dlrm_inputs(m, k, b, seed=seed)
        cases.append((b, to_device(x, O.F16), to_device(up, O.F16), O.dlrm_fwd(O.F16, x, m, k, b),
                      O.dlrm_bwd(O.F16, x, up, m, k, b)))
    results = []
    for i in range(75):
        b, dx, dup, _, _ = cases[i % 2]
        results.append((i % 2, api.dlrm_fwd(dx, m, k, b), api.dlrm_bwd(dx, dup, m, k, b)))
    api.check_device()
    for which, out, (mlp, grad) in results:
        _, _, _, want_fwd, (want_mlp, want_grad) = cases[which]
        assert O.max_rel_err(O.F16, out.cpu().numpy().reshape(-1), want_fwd) <= 2e-3
        assert np.array_equal(mlp.cpu().numpy().reshape(-1).view(np.uint16),
                              np.asarray(want_mlp).reshape(-1).view(np.uint16))
        assert O.max_rel_err(O.F16, grad.cpu().numpy().reshape(-1), want_grad) <= 2e-3
