"""ShardedHostGemm on two GPUs (one process each, NCCL): rows of A and half of B per rank
from pinned host memory, B slabs exchanged over NVLink, rows of D back; the gathered result
is compared with the CPU oracle.  Needs two GPUs: skipped on a single-GPU box."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

M, N, K, SEED = 1024, 512, 384, 31


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    from rocwmma_b200 import api, shard, synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    op = shard.ShardedHostGemm(synth.F16, synth.F16, M, N, K)
    row0, rows = shard.gemm_shard(M, world, rank)
    slab = N // world
    a = torch.from_numpy(synth.rows(SEED, 1, synth.F16, row0, rows, K)).pin_memory()
    b = torch.from_numpy(synth.rows(SEED, 2, synth.F16, 0, N, K)[rank * slab:(rank + 1) * slab]
                         .copy()).pin_memory()
    c = torch.from_numpy(synth.rows(SEED, 3, synth.F16, row0, rows, N)).pin_memory()
    d = torch.zeros(rows, N, dtype=torch.float16).pin_memory()
    for alpha, beta, tag in ((1.0, 0.0, "d0"), (1.5, -0.5, "d1")):
        d.fill_(float("nan"))
        op(a, b, c if beta != 0 else None, d, alpha, beta)
        np.save(os.path.join(out_dir, f"{tag}_{rank}.npy"), d.numpy())
    api.check_device()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_host_gemm_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    import oracle as O
    from rocwmma_b200 import synth
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    a = synth.matrix(SEED, 1, synth.F16, M, K)
    bt = synth.matrix(SEED, 2, synth.F16, N, K)
    c = synth.matrix(SEED, 3, synth.F16, M, N)
    for alpha, beta, tag in ((1.0, 0.0, "d0"), (1.5, -0.5, "d1")):
        want = O.gemm(O.F16, O.F16, M, N, K, a, bt, c, alpha, beta)
        got = np.concatenate([np.load(tmp_path / f"{tag}_{r}.npy").reshape(-1)
                              for r in range(world)])
        err = O.max_rel_err(O.F16, got, want)
        assert 0 <= err <= 2e-3, (tag, err)
