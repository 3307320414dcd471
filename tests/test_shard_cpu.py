"""Multi-GPU host logic on CPU ranks (gloo, world size 2): the shards tile the problem,
each rank regenerates exactly its rows, and the gathered per-rank results equal the
single-rank result.  The per-rank computation here is the CPU oracle -- this tests the
partitioning and the reductions, not the kernels."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rocwmma_b200 import shard, synth


def test_ranges_tile_the_problem():
    for total, world, align in [(8192, 8, 128), (8192, 3, 128), (65536, 8, 8), (1000, 4, 8),
                                (100, 8, 128)]:
        covered = 0
        for r in range(world):
            first, count = shard.row_range(total, world, r, align)
            assert first == covered or count == 0
            assert first % align == 0 or count == 0
            covered += count
        assert covered == total


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, n, k, seed = 512, 96, 160, 17
    row0, rows = shard.gemm_shard(m, world, rank)
    a = synth.rows(seed, 1, synth.F16, row0, rows, k).reshape(-1)
    bt = synth.matrix(seed, 2, synth.F16, n, k)            # replicated
    c = np.zeros(rows * n, np.float16)
    d = O.gemm(O.F16, O.F16, rows, n, k, a, bt, c, 1.0, 0.0)
    parts = [torch.empty(shard.gemm_shard(m, world, r)[1] * n, dtype=torch.float16)
             for r in range(world)]
    dist.all_gather(parts, torch.from_numpy(d))
    slowest = shard.max_over_ranks(float(rank + 1))
    # DLRM: batch split
    b0, bn = shard.dlrm_shard(48, world, rank)
    x = synth.rows(seed, 3, synth.F16, 0, 48, 5 * 16, dist="normal")[b0:b0 + bn].reshape(-1)
    fwd = O.dlrm_fwd(O.F16, np.ascontiguousarray(x), 5, 16, bn)
    fparts = [torch.empty(shard.dlrm_shard(48, world, r)[1] * 26, dtype=torch.float16)
              for r in range(world)]
    dist.all_gather(fparts, torch.from_numpy(fwd))
    if rank == 0:
        np.save(os.path.join(out_dir, "d.npy"), torch.cat(parts).numpy())
        np.save(os.path.join(out_dir, "f.npy"), torch.cat(fparts).numpy())
        np.save(os.path.join(out_dir, "t.npy"), np.array([slowest]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_result(tmp_path):
    import oracle as O
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    m, n, k, seed = 512, 96, 160, 17
    a = synth.matrix(seed, 1, synth.F16, m, k)
    bt = synth.matrix(seed, 2, synth.F16, n, k)
    want = O.gemm(O.F16, O.F16, m, n, k, a, bt, np.zeros(m * n, np.float16), 1.0, 0.0)
    got = np.load(tmp_path / "d.npy")
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    x = synth.rows(seed, 3, synth.F16, 0, 48, 5 * 16, dist="normal").reshape(-1)
    wantf = O.dlrm_fwd(O.F16, x, 5, 16, 48)
    assert np.array_equal(np.load(tmp_path / "f.npy").view(np.uint16), wantf.view(np.uint16))
    assert np.load(tmp_path / "t.npy")[0] == 2.0      # max over ranks of (rank + 1)
