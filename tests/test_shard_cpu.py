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


def test_pair_kernel_tile_schedule_hands_out_every_tile_once():
    """The CTA-pair GEMM's tile schedule (wide tile columns, then 128-wide ones that fill the
    last partial wave): every tile exactly once, for many grids and pair counts, and the
    busiest pair of a 4096^2 output carries less than the 4 wide tiles it had before."""
    import ctypes as C
    import os

    import numpy as np

    from rocwmma_b200 import _lib
    lib = C.CDLL(os.path.join(os.path.dirname(_lib.LIB_PATH), "libb200wmma_test.so"))
    fn = lib.b200wmma_test_tile_schedule
    fn.restype = C.c_int
    fn.argtypes = [C.c_uint32] * 7 + [C.c_void_p, C.c_void_p]

    def walk(tiles_m, wide, tail, pairs, band=16, bn=256, bn_tail=128):
        counts = np.zeros(tiles_m * (wide + tail), np.uint32)
        loads = np.zeros(pairs, np.uint32)
        total = fn(tiles_m, wide, tail, bn, bn_tail, band, pairs, counts.ctypes.data,
                   loads.ctypes.data)
        return total, counts, loads

    rng = np.random.default_rng(0)
    cases = [(16, 16, 0, 74), (16, 13, 6, 74), (32, 32, 0, 74), (1, 1, 0, 1), (3, 0, 5, 7),
             (16, 13, 6, 1), (5, 2, 1, 74)]
    cases += [(int(rng.integers(1, 40)), int(rng.integers(0, 20)), int(rng.integers(0, 9)),
               int(rng.integers(1, 80))) for _ in range(200)]
    for tiles_m, wide, tail, pairs in cases:
        if wide + tail == 0:
            continue
        total, counts, loads = walk(tiles_m, wide, tail, pairs, band=int(rng.integers(1, 20)))
        assert total == tiles_m * (wide + tail), (tiles_m, wide, tail, pairs, total)
        assert (counts == 1).all(), (tiles_m, wide, tail, pairs)
    # 4096^2 on 74 pairs: 256-wide tiles only -> 4 tiles on the busiest pair; 13 wide + 6 narrow
    # tile columns -> at most 3 wide + 1 narrow, or 2 wide + 3 narrow
    _, _, uniform = walk(16, 16, 0, 74)
    _, _, mixed = walk(16, 13, 6, 74)
    assert uniform.max() == 4 * 256
    assert mixed.max() <= 3 * 256 + 128 and mixed.sum() == 16 * (13 * 256 + 6 * 128)
