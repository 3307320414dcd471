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


def test_pair_kernel_tile_order_snake_and_mirror():
    """Tile order of the CTA-pair GEMM.  snake: odd bands of tile rows walk their columns right
    to left, so a band begins where the band before it ended.  mirror: the exact reverse
    sequence, so a launch begins on the tiles the launch before it ended on.  Either way
    every tile is handed out exactly once."""
    import ctypes as C
    import os

    import numpy as np

    from rocwmma_b200 import _lib
    lib = C.CDLL(os.path.join(os.path.dirname(_lib.LIB_PATH), "libb200wmma_test.so"))
    fn = lib.b200wmma_test_tile_order
    fn.restype = C.c_int
    fn.argtypes = [C.c_uint32] * 7 + [C.c_void_p]

    def order(tiles_m, cols, band, pairs, snake, mirror):
        seq = np.full(tiles_m * cols, 0xFFFFFFFF, np.uint32)
        assert fn(tiles_m, cols, 256, band, pairs, snake, mirror, seq.ctypes.data) == tiles_m * cols
        assert sorted(seq.tolist()) == list(range(tiles_m * cols))      # a permutation
        return seq.reshape(tiles_m, cols).astype(np.int64)

    rng = np.random.default_rng(1)
    shapes = [(32, 32, 8, 74), (4, 37, 8, 74), (16, 16, 16, 74), (5, 3, 2, 7), (1, 9, 4, 3)]
    shapes += [(int(rng.integers(1, 40)), int(rng.integers(1, 40)), int(rng.integers(1, 20)),
                int(rng.integers(1, 80))) for _ in range(50)]
    for tiles_m, cols, band, pairs in shapes:
        plain = order(tiles_m, cols, band, pairs, 0, 0)
        snake = order(tiles_m, cols, band, pairs, 1, 0)
        total = tiles_m * cols
        # mirror = the same tiles at positions counted from the end
        assert np.array_equal(order(tiles_m, cols, band, pairs, 0, 1), total - 1 - plain)
        assert np.array_equal(order(tiles_m, cols, band, pairs, 1, 1), total - 1 - snake)
        for g, r0 in enumerate(range(0, tiles_m, band)):
            rows = slice(r0, min(tiles_m, r0 + band))
            if g % 2 == 0:
                assert np.array_equal(snake[rows], plain[rows])
            else:       # odd band: same positions, columns reversed
                assert np.array_equal(snake[rows], plain[rows][:, ::-1])
        # consecutive bands meet on the same column under snake order
        for g in range(1, -(-tiles_m // band)):
            last_prev = np.unravel_index(np.argmax(np.where(
                np.arange(tiles_m)[:, None] // band == g - 1, snake, -1)), snake.shape)
            first_next = np.unravel_index(np.argmin(np.where(
                np.arange(tiles_m)[:, None] // band == g, snake, total)), snake.shape)
            assert last_prev[1] == first_next[1]


def _oracle_compute(in_t, out_t, n, k):
    """Stands in for the GEMM launch of ShardedHostGemm on CPU ranks: the CPU oracle on the
    rank's rows and the gathered B."""
    import oracle as O

    def compute(m_local, a, b, c, d, alpha, beta):
        cc = c.numpy() if c is not None else np.zeros(m_local * n, np.float16)
        res = O.gemm(in_t, out_t, m_local, n, k, a.numpy()[:m_local * k], b.numpy(),
                     cc[:m_local * n], alpha, beta)
        d[:m_local * n] = torch.from_numpy(res)
    return compute


def _sharded_host_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, n, k, seed = 512, 128, 96, 23
    op = shard.ShardedHostGemm(synth.F16, synth.F16, m, n, k, device="cpu",
                               compute=_oracle_compute(synth.F16, synth.F16, n, k))
    row0, rows = shard.gemm_shard(m, world, rank)
    assert (op.row0, op.m_local) == (row0, rows) and op.n_slab == n // world
    a_rows = torch.from_numpy(synth.rows(seed, 1, synth.F16, row0, rows, k))
    b_all = synth.rows(seed, 2, synth.F16, 0, n, k)
    b_slab = torch.from_numpy(b_all[rank * op.n_slab:(rank + 1) * op.n_slab].copy())
    c_rows = torch.from_numpy(synth.rows(seed, 3, synth.F16, row0, rows, n))
    d_rows = torch.zeros(rows, n, dtype=torch.float16)
    for alpha, beta, tag in ((1.0, 0.0, "d0"), (1.5, -0.5, "d1")):   # second call reuses buffers
        op(a_rows, b_slab, c_rows if beta != 0 else None, d_rows, alpha, beta)
        # every rank now holds all of B although it supplied only its slab
        assert np.array_equal(op.b_dev.numpy().view(np.uint16), b_all.reshape(-1).view(np.uint16))
        parts = [torch.empty(shard.gemm_shard(m, world, r)[1] * n, dtype=torch.float16)
                 for r in range(world)]
        dist.all_gather(parts, d_rows.reshape(-1).clone())
        if rank == 0:
            np.save(os.path.join(out_dir, tag + ".npy"), torch.cat(parts).numpy())
    assert op.h2d_bytes == (rows * k + op.n_slab * k) * 2 and op.d2h_bytes == rows * n * 2
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_host_gemm_exchanges_b_slabs(tmp_path):
    """ShardedHostGemm on two gloo ranks: each rank supplies its rows of A and HALF of B; after
    the all-gather both hold all of B, and the gathered rows of D equal the single-rank result."""
    import oracle as O
    world = 2
    mp.spawn(_sharded_host_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world,
             join=True)
    m, n, k, seed = 512, 128, 96, 23
    a = synth.matrix(seed, 1, synth.F16, m, k)
    bt = synth.matrix(seed, 2, synth.F16, n, k)
    c = synth.matrix(seed, 3, synth.F16, m, n)
    for alpha, beta, tag in ((1.0, 0.0, "d0"), (1.5, -0.5, "d1")):
        want = O.gemm(O.F16, O.F16, m, n, k, a, bt, c, alpha, beta)
        got = np.load(tmp_path / (tag + ".npy"))
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), tag


def _leaving_worker(rank, world, port, out_dir):
    """Rank 1 completes step 0 and then leaves (between steps, nothing of its own in flight)
    without telling anyone; rank 0 must get an error out of its next step -- not hang -- and
    stay usable afterwards."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    m, n, k, seed = 256, 64, 32, 29
    op = shard.ShardedHostGemm(synth.F16, synth.F16, m, n, k, device="cpu",
                               compute=_oracle_compute(synth.F16, synth.F16, n, k))
    row0, rows = shard.gemm_shard(m, world, rank)
    a_rows = torch.from_numpy(synth.rows(seed, 1, synth.F16, row0, rows, k))
    b_all = synth.rows(seed, 2, synth.F16, 0, n, k)
    b_slab = torch.from_numpy(b_all[rank * op.n_slab:(rank + 1) * op.n_slab].copy())
    d_rows = torch.zeros(rows, n, dtype=torch.float16)
    op(a_rows, b_slab, None, d_rows, 1.0, 0.0)                  # step 0: everyone takes part
    first = d_rows.clone()
    if rank == 1:
        os._exit(0)                                             # leaves between steps
    status = "no error"
    try:
        op(a_rows, b_slab, None, d_rows, 1.0, 0.0)              # step 1: the peer is gone
    except Exception as e:                                      # noqa: BLE001
        status = "error: " + type(e).__name__
    # the survivor is still usable: its own rows can be recomputed locally from the B it
    # gathered in step 0
    local = torch.zeros_like(d_rows)
    op.compute(rows, torch.from_numpy(a_rows.numpy().reshape(-1)), op.b_dev, None,
               local.reshape(-1), 1.0, 0.0)
    with open(os.path.join(out_dir, "status.txt"), "w") as f:
        f.write(status + "\n" + str(bool(torch.equal(local, first))))
    os._exit(0)     # no collective shutdown is possible without the peer


def test_a_rank_that_leaves_between_steps_is_reported_not_waited_for(tmp_path):
    world = 2
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, world, port, str(tmp_path)))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert not p.is_alive(), "a rank hung instead of reporting the missing peer"
    status, usable = open(tmp_path / "status.txt").read().split("\n")
    assert status.startswith("error"), status
    assert usable == "True"


def test_split_tiles_cover_k_exactly_once():
    """A launch whose last wave is less than half full cuts that wave's tiles in two along K
    (TileSchedule::splitTiles): every other tile is handed out once as a whole, every split
    tile as exactly its two halves, to two different pairs, and no pair carries more than one
    half-tile beyond the whole waves."""
    import ctypes as C
    import os

    import numpy as np

    from rocwmma_b200 import _lib
    lib = C.CDLL(os.path.join(os.path.dirname(_lib.LIB_PATH), "libb200wmma_test.so"))
    fn = lib.b200wmma_test_tile_split
    fn.restype = C.c_int
    fn.argtypes = [C.c_uint32] * 8 + [C.c_void_p] * 3
    rng = np.random.default_rng(5)
    cases = [(16, 16, 16, 74), (16, 16, 8, 74), (4, 20, 8, 74), (3, 27, 2, 74), (9, 9, 4, 37)]
    cases += [(int(rng.integers(1, 40)), int(rng.integers(1, 40)), int(rng.integers(1, 20)),
               int(rng.integers(2, 80))) for _ in range(100)]
    checked = 0
    for tiles_m, cols, band, pairs in cases:
        tiles = tiles_m * cols
        rem = tiles % pairs
        if tiles <= pairs or rem == 0 or 2 * rem > pairs:
            continue                      # the launcher would not split this one
        for snake, mirror in ((0, 0), (1, 0), (1, 1)):
            parts = np.zeros(tiles, np.uint32)
            whole = np.zeros(tiles, np.uint32)
            per_pair = np.zeros(pairs, np.uint32)
            total = fn(tiles_m, cols, 256, band, pairs, snake, mirror, rem, parts.ctypes.data,
                       whole.ctypes.data, per_pair.ctypes.data)
            assert total == tiles + rem, (tiles_m, cols, band, pairs, total)
            assert (whole + (parts == 3)).tolist() == [1] * tiles       # every tile covered once
            assert int((parts == 3).sum()) == rem and not ((parts != 0) & (parts != 3)).any()
            assert not ((whole != 0) & (parts != 0)).any()
            # whole waves for everybody, then at most one half
            assert per_pair.max() - per_pair.min() <= 1
            assert per_pair.max() == 2 * (tiles // pairs) + 1
            checked += 1
    assert checked >= 30
