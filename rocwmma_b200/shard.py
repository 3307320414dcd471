"""How the paths are split over the GPUs of one node.

Every path shards without an exchange step (no collective in the timed region):
GEMM by rows of A / C / D with B replicated, DLRM by batch, GEMV by rows.  A shard is
a contiguous range; ranges are aligned so that seeded inputs regenerate per shard
(rocwmma_b200.synth.CHUNK_ROWS) and so that packed DLRM rows stay 16-byte aligned.
"""
from __future__ import annotations

from .synth import CHUNK_ROWS


def row_range(total: int, world: int, rank: int, align: int = CHUNK_ROWS):
    """(first, count) of rank's contiguous share of `total` rows: equal shares rounded up to
    `align`, the last ranks may get fewer (or none)."""
    assert 0 <= rank < world
    per = -(-total // world)
    per = -(-per // align) * align
    first = min(total, rank * per)
    return first, max(0, min(per, total - first))


def gemm_shard(m: int, world: int, rank: int):
    """Rows of A, C and D owned by `rank` (B is replicated)."""
    return row_range(m, world, rank, CHUNK_ROWS)


def dlrm_shard(batch: int, world: int, rank: int):
    """Samples owned by `rank`; multiples of 8 keep the packed rows 16-byte aligned."""
    return row_range(batch, world, rank, 8)


def gemv_shard(m: int, world: int, rank: int):
    """Rows of A and y owned by `rank`; each rank holds its own column-major block with
    lda = its row count, x is replicated.  Multiples of 64 rows (one thread block's share)."""
    return row_range(m, world, rank, 64)


def max_over_ranks(value: float, device=None) -> float:
    """Slowest rank's time (torch.distributed must be initialised when world > 1)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class ShardedHostGemm:
    """D = alpha * A * B + beta * C with HOST buffers over the ranks of a torch.distributed job
    (one process per GPU): the multi-GPU form of api.gemm_host.

    Rank r owns rows gemm_shard(m, world, r) of A, C and D, and, for the way in, an equal
    slab of B (rows of the K-major [n][k] storage of a column-major B).  One call

      1. copies the rank's B slab from (pinned) host memory into its place in the rank's
         full-size device copy of B, and its rows of A (and C),
      2. exchanges the slabs GPU to GPU with one in-place NCCL all-gather over NVLink, so
         every rank ends up with all of B while each byte of B crossed PCIe only once in the
         whole job,
      3. runs the block-cooperative GEMM on the rank's rows (the kernel reads this GPU's own
         memory only),
      4. copies the rank's rows of D back to host memory and waits for them.

    The A / C upload is issued after the all-gather has been handed to NCCL, so it overlaps
    the exchange.  Device buffers are allocated once, in the constructor.  With world == 1
    this is api.gemm_host.  A row-major, B column-major (the K-major operand forms).
    """

    def __init__(self, in_t, out_t, m, n, k, rank=None, world=None, group=None, device=None,
                 compute=None):
        """device / compute exist for the host-logic tests, which run the exchange on CPU
        tensors over gloo: `device` is where the per-rank buffers live (default: the current
        CUDA device) and `compute(m_local, a, b, c, d, alpha, beta)` stands in for the GEMM
        launch (default: api.gemm).  The product path passes neither."""
        import torch
        import torch.distributed as dist

        from . import api
        self.api, self.torch, self.dist = api, torch, dist
        self.group = group
        self.compute = compute
        multi = dist.is_available() and dist.is_initialized()
        self.world = world if world is not None else (dist.get_world_size(group) if multi else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if multi else 0)
        self.in_t, self.out_t, self.m, self.n, self.k = in_t, out_t, m, n, k
        self.row0, self.m_local = gemm_shard(m, self.world, self.rank)
        if self.world > 1:
            if n % self.world:
                raise ValueError("n must divide by the number of ranks (equal B slabs)")
            self.n_slab = n // self.world
            dev = device if device is not None else torch.device("cuda",
                                                                   torch.cuda.current_device())
            self.device = torch.device(dev)
            tin, tout = api.torch_dtype(in_t), api.torch_dtype(out_t)
            self.b_dev = torch.empty(n * k, dtype=tin, device=dev)
            self.a_dev = torch.empty(max(1, self.m_local) * k, dtype=tin, device=dev)
            self.c_dev = None
            self.d_dev = torch.empty(max(1, self.m_local) * n, dtype=tout, device=dev)
            lo = self.rank * self.n_slab * k
            self.b_slab = self.b_dev[lo:lo + self.n_slab * k]
            self._streams = None
            self._events = None

    @property
    def h2d_bytes(self):
        """Bytes this rank uploads per call (beta == 0)."""
        e = self.api.torch_dtype(self.in_t).itemsize
        if self.world == 1:
            return (self.m * self.k + self.n * self.k) * e
        return (self.m_local * self.k + self.n_slab * self.k) * e

    @property
    def d2h_bytes(self):
        return self.m_local * self.n * self.api.torch_dtype(self.out_t).itemsize

    def __call__(self, a_rows, b_slab, c_rows, d_rows, alpha, beta):
        """a_rows: this rank's rows of A [m_local][k]; b_slab: this rank's slab of B
        [n / world][k] (all of B when world == 1); c_rows / d_rows: this rank's rows of
        C (None when beta == 0) and D [m_local][n].  Host tensors, ideally pinned.  Returns
        d_rows after the copy back has completed."""
        api, torch = self.api, self.torch
        if self.world == 1:
            return api.gemm_host(self.in_t, self.out_t, self.m, self.n, self.k, a_rows, b_slab,
                                 c_rows, d_rows, alpha, beta)
        for t in (a_rows, b_slab, c_rows, d_rows):
            if t is not None and t.is_cuda:
                raise ValueError("ShardedHostGemm takes host tensors")
        if beta != 0 and self.c_dev is None:
            self.c_dev = torch.empty_like(self.d_dev)
        if self.device.type != "cuda":
            return self._call_serial(a_rows, b_slab, c_rows, d_rows, alpha, beta)
        # Pipeline.  PCIe is the critical path (at 8 ranks the uploads of one step take
        # 1.4 ms and the rows of D as long again, against 0.24 ms for the exchange and 0.1 ms
        # for the kernel), and it is full duplex: B goes first, since every row of D needs all
        # of it; then the rank's rows travel in slabs -- A (and C) in on one copy stream, the
        # GEMM of a slab as soon as it has landed, its rows of D out on a second copy stream
        # while later slabs of A are still arriving.
        cur = torch.cuda.current_stream()
        if self._streams is None:
            self._streams = (torch.cuda.Stream(), torch.cuda.Stream())
            self._events = [torch.cuda.Event() for _ in range(2 * self.SLABS + 2)]
        h2d, d2h = self._streams
        ev = self._events
        h2d.wait_stream(cur)
        d2h.wait_stream(cur)
        with torch.cuda.stream(h2d):
            self.b_slab.copy_(b_slab.reshape(-1), non_blocking=True)
            ev[0].record(h2d)
        cur.wait_event(ev[0])
        work = self.dist.all_gather_into_tensor(self.b_dev, self.b_slab, group=self.group,
                                                async_op=True)
        rows_per = -(-self.m_local // self.SLABS)
        rows_per = -(-rows_per // 128) * 128
        slabs = [(r, min(rows_per, self.m_local - r)) for r in range(0, self.m_local, rows_per)]
        a_flat, d_flat = a_rows.reshape(-1), d_rows.reshape(-1)
        c_flat = c_rows.reshape(-1) if beta != 0 else None
        with torch.cuda.stream(h2d):
            for i, (r0, rows) in enumerate(slabs):
                self.a_dev[r0 * self.k:(r0 + rows) * self.k].copy_(
                    a_flat[r0 * self.k:(r0 + rows) * self.k], non_blocking=True)
                if beta != 0:
                    self.c_dev[r0 * self.n:(r0 + rows) * self.n].copy_(
                        c_flat[r0 * self.n:(r0 + rows) * self.n], non_blocking=True)
                ev[1 + i].record(h2d)
        work.wait()          # the current stream waits for the exchange; the host does not
        for i, (r0, rows) in enumerate(slabs):
            cur.wait_event(ev[1 + i])
            lo, hi = r0 * self.n, (r0 + rows) * self.n
            api.gemm(self.in_t, self.out_t, rows, self.n, self.k,
                     self.a_dev[r0 * self.k:(r0 + rows) * self.k], self.b_dev,
                     self.c_dev[lo:hi] if beta != 0 else None, alpha, beta,
                     out=self.d_dev[lo:hi])
            done = ev[1 + self.SLABS + i]
            done.record(cur)
            d2h.wait_event(done)
            with torch.cuda.stream(d2h):
                d_flat[lo:hi].copy_(self.d_dev[lo:hi], non_blocking=True)
        cur.wait_stream(d2h)
        d2h.synchronize()
        return d_rows

    SLABS = 4

    def _call_serial(self, a_rows, b_slab, c_rows, d_rows, alpha, beta):
        """The same steps one after the other (host-logic tests on CPU tensors)."""
        self.b_slab.copy_(b_slab.reshape(-1))
        self.dist.all_gather_into_tensor(self.b_dev, self.b_slab, group=self.group)
        if self.m_local:
            self.a_dev[:self.m_local * self.k].copy_(a_rows.reshape(-1))
            c_dev = None
            if beta != 0:
                self.c_dev[:self.m_local * self.n].copy_(c_rows.reshape(-1))
                c_dev = self.c_dev
            if self.compute is not None:
                self.compute(self.m_local, self.a_dev, self.b_dev, c_dev, self.d_dev, alpha, beta)
            else:
                self.api.gemm(self.in_t, self.out_t, self.m_local, self.n, self.k, self.a_dev,
                              self.b_dev, c_dev, alpha, beta, out=self.d_dev)
            d_rows.reshape(-1).copy_(self.d_dev[:self.m_local * self.n])
        return d_rows
