"""Device-side unit tests of the fragment API, after the reference's API-level suites:
load/store round trip (test/unit/load_store_matrix_sync_test), cooperative round trip with
1..4 warps (test/unit/load_store_matrix_coop_sync_test), fill_fragment
(test/unit/fill_fragment_test), contamination (test/unit/contamination_test: data outside
the tiles must never be touched) and MappingUtil (test/unit/map_util_test).

The kernels live in rocwmma_b200/csrc/test_kernels.cu (libb200wmma_test.so)."""
import ctypes as C

import numpy as np
import pytest
import torch

from rocwmma_b200 import _lib as L

SHAPES = {0: (16, 16, 16), 1: (32, 32, 32), 2: (64, 16, 32)}
# The reference's unit-test grid of (first, second) block sizes (test/unit/unit_test_params.hpp:
# 85-110; 128 and 256 are its extended sizes, kept here where a lane's share still fits the
# register file): matrix_a is first x second (BlockM x BlockK), matrix_b second x first
# (BlockK x BlockN), the accumulator first x second (BlockM x BlockN).  Shape ids 100 + i.
PAIRS = [(16, 16), (16, 32), (16, 64), (32, 8), (32, 16), (32, 32), (32, 64), (64, 8), (64, 16),
         (64, 32), (64, 64), (128, 8), (128, 16), (256, 8)]
# its thread blocks (unit_test_params.hpp:159-172): (warps_x, warps_y) of a (warps_x*32, warps_y) block
THREAD_BLOCKS = [(1, 1), (1, 2), (2, 1), (1, 4), (2, 2), (4, 1)]
NP = {1: np.int8, 2: np.float16, 4: np.float32, 8: np.float64}
MATRIX = {0: "a", 1: "b", 2: "acc"}


def tlib():
    lib = C.CDLL(L.TEST_LIB_PATH)
    lib.b200wmma_test_round_trip.restype = C.c_int
    lib.b200wmma_test_round_trip.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                             C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                             C.c_int, C.c_int, C.c_void_p]
    lib.b200wmma_test_geometry.restype = C.c_int
    lib.b200wmma_test_geometry.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_uint32)]
    lib.b200wmma_test_mapping.restype = C.c_int
    lib.b200wmma_test_mapping.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                          C.c_uint32, C.c_uint32, C.c_void_p]
    lib.b200wmma_test_bounded_wait.restype = C.c_int
    lib.b200wmma_test_bounded_wait.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p]
    lib.b200wmma_test_bulk_copy.restype = C.c_int
    lib.b200wmma_test_bulk_copy.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                            C.c_void_p, C.c_void_p]
    return lib


def tile_hw(matrix, shape):
    if shape >= 100:
        first, second = PAIRS[shape - 100]
        return {0: (first, second), 1: (second, first), 2: (first, second)}[matrix]
    bm, bn, bk = SHAPES[shape]
    return {0: (bm, bk), 1: (bk, bn), 2: (bm, bn)}[matrix]


def pair_fits(eb, matrix, pair):
    """8-bit operand fragments need BlockK >= 16 (the reference's own minimum)."""
    return matrix == 2 or eb != 1 or pair[1] >= 16


def test_fragment_geometry_matches_the_reference_rules():
    """A is BlockM x BlockK, B is BlockK x BlockN, the accumulator BlockM x BlockN
    (internal/io_shape.hpp:44-80); a lane holds rows*cols/32 elements
    (internal/io_traits.hpp:60-66).  Host-side: needs no GPU."""
    lib = tlib()
    out = (C.c_uint32 * 4)()
    for eb in NP:
        for matrix in MATRIX:
            for shape in SHAPES:
                assert lib.b200wmma_test_geometry(eb, matrix, shape, out) == 0
                h, w = tile_hw(matrix, shape)
                assert (out[0], out[1]) == (h, w)
                assert out[2] == h * w // 32
                assert out[3] == SHAPES[shape][2]


def _random(eb, n, rng):
    if eb == 1:
        return rng.integers(-128, 128, n, dtype=np.int8)
    return rng.uniform(-4, 4, n).astype(NP[eb])


def _run_round_trip(eb, matrix, layout, shape, mode, warps, tiles_r=3, tiles_c=2, pad=5):
    """Returns (input, output) as 2-D arrays in STORAGE order (rows of length ld), plus the
    storage extents the tiles cover."""
    h, w = tile_hw(matrix, shape)
    rows, cols = tiles_r * h, tiles_c * w
    # storage: row-major -> rows x ld with ld >= cols; col-major -> cols x ld with ld >= rows
    major, minor = (rows, cols) if layout == 0 else (cols, rows)
    ld = minor + pad
    rng = np.random.default_rng(eb * 100 + matrix * 10 + shape)
    src = _random(eb, (major + 2) * ld, rng)          # two extra storage rows as a border
    sentinel = np.full_like(src, 77)
    t_in = torch.from_numpy(src).cuda()
    t_out = torch.from_numpy(sentinel).cuda()
    if isinstance(warps, tuple):                 # (warps_x, warps_y) thread block
        warps = warps[0] + 16 * warps[1]
    rc = tlib().b200wmma_test_round_trip(eb, matrix, layout, shape, t_in.data_ptr(),
                                         t_out.data_ptr(), ld, tiles_r, tiles_c, mode, warps,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return (src.reshape(major + 2, ld), t_out.cpu().numpy().reshape(major + 2, ld), major, minor)


@pytest.mark.gpu
@pytest.mark.parametrize("eb", [1, 2, 4, 8])
@pytest.mark.parametrize("matrix", [0, 1, 2])
@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("shape", [0, 1, 2])
def test_load_store_round_trip_and_contamination(eb, matrix, layout, shape):
    src, out, major, minor = _run_round_trip(eb, matrix, layout, shape, mode=0, warps=4)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()


@pytest.mark.gpu
@pytest.mark.parametrize("eb", [1, 2, 4, 8])
@pytest.mark.parametrize("matrix", [0, 1, 2])
@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("pair", range(len(PAIRS)), ids=[f"{a}x{b}" for a, b in PAIRS])
def test_round_trip_over_the_reference_block_grid(eb, matrix, layout, pair):
    """load_matrix_sync / store_matrix_sync round trip and contamination check for every block
    size of the reference's unit-test grid, from 32 x 8 up to 256 x 8, four element sizes."""
    if not pair_fits(eb, matrix, PAIRS[pair]):
        pytest.skip("8-bit operand fragments start at BlockK = 16, as in the reference")
    src, out, major, minor = _run_round_trip(eb, matrix, layout, 100 + pair, mode=0, warps=(2, 2),
                                             tiles_r=2, tiles_c=3, pad=3)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()


@pytest.mark.gpu
@pytest.mark.parametrize("block", THREAD_BLOCKS, ids=[f"{x * 32}x{y}" for x, y in THREAD_BLOCKS])
@pytest.mark.parametrize("eb,matrix,layout,pair", [(2, 0, 0, 3), (2, 1, 1, 4), (4, 2, 0, 6),
                                                   (1, 0, 1, 9), (8, 1, 0, 0), (2, 0, 1, 12),
                                                   (4, 1, 1, 7), (2, 2, 1, 13)])
def test_thread_block_arrangements(block, eb, matrix, layout, pair):
    """The reference's thread blocks -- (32,1), (32,2), (64,1), (32,4), (64,2), (128,1) -- each
    warp moving its own tile, and all warps of the block moving one tile cooperatively."""
    src, out, major, minor = _run_round_trip(eb, matrix, layout, 100 + pair, mode=0, warps=block)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()
    nwarps = block[0] * block[1]
    src, out, major, minor = _run_round_trip(eb, matrix, layout, 100 + pair, mode=nwarps,
                                             warps=block)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()


@pytest.mark.gpu
@pytest.mark.parametrize("warps", [1, 2, 3, 4])
@pytest.mark.parametrize("eb,matrix,layout,shape", [(2, 0, 0, 0), (2, 1, 1, 0), (4, 2, 0, 1),
                                                    (1, 0, 1, 1), (8, 1, 0, 0), (2, 0, 1, 2),
                                                    (4, 1, 1, 2), (2, 2, 1, 0)])
def test_cooperative_round_trip(warps, eb, matrix, layout, shape):
    """Each of the W warps of a block moves its slice; together they move the whole tile.
    W = 3 does not divide the work: the split falls back to the largest halved count and the
    surplus warp touches nothing -- the tile must still arrive complete."""
    src, out, major, minor = _run_round_trip(eb, matrix, layout, shape, mode=warps, warps=warps)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()


@pytest.mark.gpu
@pytest.mark.parametrize("eb,matrix,layout,shape", [(2, 0, 0, 0), (4, 2, 1, 1), (8, 1, 0, 2),
                                                    (1, 1, 1, 1)])
def test_fill_fragment(eb, matrix, layout, shape):
    src, out, major, minor = _run_round_trip(eb, matrix, layout, shape, mode=-1, warps=2)
    assert (out[:major, :minor] == src[0, 0]).all()
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()


@pytest.mark.gpu
def test_mapping_util():
    """blockDim = (32 * warps_x, warps_y): warp (x, y) of the grid owns tile row x, tile
    column y of 16 x 32 tiles (internal/mapping_util_impl.hpp:46-98, 166-179)."""
    gx, gy, wx, wy, ldm = 2, 3, 2, 2, 500
    n_warps = gx * gy * wx * wy
    out = torch.zeros(n_warps * 12, dtype=torch.int32, device="cuda")
    assert tlib().b200wmma_test_mapping(out.data_ptr(), gx, gy, wx, wy, ldm,
                                        torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    o = out.cpu().numpy().reshape(n_warps, 12)
    seen = set()
    for by in range(gy):
        for bx in range(gx):
            for ty in range(wy):
                for tx in range(wx):
                    warp = ((by * gx + bx) * wy + ty) * wx + tx
                    r = o[warp]
                    assert (r[0], r[1]) == (tx, ty)                       # waveCoord
                    brow, bcol = bx * wx + tx, by * wy + ty
                    assert (r[2], r[3]) == (brow, bcol)                   # blockCoord
                    assert (r[4], r[5]) == (brow * 16, bcol * 32)         # matrixCoord
                    assert (r[6], r[7]) == (wx, wy)                       # workgroupDim
                    assert r[8] == brow * 16 * ldm + bcol * 32            # row-major offset
                    assert r[9] == bcol * 32 * ldm + brow * 16            # col-major offset
                    assert r[10] == brow * 16 * 1000 + 7                  # matrixCoordN(7)
                    assert r[11] == 0 + bcol * 100 + 5                    # laneId, blockCoordM(5)
                    seen.add((brow, bcol))
    assert len(seen) == n_warps


@pytest.mark.gpu
def test_bounded_wait_gives_up_and_reports():
    """Failure detection without a fault: a barrier that nothing ever signals.  The wait has a
    ~1 ms limit, after which it raises the block's abort flag and returns false; a second
    waiter with a far longer limit leaves because of the flag.  The kernel ends normally and
    the context stays usable."""
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = tlib().b200wmma_test_bounded_wait(out.data_ptr(), 2_000_000,
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    gave_up, code, follower_left, flag = out.cpu().tolist()
    assert gave_up == 1 and code == 2 and follower_left == 1 and flag == 1
    # the device is still healthy
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


@pytest.mark.gpu
@pytest.mark.parametrize("rows,row_bytes", [(1, 16), (27, 256), (32, 512), (5, 2048)])
def test_untiled_bulk_copies_round_trip(rows, row_bytes):
    """cp.async.bulk global -> shared (mbarrier completion, one copy per lane) and shared ->
    global (bulk-group completion) of the block API: dst = src + 1 for every byte."""
    src = torch.randint(0, 256, (rows * row_bytes,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros_like(src)
    status = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    rc = tlib().b200wmma_test_bulk_copy(src.data_ptr(), dst.data_ptr(), rows, row_bytes,
                                        status.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.equal(dst, src + 1)  # uint8 arithmetic wraps, like the kernel's


@pytest.mark.gpu
@pytest.mark.parametrize("eb", [1, 2, 4, 8])
@pytest.mark.parametrize("matrix", [0, 1])
@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("shape", [0, 1, 2])
def test_apply_transpose(eb, matrix, layout, shape):
    """applyTranspose(A row-major) is B col-major of the same memory (and so on): storing the
    transposed fragment with its own, orthogonal, layout must reproduce the input image
    (rocwmma_transforms_impl.hpp:58-172)."""
    src, out, major, minor = _run_round_trip(eb, matrix, layout, shape, mode=-2, warps=2)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
    assert (out[:major, minor:] == 77).all() and (out[major:] == 77).all()


@pytest.mark.gpu
@pytest.mark.parametrize("matrix,layout", [(0, 0), (1, 1), (2, 0)])
def test_apply_data_layout_is_a_recast(matrix, layout):
    src, out, major, minor = _run_round_trip(2, matrix, layout, 1, mode=-3, warps=2)
    assert np.array_equal(out[:major, :minor], src[:major, :minor])
