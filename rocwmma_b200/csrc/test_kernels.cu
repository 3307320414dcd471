// Device-side unit-test kernels for the fragment API (built into libb200wmma_test.so,
// used only by tests/).  They mirror the reference's API-level unit tests:
//   * load -> store round trip per warp     (test/unit/load_store_matrix_sync_test/device/
//                                            load_store_matrix_sync.hpp:38-135)
//   * cooperative load -> store round trip  (test/unit/load_store_matrix_coop_sync_test/device/
//                                            load_store_matrix_coop_sync.hpp:39-250)
//   * fill_fragment -> store                (test/unit/fill_fragment_test/device/
//                                            fill_fragment.hpp:37-120)
//   * MappingUtil coordinates               (test/unit/map_util_test)
// Contamination (writes outside the tile) is checked on the host side by padding the
// buffers, as the reference does (test/unit/contamination_test).
#include <cstdint>
#include <cuda_runtime.h>
#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_block.hpp>
#include <rocwmma/rocwmma_coop.hpp>
#include <rocwmma/rocwmma_transforms.hpp>
#include "tile_schedule.cuh"

using namespace rocwmma;

#define TEST_API extern "C" __attribute__((visibility("default")))

namespace
{
    template <typename Layout>
    __device__ inline uint32_t tileOrigin(uint32_t tr, uint32_t tc, uint32_t h, uint32_t w,
                                          uint32_t ld)
    {
        return std::is_same<Layout, row_major>::value ? tr * h * ld + tc * w
                                                      : tc * w * ld + tr * h;
    }

    // mode -2: load, applyTranspose, store the transposed fragment in the orthogonal layout
    //          (same memory image) -- matrix_a and matrix_b only
    // mode -3: load, applyDataLayout to the other layout and back, store
    // mode 0: every warp moves its own tile with load/store_matrix_sync
    // mode W > 0: the W warps of a block move ONE tile with the cooperative calls
    // mode -1: fill_fragment(value read from in[0]) then store_matrix_sync
    template <typename MatrixT, uint32_t BM, uint32_t BN, uint32_t BK, typename DataT,
              typename Layout>
    __global__ void roundTrip(DataT const* in, DataT* out, uint32_t ld, uint32_t tilesR,
                              uint32_t tilesC, int mode)
    {
        using Frag = fragment<MatrixT, BM, BN, BK, DataT, Layout>;
        Frag           frag;
        const uint32_t h = Frag::height(), w = Frag::width();
        // thread blocks are (warps_x * 32, warps_y) as in the reference's unit tests
        // (test/unit/unit_test_params.hpp:159-172); warps are numbered x first
        const uint32_t warpInBlock
            = (threadIdx.y * blockDim.x + threadIdx.x) / Constants::AMDGCN_WAVE_SIZE;
        const uint32_t warpsPerBlk = blockDim.x * blockDim.y / Constants::AMDGCN_WAVE_SIZE;
        if(mode > 0)
        {
            const uint32_t tile = blockIdx.x;
            if(tile >= tilesR * tilesC)
                return;
            const uint32_t off = tileOrigin<Layout>(tile / tilesC, tile % tilesC, h, w, ld);
            load_matrix_coop_sync(frag, in + off, ld, warpInBlock, warpsPerBlk);
            store_matrix_coop_sync(out + off, frag, ld, warpInBlock, warpsPerBlk);
            return;
        }
        const uint32_t tile = blockIdx.x * warpsPerBlk + warpInBlock;
        if(tile >= tilesR * tilesC)
            return;
        const uint32_t off = tileOrigin<Layout>(tile / tilesC, tile % tilesC, h, w, ld);
        if(mode == -2)
        {
            if constexpr(!std::is_same<MatrixT, accumulator>::value && BN % 16u == 0u)
            {
                load_matrix_sync(frag, in + off, ld);
                auto t = applyTranspose(frag);
                // the transpose in the orthogonal layout addresses memory exactly like frag
                store_matrix_sync(out + off, t, ld);
            }
            return;
        }
        if(mode == -3)
        {
            using Other = typename detail::OrthogonalLayout<Layout>::type;
            load_matrix_sync(frag, in + off, ld);
            auto const& o = applyDataLayout<Other>(frag);
            auto const& back = applyDataLayout<Layout>(o);
            store_matrix_sync(out + off, back, ld);
            return;
        }
        if(mode == 0)
            load_matrix_sync(frag, in + off, ld);
        else
            fill_fragment(frag, in[0]);
        store_matrix_sync(out + off, frag, ld);
    }

    template <typename MatrixT, uint32_t BM, uint32_t BN, uint32_t BK, typename DataT,
              typename Layout>
    int launchRT(void const* in, void* out, uint32_t ld, uint32_t tilesR, uint32_t tilesC, int mode,
                 int warps, cudaStream_t s)
    {
        // `warps` packs the thread block: warps_x + 16 * warps_y (warps_y = 0 means 1)
        const uint32_t wx = uint32_t(warps) & 15u, wy = (uint32_t(warps) >> 4) ? (uint32_t(warps) >> 4) : 1u;
        const uint32_t perBlock = wx * wy;
        const uint32_t tiles    = tilesR * tilesC;
        const uint32_t blocks   = mode > 0 ? tiles : (tiles + perBlock - 1) / perBlock;
        roundTrip<MatrixT, BM, BN, BK, DataT, Layout><<<blocks, dim3(wx * 32, wy), 0, s>>>(
            static_cast<DataT const*>(in), static_cast<DataT*>(out), ld, tilesR, tilesC, mode);
        return cudaGetLastError() == cudaSuccess ? 0 : -4;
    }

    template <typename MatrixT, uint32_t BM, uint32_t BN, uint32_t BK, typename DataT>
    int byLayout(int layout, void const* in, void* out, uint32_t ld, uint32_t tr, uint32_t tc,
                 int mode, int warps, cudaStream_t s)
    {
        return layout == 0
                   ? launchRT<MatrixT, BM, BN, BK, DataT, row_major>(in, out, ld, tr, tc, mode,
                                                                     warps, s)
                   : launchRT<MatrixT, BM, BN, BK, DataT, col_major>(in, out, ld, tr, tc, mode,
                                                                     warps, s);
    }

    template <uint32_t BM, uint32_t BN, uint32_t BK, typename DataT>
    int byMatrix(int matrix, int layout, void const* in, void* out, uint32_t ld, uint32_t tr,
                 uint32_t tc, int mode, int warps, cudaStream_t s)
    {
        switch(matrix)
        {
        case 0:
            return byLayout<matrix_a, BM, BN, BK, DataT>(layout, in, out, ld, tr, tc, mode, warps,
                                                         s);
        case 1:
            return byLayout<matrix_b, BM, BN, BK, DataT>(layout, in, out, ld, tr, tc, mode, warps,
                                                         s);
        case 2:
            return byLayout<accumulator, BM, BN, BK, DataT>(layout, in, out, ld, tr, tc, mode,
                                                            warps, s);
        }
        return -1;
    }

    // The reference's unit tests run over (first, second) block-size pairs
    // (test/unit/unit_test_params.hpp:85-110): matrix_a is first x second (BlockM x BlockK),
    // matrix_b second x first (BlockK x BlockN), the accumulator first x second
    // (BlockM x BlockN).  Pairs a type cannot hold (8-bit operands need BlockK >= 16) return -2.
    template <uint32_t X, uint32_t Y, typename DataT>
    int byPair(int matrix, int layout, void const* in, void* out, uint32_t ld, uint32_t tr,
               uint32_t tc, int mode, int warps, cudaStream_t s)
    {
        if(matrix == 2)
        {
            if constexpr(Y % 8u == 0u)
                return byLayout<accumulator, X, Y, 16, DataT>(layout, in, out, ld, tr, tc, mode,
                                                              warps, s);
            else
                return -2;
        }
        constexpr uint32_t minK = sizeof(DataT) == 1 ? 16u : sizeof(DataT) == 2 ? 8u : 4u;
        if constexpr(Y % minK == 0u)
        {
            if(matrix == 0)
                return byLayout<matrix_a, X, 16, Y, DataT>(layout, in, out, ld, tr, tc, mode, warps,
                                                           s);
            if(matrix == 1)
                return byLayout<matrix_b, 16, X, Y, DataT>(layout, in, out, ld, tr, tc, mode, warps,
                                                           s);
            return -1;
        }
        else
            return -2;
    }

    template <typename DataT>
    int byShape(int shape, int matrix, int layout, void const* in, void* out, uint32_t ld,
                uint32_t tr, uint32_t tc, int mode, int warps, cudaStream_t s)
    {
        switch(shape)
        {
        case 0:
            return byMatrix<16, 16, 16, DataT>(matrix, layout, in, out, ld, tr, tc, mode, warps, s);
        case 1:
            return byMatrix<32, 32, 32, DataT>(matrix, layout, in, out, ld, tr, tc, mode, warps, s);
        case 2:
            return byMatrix<64, 16, 32, DataT>(matrix, layout, in, out, ld, tr, tc, mode, warps, s);
            // 100 + i: the i-th (first, second) pair of the reference's unit-test grid
#define B200WMMA_PAIR(ID, X, Y) \
    case 100 + ID:              \
        return byPair<X, Y, DataT>(matrix, layout, in, out, ld, tr, tc, mode, warps, s);
            B200WMMA_PAIR(0, 16, 16)
            B200WMMA_PAIR(1, 16, 32)
            B200WMMA_PAIR(2, 16, 64)
            B200WMMA_PAIR(3, 32, 8)
            B200WMMA_PAIR(4, 32, 16)
            B200WMMA_PAIR(5, 32, 32)
            B200WMMA_PAIR(6, 32, 64)
            B200WMMA_PAIR(7, 64, 8)
            B200WMMA_PAIR(8, 64, 16)
            B200WMMA_PAIR(9, 64, 32)
            B200WMMA_PAIR(10, 64, 64)
            B200WMMA_PAIR(11, 128, 8)
            B200WMMA_PAIR(12, 128, 16)
            B200WMMA_PAIR(13, 256, 8)
#undef B200WMMA_PAIR
        }
        return -1;
    }

    __global__ void mappingKernel(uint32_t* out, uint32_t ldm)
    {
        using Map = MappingUtil<16, 32, float, row_major>;
        using MapC = MappingUtil<16, 32, float, col_major>;
        if((threadIdx.x % Constants::AMDGCN_WAVE_SIZE) != 0)
            return;
        const uint32_t warpsX = blockDim.x / Constants::AMDGCN_WAVE_SIZE;
        const uint32_t warp   = ((blockIdx.y * gridDim.x + blockIdx.x) * blockDim.y + threadIdx.y)
                                  * warpsX
                              + threadIdx.x / Constants::AMDGCN_WAVE_SIZE;
        uint32_t* o = out + warp * 12;
        auto      wc = Map::waveCoord();
        auto      bc = Map::blockCoord();
        auto      mc = Map::matrixCoord();
        auto      wg = Map::workgroupDim();
        o[0] = get<0>(wc), o[1] = get<1>(wc);
        o[2] = get<0>(bc), o[3] = get<1>(bc);
        o[4] = get<0>(mc), o[5] = get<1>(mc);
        o[6] = get<0>(wg), o[7] = get<1>(wg);
        o[8]  = Map::dataOffset(mc, ldm);
        o[9]  = MapC::dataOffset(mc, ldm);
        o[10] = get<0>(Map::matrixCoordN(7)) * 1000 + get<1>(Map::matrixCoordN(7));
        o[11] = Map::laneId() + get<1>(Map::blockCoordM(5)) * 100 + get<0>(Map::blockCoordM(5));
    }

    // A wait that nothing will ever satisfy: the barrier expects one arrival and gets none.
    // The bounded wait must give up after `limitCycles`, raise the block's abort flag and
    // let the kernel finish normally; out[0] = 1 if it returned false, out[1] = wait code,
    // out[2] = 1 if a second waiter in the block saw the abort flag and left too.
    __global__ void boundedWaitKernel(uint32_t* out, long long limitCycles)
    {
        __shared__ uint64_t                    bar;
        __shared__ rocwmma::block::AbortState abortState;
        if(threadIdx.x == 0)
        {
            rocwmma::block::mbar_init(&bar, 1);
            abortState.flag = 0;
            abortState.code = 0;
            rocwmma::block::mbar_init_fence();
        }
        __syncthreads();
        if(threadIdx.x == 0)
        {
            const bool ok = rocwmma::block::mbar_wait(&bar, 0, &abortState,
                                                      rocwmma::block::WAIT_STAGE_FULL, limitCycles);
            out[0] = ok ? 0u : 1u;
            out[1] = abortState.code;
        }
        else if(threadIdx.x == 32)
        {
            // much longer limit: this one must leave because of the flag, not its own clock
            const bool ok = rocwmma::block::mbar_wait(&bar, 0, &abortState,
                                                      rocwmma::block::WAIT_ACC_FULL,
                                                      limitCycles * 1000);
            out[2] = ok ? 0u : 1u;
        }
        __syncthreads();
        out[3] = abortState.flag;
    }

    // Untiled bulk copies: rows of `rowBytes` go global -> shared (one copy per lane, all
    // signalling one mbarrier that every lane arrives on once) and come back shared -> global
    // with every byte incremented, which shows that both directions and the proxy fence
    // between them work.  out status: 0 ok, 1 the wait ran out.
    __global__ void bulkCopyKernel(uint8_t const* src, uint8_t* dst, uint32_t rows,
                                   uint32_t rowBytes, uint32_t* status)
    {
        extern __shared__ __align__(128) uint8_t tile[];
        __shared__ uint64_t                    bar;
        __shared__ rocwmma::block::AbortState abortState;
        namespace blk = rocwmma::block;
        const uint32_t lane = threadIdx.x;
        if(lane == 0)
        {
            blk::mbar_init(&bar, 32);
            abortState.flag = 0;
            abortState.code = 0;
            blk::mbar_init_fence();
        }
        __syncwarp();
        const bool     mine = lane < rows;
        const uint32_t barA = blk::smem_addr(&bar);
        blk::mbar_arrive_expect_tx(barA, mine ? rowBytes : 0u);
        if(mine)
            blk::bulk_load(blk::smem_addr(tile) + lane * rowBytes, src + size_t(lane) * rowBytes,
                           rowBytes, barA);
        const bool ok = blk::mbar_wait(&bar, 0, &abortState, blk::WAIT_STAGE_FULL, 200000000ll);
        if(__all_sync(0xffffffffu, ok))
        {
            for(uint32_t i = lane; i < rows * rowBytes; i += 32)
                tile[i] = uint8_t(tile[i] + 1u);
            blk::fence_async_shared();
            __syncwarp();
            if(mine)
                blk::bulk_store(dst + size_t(lane) * rowBytes, blk::smem_addr(tile) + lane * rowBytes,
                                rowBytes);
            blk::tma_store_commit();
            blk::tma_store_wait_all<0>();
            if(lane == 0)
                status[0] = 0u;
        }
        else if(lane == 0)
            status[0] = 1u;
    }
} // namespace

// rows <= 32 rows of row_bytes (a multiple of 16, rows * row_bytes <= 64 KiB) travel
// src -> shared memory -> dst through cp.async.bulk in both directions; dst[i] = src[i] + 1.
TEST_API int b200wmma_test_bulk_copy(const void* src, void* dst, uint32_t rows, uint32_t row_bytes,
                                     uint32_t* status, void* stream)
{
    if(rows == 0 || rows > 32 || row_bytes == 0 || row_bytes % 16 != 0
       || size_t(rows) * row_bytes > 65536 || (reinterpret_cast<uintptr_t>(src) % 16) != 0
       || (reinterpret_cast<uintptr_t>(dst) % 16) != 0)
        return -1;
    if(cudaFuncSetAttribute(bulkCopyKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536)
       != cudaSuccess)
        return -4;
    bulkCopyKernel<<<1, 32, rows * row_bytes, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t const*>(src), static_cast<uint8_t*>(dst), rows, row_bytes, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Host-side walk over the pair kernel's tile schedule: counts[tm * (wide_cols + tail_cols) + c]
// is incremented for every tile some pair is given (tile column c counts wide columns first),
// loads[p] is the summed width of pair p's tiles.  Returns the number of tiles handed out, or
// -1 when a tile lies outside the grid or has the wrong width.
TEST_API int b200wmma_test_tile_schedule(uint32_t tiles_m, uint32_t wide_cols, uint32_t tail_cols,
                                         uint32_t bn, uint32_t bn_tail, uint32_t band,
                                         uint32_t pairs, uint32_t* counts, uint32_t* loads)
{
    b200wmma::TileSchedule sc{tiles_m, wide_cols, tail_cols, bn, bn_tail, band, pairs};
    int                    total = 0;
    for(uint32_t p = 0; p < pairs; ++p)
    {
        uint32_t tm, col0, width;
        for(uint32_t i = 0; sc.get(p, i, tm, col0, width); ++i)
        {
            uint32_t c;
            if(col0 < wide_cols * bn)
            {
                if(width != bn || col0 % bn != 0)
                    return -1;
                c = col0 / bn;
            }
            else
            {
                if(width != bn_tail || (col0 - wide_cols * bn) % bn_tail != 0)
                    return -1;
                c = wide_cols + (col0 - wide_cols * bn) / bn_tail;
            }
            if(tm >= tiles_m || c >= wide_cols + tail_cols)
                return -1;
            counts[tm * (wide_cols + tail_cols) + c] += 1;
            loads[p] += width;
            ++total;
            if(i > 100000)
                return -1;
        }
    }
    return total;
}

// Order of the wide tiles: seq[tm * wide_cols + c] receives the position p + i * pairs at which
// the schedule with the given `snake` / `mirror` settings hands out tile (tm, c) (no tail
// columns).  Returns the number of tiles, or -1 when a tile lies outside the grid.
TEST_API int b200wmma_test_tile_order(uint32_t tiles_m, uint32_t wide_cols, uint32_t bn,
                                      uint32_t band, uint32_t pairs, uint32_t snake,
                                      uint32_t mirror, uint32_t* seq)
{
    b200wmma::TileSchedule sc{tiles_m, wide_cols, 0u, bn, 0u, band, pairs, snake, mirror};
    int                    total = 0;
    for(uint32_t p = 0; p < pairs; ++p)
    {
        uint32_t tm, col0, width;
        for(uint32_t i = 0; sc.get(p, i, tm, col0, width); ++i)
        {
            if(width != bn || col0 % bn != 0 || tm >= tiles_m || col0 / bn >= wide_cols)
                return -1;
            seq[tm * wide_cols + col0 / bn] = p + i * pairs;
            ++total;
        }
    }
    return total;
}

// Work items of a launch whose last `split_tiles` tiles are cut in two along K:
// parts[tm * wide_cols + c] receives a bit mask of the K parts handed out for tile (tm, c)
// -- bit 0 set alone (with ways == 1) for a whole tile, bits 0 and 1 for the two halves of a
// split tile -- and whole[...] how often the tile was handed out as a whole.  Returns the
// number of work items, or -1 on an inconsistent item.
TEST_API int b200wmma_test_tile_split(uint32_t tiles_m, uint32_t wide_cols, uint32_t bn,
                                      uint32_t band, uint32_t pairs, uint32_t snake,
                                      uint32_t mirror, uint32_t split_tiles, uint32_t* parts,
                                      uint32_t* whole, uint32_t* per_pair)
{
    b200wmma::TileSchedule sc{tiles_m, wide_cols, 0u, bn, 0u, band, pairs, snake, mirror, split_tiles};
    int                    total = 0;
    for(uint32_t p = 0; p < pairs; ++p)
    {
        uint32_t tm, col0, width, part, ways, splitIndex;
        for(uint32_t i = 0; sc.getItem(p, i, tm, col0, width, part, ways, splitIndex); ++i)
        {
            if(width != bn || col0 % bn != 0 || tm >= tiles_m || col0 / bn >= wide_cols
               || part >= ways || (ways != 1u && ways != 2u) || (ways == 2u && splitIndex >= split_tiles))
                return -1;
            const uint32_t idx = tm * wide_cols + col0 / bn;
            if(ways == 1u)
                whole[idx] += 1;
            else
            {
                if(parts[idx] & (1u << part))
                    return -1; // the same half twice
                parts[idx] |= 1u << part;
            }
            per_pair[p] += ways == 1u ? 2u : 1u; // in half-tiles
            ++total;
        }
    }
    return total;
}

// Runs the never-satisfied wait with a limit of `limit_cycles` SM cycles (keep it around a
// millisecond); the kernel always terminates by itself.
TEST_API int b200wmma_test_bounded_wait(uint32_t* out4, long long limit_cycles, void* stream)
{
    if(limit_cycles <= 0 || limit_cycles > 20000000ll)
        return -1;
    boundedWaitKernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(out4, limit_cycles);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// elem_bytes 1/2/4/8 -> int8_t / float16_t / float32_t / float64_t; matrix 0/1/2 = a/b/acc;
// layout 0 row, 1 col; shape 0 = 16x16x16, 1 = 32x32x32, 2 = 64x16x32, 100 + i = the i-th block-size
// pair of the reference's unit-test grid (see byPair); mode see roundTrip; warps = warps_x +
// 16 * warps_y of the (warps_x * 32, warps_y) thread block.  -2: the type cannot hold the pair.
TEST_API int b200wmma_test_round_trip(int elem_bytes, int matrix, int layout, int shape,
                                      const void* in, void* out, uint32_t ld, uint32_t tiles_r,
                                      uint32_t tiles_c, int mode, int warps, void* stream)
{
    auto s = static_cast<cudaStream_t>(stream);
    {
        const int wx = warps & 15, wy = (warps >> 4) ? (warps >> 4) : 1;
        if(wx < 1 || wx * wy > 8)
            return -1;
    }
    switch(elem_bytes)
    {
    case 1:
        return byShape<int8_t>(shape, matrix, layout, in, out, ld, tiles_r, tiles_c, mode, warps,
                               s);
    case 2:
        return byShape<float16_t>(shape, matrix, layout, in, out, ld, tiles_r, tiles_c, mode,
                                  warps, s);
    case 4:
        return byShape<float32_t>(shape, matrix, layout, in, out, ld, tiles_r, tiles_c, mode,
                                  warps, s);
    case 8:
        return byShape<float64_t>(shape, matrix, layout, in, out, ld, tiles_r, tiles_c, mode,
                                  warps, s);
    }
    return -1;
}

// Fragment geometry as the device sees it: out[0..3] = height, width, num_elements, kDim.
TEST_API int b200wmma_test_geometry(int elem_bytes, int matrix, int shape, uint32_t* out4)
{
#define GEOM(T, M, BM, BN, BK)                                   \
    {                                                            \
        using F = fragment<M, BM, BN, BK, T, row_major>;         \
        out4[0] = F::height();                                   \
        out4[1] = F::width();                                    \
        out4[2] = F::num_elements;                               \
        out4[3] = F::kDim();                                     \
        return 0;                                                \
    }
#define GEOM_SHAPE(T, M)                 \
    switch(shape)                        \
    {                                    \
    case 0:                              \
        GEOM(T, M, 16, 16, 16)           \
    case 1:                              \
        GEOM(T, M, 32, 32, 32)           \
    case 2:                              \
        GEOM(T, M, 64, 16, 32)           \
    }                                    \
    return -1;
#define GEOM_MATRIX(T)                   \
    switch(matrix)                       \
    {                                    \
    case 0:                              \
        GEOM_SHAPE(T, matrix_a)          \
    case 1:                              \
        GEOM_SHAPE(T, matrix_b)          \
    case 2:                              \
        GEOM_SHAPE(T, accumulator)       \
    }                                    \
    return -1;
    switch(elem_bytes)
    {
    case 1:
        GEOM_MATRIX(int8_t)
    case 2:
        GEOM_MATRIX(float16_t)
    case 4:
        GEOM_MATRIX(float32_t)
    case 8:
        GEOM_MATRIX(float64_t)
    }
    return -1;
}

// Launches grid (gx, gy) of blocks (32 * wx, wy); out holds 12 words per warp.
TEST_API int b200wmma_test_mapping(uint32_t* out, uint32_t gx, uint32_t gy, uint32_t wx,
                                   uint32_t wy, uint32_t ldm, void* stream)
{
    mappingKernel<<<dim3(gx, gy), dim3(32 * wx, wy), 0, static_cast<cudaStream_t>(stream)>>>(out,
                                                                                            ldm);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
