// Double-precision macro-tile GEMM on the fragment API: D = alpha * A * B + beta * C.
//
// Same structure as the reference's perf_dgemm (samples/perf_dgemm.cpp:464: macro
// tile staged through shared memory, per-warp sub-tiles of fragments, mma_sync in
// the K loop), written for sm_100a: fp64 has no tcgen05 form, so the warp-level
// DMMA path (mma.sync m16n8k4 behind rocwmma::mma_sync) does the arithmetic, and
// cp.async replaces the global->register->LDS copy with a 3-deep asynchronous
// ring.  128 x 128 macro tile, 8 warps of 64 x 32, K step 16.
//
// Operands are read K-major (A row-major, B column-major); other layouts are
// transposed into scratch first.
#include "common.cuh"
#include "runtime.cuh"
#include <rocwmma/rocwmma.hpp>

using namespace rocwmma;

namespace
{
    constexpr uint32_t BM = 128, BN = 128, BK = 16;
    constexpr uint32_t LD      = BK + 4; // padded row: conflict-free 64-bit fragment reads
    constexpr uint32_t STAGES  = 3;
    constexpr uint32_t THREADS = 256;
    constexpr uint32_t WM = 64, WN = 32; // warp tile
    constexpr uint32_t STAGE_ELEMS = (BM + BN) * LD;
    constexpr uint32_t SMEM_BYTES  = STAGES * STAGE_ELEMS * sizeof(double);

    __device__ inline void cpAsync16(void* smem, void const* gmem, uint32_t srcBytes)
    {
        const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem),
                     "r"(srcBytes)
                     : "memory");
    }
    __device__ inline void cpAsyncCommit()
    {
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    template <int N>
    __device__ inline void cpAsyncWait()
    {
        asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
    }

    // Copies `rows` rows of BK doubles (row r at src + r*ld) into a padded tile;
    // rows >= rowsValid and columns >= kValid are zero-filled.
    __device__ inline void loadTile(double* tile, double const* src, uint32_t ld,
                                    uint32_t rowsValid, uint32_t kValid)
    {
        // 128 rows x 8 chunks of 16 bytes = 1024 chunks, 4 per thread
#pragma unroll
        for(uint32_t i = 0; i < (128 * (BK / 2)) / THREADS; ++i)
        {
            const uint32_t chunk = threadIdx.x + i * THREADS;
            const uint32_t r     = chunk / (BK / 2);
            const uint32_t c     = (chunk % (BK / 2)) * 2;
            uint32_t       bytes = 0;
            if(r < rowsValid && c < kValid)
                bytes = (kValid - c >= 2) ? 16u : 8u;
            double const* g = (bytes != 0) ? (src + size_t(r) * ld + c) : src;
            cpAsync16(tile + r * LD + c, g, bytes);
        }
    }

    __global__ void __launch_bounds__(THREADS, 1)
        gemm_f64_kernel(uint32_t m, uint32_t n, uint32_t k, double const* __restrict__ a,
                        double const* __restrict__ b, double const* __restrict__ c,
                        double* __restrict__ d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                        uint32_t ldd, double alpha, double beta)
    {
        extern __shared__ __align__(16) uint8_t smemRaw[];
        double* smem = reinterpret_cast<double*>(smemRaw);

        using FragA   = fragment<matrix_a, WM, WN, 4, double, row_major>;
        using FragB   = fragment<matrix_b, WM, WN, 4, double, col_major>;
        using FragAcc = fragment<accumulator, WM, WN, 4, double>;

        const uint32_t warp  = threadIdx.x / 32;
        const uint32_t lane  = threadIdx.x % 32;
        const uint32_t warpM = (warp % 2) * WM; // 2 warps down
        const uint32_t warpN = (warp / 2) * WN; // 4 warps across

        // Tile order: a band of GROUP tile rows walks all tile columns, so that the
        // concurrently running blocks share B columns and A rows in L2.
        const uint32_t tilesM = (m + BM - 1) / BM, tilesN = (n + BN - 1) / BN;
        constexpr uint32_t GROUP = 8;
        const uint32_t     t = blockIdx.x, perGroup = GROUP * tilesN;
        const uint32_t     firstM = (t / perGroup) * GROUP;
        const uint32_t     rows   = min(tilesM - firstM, GROUP);
        const uint32_t     tm = firstM + (t % perGroup) % rows, tn = (t % perGroup) / rows;
        const uint32_t     m0 = tm * BM, n0 = tn * BN;

        double const* aBase = a + size_t(m0) * lda;
        double const* bBase = b + size_t(n0) * ldb;
        const uint32_t aRows = min(BM, m - m0), bRows = min(BN, n - n0);
        const uint32_t numKB = (k + BK - 1) / BK;

        FragAcc acc;
        fill_fragment(acc, 0.0);

        // prologue: STAGES-1 slots in flight
#pragma unroll
        for(uint32_t s = 0; s < STAGES - 1; ++s)
        {
            if(s < numKB)
            {
                double* st = smem + s * STAGE_ELEMS;
                loadTile(st, aBase + s * BK, lda, aRows, k - s * BK);
                loadTile(st + BM * LD, bBase + s * BK, ldb, bRows, k - s * BK);
            }
            cpAsyncCommit();
        }

        for(uint32_t kb = 0; kb < numKB; ++kb)
        {
            cpAsyncWait<STAGES - 2>();
            synchronize_workgroup();

            // refill the slot consumed in the previous iteration
            const uint32_t next = kb + STAGES - 1;
            if(next < numKB)
            {
                double* st = smem + (next % STAGES) * STAGE_ELEMS;
                loadTile(st, aBase + next * BK, lda, aRows, k - next * BK);
                loadTile(st + BM * LD, bBase + next * BK, ldb, bRows, k - next * BK);
            }
            cpAsyncCommit();

            double const* sa = smem + (kb % STAGES) * STAGE_ELEMS + warpM * LD;
            double const* sb = smem + (kb % STAGES) * STAGE_ELEMS + BM * LD + warpN * LD;
#pragma unroll
            for(uint32_t kk = 0; kk < BK; kk += 4)
            {
                FragA fa;
                FragB fb;
                load_matrix_sync(fa, sa + kk, LD);
                load_matrix_sync(fb, sb + kk, LD);
                mma_sync(acc, fa, fb, acc);
            }
        }
        cpAsyncWait<0>();

        // epilogue: each unit is two neighbouring columns of one row -> 16-byte accesses
        using Geom          = FragAcc::Geom;
        const bool useC     = (beta != 0.0) && (c != nullptr);
        const bool vecOK    = ((reinterpret_cast<uintptr_t>(d) | (uintptr_t(ldd) * 8)) % 16 == 0)
                           && (!useC
                               || ((reinterpret_cast<uintptr_t>(c) | (uintptr_t(ldc) * 8)) % 16 == 0));
#pragma unroll
        for(uint32_t u = 0; u < Geom::Units; ++u)
        {
            const Coord2d  rc  = Geom::unitCoord(u, lane);
            const uint32_t row = m0 + warpM + rc.data[0];
            const uint32_t col = n0 + warpN + rc.data[1];
            if(row >= m || col >= n)
                continue;
            double v0 = acc.x[2 * u], v1 = acc.x[2 * u + 1];
            const bool pair = (col + 1 < n);
            if(pair && vecOK)
            {
                double2 out;
                if(useC)
                {
                    const double2 cv
                        = *reinterpret_cast<double2 const*>(c + size_t(row) * ldc + col);
                    out.x = __dadd_rn(__dmul_rn(alpha, v0), __dmul_rn(beta, cv.x));
                    out.y = __dadd_rn(__dmul_rn(alpha, v1), __dmul_rn(beta, cv.y));
                }
                else
                {
                    out.x = __dmul_rn(alpha, v0);
                    out.y = __dmul_rn(alpha, v1);
                }
                *reinterpret_cast<double2*>(d + size_t(row) * ldd + col) = out;
            }
            else
            {
                const double c0 = useC ? c[size_t(row) * ldc + col] : 0.0;
                d[size_t(row) * ldd + col]
                    = useC ? __dadd_rn(__dmul_rn(alpha, v0), __dmul_rn(beta, c0))
                           : __dmul_rn(alpha, v0);
                if(pair)
                {
                    const double c1 = useC ? c[size_t(row) * ldc + col + 1] : 0.0;
                    d[size_t(row) * ldd + col + 1]
                        = useC ? __dadd_rn(__dmul_rn(alpha, v1), __dmul_rn(beta, c1))
                               : __dmul_rn(alpha, v1);
                }
            }
        }
    }

    __global__ void transposeF64(double const* __restrict__ in, double* __restrict__ out,
                                 uint32_t rows, uint32_t cols, uint32_t ldIn, uint32_t ldOut)
    {
        __shared__ double tile[32][33];
        const uint32_t    c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
        for(uint32_t j = threadIdx.y; j < 32; j += blockDim.y)
        {
            const uint32_t r = r0 + j, cc = c0 + threadIdx.x;
            if(r < rows && cc < cols)
                tile[j][threadIdx.x] = in[size_t(r) * ldIn + cc];
        }
        __syncthreads();
        for(uint32_t j = threadIdx.y; j < 32; j += blockDim.y)
        {
            const uint32_t cc = c0 + j, r = r0 + threadIdx.x;
            if(r < rows && cc < cols)
                out[size_t(cc) * ldOut + r] = tile[threadIdx.x][j];
        }
    }
} // namespace

namespace b200wmma
{
    int gemmF64(uint32_t m, uint32_t n, uint32_t k, double const* a, double const* b,
                double const* c, double* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                double alpha, double beta, int layoutA, int layoutB, cudaStream_t stream)
    {
        // Every argument is checked before anything is enqueued: the transposition pass
        // below reads a and b with the caller's leading dimensions.
        const bool aT = layoutA == B200WMMA_COL_MAJOR, bT = layoutB == B200WMMA_ROW_MAJOR;
        if(lda < (aT ? m : k) || ldb < (bT ? n : k) || ldd < n || (beta != 0.0 && ldc < n))
            return B200WMMA_ERR_INVALID_ARG;
        // operands that are transposed are read element by element and need no alignment
        if((!aT && ((reinterpret_cast<uintptr_t>(a) % 16) || (lda % 2)))
           || (!bT && ((reinterpret_cast<uintptr_t>(b) % 16) || (ldb % 2))))
            return B200WMMA_ERR_ALIGNMENT;
        if(aT || bT)
        {
            const uint32_t kPad   = (k + 1) / 2 * 2;
            const size_t   aElems = layoutA == B200WMMA_COL_MAJOR ? size_t(m) * kPad : 0;
            const size_t   bElems = layoutB == B200WMMA_ROW_MAJOR ? size_t(n) * kPad : 0;
            double* scratch = static_cast<double*>(deviceScratch((aElems + bElems) * 8 + 16));
            if(!scratch)
                return B200WMMA_ERR_CUDA;
            dim3 block(32, 8);
            if(aElems)
            {
                transposeF64<<<dim3((m + 31) / 32, (k + 31) / 32), block, 0, stream>>>(
                    a, scratch, k, m, lda, kPad);
                a   = scratch;
                lda = kPad;
            }
            if(bElems)
            {
                transposeF64<<<dim3((n + 31) / 32, (k + 31) / 32), block, 0, stream>>>(
                    b, scratch + aElems, k, n, ldb, kPad);
                b   = scratch + aElems;
                ldb = kPad;
            }
            B200WMMA_CUDA_TRY(cudaGetLastError());
        }
        static bool attrDone[64] = {};
        int         dev          = 0;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev >= 0 && dev < 64 && !attrDone[dev])
        {
            B200WMMA_CUDA_TRY(cudaFuncSetAttribute(
                gemm_f64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)));
            attrDone[dev] = true;
        }
        const uint32_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
        gemm_f64_kernel<<<tiles, THREADS, SMEM_BYTES, stream>>>(m, n, k, a, b, c, d, lda, ldb, ldc,
                                                                ldd, alpha, beta);
        return cudaToStatus(cudaGetLastError());
    }
} // namespace b200wmma
