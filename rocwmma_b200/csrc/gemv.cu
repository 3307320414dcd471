// y_out = alpha * A * x + beta * y_in for a column-major A (m x k, leading dimension lda).
//
// The reference sample pushes this through a 16x16x16 tensor-core tile of which one
// column is useful (samples/simple_sgemv.cpp:103-155).  GEMV moves 4 bytes of A per
// 2 flops, so on B200 it is bound by HBM bandwidth and tensor cores cannot help.
// What the kernel has to do is keep enough bytes of A in flight; the arithmetic is
// cheap enough to be done EXACTLY as the host routine does it
// (samples/simple_sgemv.cpp:46-67): one accumulator per row, products added one by
// one in ascending column order, rounded multiply then rounded add, then
// alpha * acc + beta * y.  Results are therefore bit-identical to the host routine,
// whatever the size (a K-split or tree reduction would differ from it by the
// rounding noise of a 16384-term fp32 sum, which alone exceeds 1e-4 relative).
//
//   * a block owns 64 consecutive rows; four loader warps stream 64-row x 32-column
//     tiles of A through a 10-slot shared-memory ring with 16-byte cp.async copies,
//     full/empty mbarriers per slot; the 32 values of x that belong to a tile travel in
//     the same slot, so that no compute thread ever waits on a global load (with x read
//     straight from global memory the kernel was bound by that latency, 3.8 TB/s);
//   * 64 compute threads, one per row, read their row's element of each column from
//     the slot (consecutive threads, consecutive addresses) and x[h] by warp-uniform
//     vector loads;
//   * 2 blocks per SM, 80 KiB of loads in flight per block.
//
// When pointer or leading dimension are not 16-byte multiples a plain-load kernel with
// the same summation order is used.
#include "common.cuh"
#include "runtime.cuh"
#include <rocwmma/rocwmma_block.hpp>

using namespace rocwmma::block;

namespace
{
    constexpr uint32_t ROWS       = 64; // rows per block, one compute thread per row
    constexpr uint32_t TILE_BYTES = 8192; // COLS columns x ROWS rows of A
    constexpr uint32_t XSEG_BYTES = 128; // the COLS values of x that go with them
    constexpr uint32_t SLOT_BYTES = TILE_BYTES + XSEG_BYTES; // one ring slot
    constexpr uint32_t STAGES     = 10;
    constexpr uint32_t CWARPS     = ROWS / 32; // compute warps
    constexpr uint32_t LWARPS     = 4; // loader warps
    constexpr uint32_t LTHREADS   = LWARPS * 32;
    constexpr uint32_t THREADS    = ROWS + LTHREADS;

    struct Control
    {
        uint64_t   full[STAGES];
        uint64_t   empty[STAGES];
        AbortState abort;
    };
    constexpr uint32_t SMEM_BYTES = STAGES * SLOT_BYTES + 128 /*alignment slack*/ + sizeof(Control);

    __device__ inline float  mulRn(float a, float b) { return __fmul_rn(a, b); }
    __device__ inline double mulRn(double a, double b) { return __dmul_rn(a, b); }
    __device__ inline float  addRn(float a, float b) { return __fadd_rn(a, b); }
    __device__ inline double addRn(double a, double b) { return __dadd_rn(a, b); }

    // 16-byte asynchronous copy global -> shared; bytes beyond srcBytes are zero-filled.
    __device__ inline void cpAsync16(uint32_t dst, void const* src, uint32_t srcBytes)
    {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                     "r"(srcBytes)
                     : "memory");
    }
    // One arrival on `bar` once all cp.async issued so far by this thread have landed.
    __device__ inline void cpAsyncArriveOn(uint64_t* bar)
    {
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(bar))
                     : "memory");
    }

    template <typename T, uint32_t N>
    struct alignas(sizeof(T) * N) Vec
    {
        T v[N];
    };

    template <typename T>
    __global__ void __launch_bounds__(THREADS, 2)
        gemvStreamKernel(uint32_t m, uint32_t k, T const* __restrict__ a, T const* __restrict__ x,
                         T const* yIn, T* yOut, T alpha, T beta, uint32_t lda, uint32_t* status)
    {
        constexpr uint32_t COLS   = TILE_BYTES / (ROWS * sizeof(T)); // 32 (fp32) / 16 (fp64)
        constexpr uint32_t CPC    = ROWS * sizeof(T) / 16; // 16-byte chunks per column
        constexpr uint32_t CHUNKS = COLS * CPC; // per ring slot (512)
        constexpr uint32_t XV     = 16 / sizeof(T);
        extern __shared__ uint8_t smemRaw[];
        const uint32_t            raw   = smem_addr(smemRaw);
        uint8_t*                  tiles = smemRaw + ((128u - (raw & 127u)) & 127u);
        Control* ctl = reinterpret_cast<Control*>(tiles + STAGES * SLOT_BYTES);

        static_assert(COLS * sizeof(T) == XSEG_BYTES, "x segment size");
        const uint32_t row0  = blockIdx.x * ROWS;
        const uint32_t numKB = (k + COLS - 1) / COLS;
        // x travels through the ring with its columns of A when it can be copied in 16-byte
        // pieces; otherwise the compute threads read it from global memory themselves
        const bool xStaged = (reinterpret_cast<uintptr_t>(x) % 16) == 0;

        if(threadIdx.x == 0)
        {
            for(uint32_t s = 0; s < STAGES; ++s)
            {
                mbar_init(&ctl->full[s], LTHREADS);
                mbar_init(&ctl->empty[s], CWARPS);
            }
            ctl->abort.flag = 0;
            ctl->abort.code = 0;
            mbar_init_fence();
        }
        __syncthreads();
        // the barriers are set up while the previous kernel of the stream drains; A, x and y
        // may be its output
        grid_dependency_wait();
        grid_launch_dependents();

        if(threadIdx.x >= ROWS)
        {
            // ---- loader warps ----
            const uint32_t t         = threadIdx.x - ROWS;
            const uint32_t tilesAddr = smem_addr(tiles);
            const uint32_t rowsValid = (m - row0) < ROWS ? (m - row0) : ROWS;
            for(uint32_t kb = 0; kb < numKB; ++kb)
            {
                const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                if(!mbar_wait(&ctl->empty[s], ph ^ 1u, &ctl->abort, WAIT_STAGE_EMPTY))
                    break;
                const uint32_t h0 = kb * COLS;
#pragma unroll
                for(uint32_t i = 0; i < CHUNKS / LTHREADS; ++i)
                {
                    const uint32_t c    = t + i * LTHREADS;
                    const uint32_t col  = c / CPC, part = c % CPC;
                    const uint32_t r    = part * XV; // first row of the chunk inside the block
                    uint32_t       bytes = 0;
                    if(h0 + col < k && r < rowsValid)
                        bytes = (rowsValid - r >= XV) ? 16u : uint32_t((rowsValid - r) * sizeof(T));
                    T const* src = bytes ? a + size_t(h0 + col) * lda + row0 + r : a;
                    cpAsync16(tilesAddr + s * SLOT_BYTES + c * 16u, src, bytes);
                }
                if(xStaged && t < XSEG_BYTES / 16u)
                {
                    const uint32_t j     = t * XV; // first column of this piece
                    uint32_t       bytes = 0;
                    if(h0 + j < k)
                        bytes = (k - h0 - j >= XV) ? 16u : uint32_t((k - h0 - j) * sizeof(T));
                    cpAsync16(tilesAddr + s * SLOT_BYTES + TILE_BYTES + t * 16u,
                              bytes ? x + h0 + j : x, bytes);
                }
                cpAsyncArriveOn(&ctl->full[s]);
            }
            asm volatile("cp.async.wait_all;" ::: "memory"); // nothing in flight when leaving
        }
        else
        {
            // ---- one row per thread, columns in ascending order ----
            // The ordered sum is a chain of dependent additions (4 cycles each); the loads of
            // the NEXT tile are issued before the chain of the current one starts, into a
            // second set of registers, so that their latency and the barrier wait hide
            // behind the chain.  (With one register set a tile cost ~600 cycles, which held a
            // block to ~25 GB/s -- just enough for one GPU's bandwidth with 256 blocks.)
            const uint32_t r   = threadIdx.x;
            T              acc = T(0);
            // copies tile kb's column values of row r, and its x values, into registers
            auto fetch = [&](uint32_t kb, T (&av)[COLS], T (&xv)[COLS]) -> bool {
                const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                const uint32_t h0 = kb * COLS;
                if(!xStaged)
                {
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        xv[j] = (h0 + j < k) ? __ldg(x + h0 + j) : T(0);
                }
                if(!mbar_wait(&ctl->full[s], ph, &ctl->abort, WAIT_STAGE_FULL))
                    return false;
                if(xStaged)
                {
                    Vec<T, XV> const* xs
                        = reinterpret_cast<Vec<T, XV> const*>(tiles + s * SLOT_BYTES + TILE_BYTES);
#pragma unroll
                    for(uint32_t j = 0; j < COLS; j += XV)
                    {
                        const Vec<T, XV> q = xs[j / XV]; // same address in every lane: broadcast
#pragma unroll
                        for(uint32_t e = 0; e < XV; ++e)
                            xv[j + e] = q.v[e];
                    }
                }
                T const* tile = reinterpret_cast<T const*>(tiles + s * SLOT_BYTES);
#pragma unroll
                for(uint32_t j = 0; j < COLS; ++j)
                    av[j] = tile[j * ROWS + r];
                return true;
            };
            // the ordered sum over one tile, then the slot goes back to the loaders (its
            // values have been consumed, so the loads are certainly complete).  Columns
            // beyond k hold zeros and must not enter the sum (adding +0 could turn a -0
            // into +0).
            auto consume = [&](uint32_t kb, T const (&av)[COLS], T const (&xv)[COLS]) {
                const uint32_t h0    = kb * COLS;
                const uint32_t valid = (k - h0) < COLS ? (k - h0) : COLS;
#pragma unroll
                for(uint32_t j = 0; j < COLS; ++j)
                    if(j < valid)
                        acc = addRn(acc, mulRn(av[j], xv[j]));
                __syncwarp();
                if((threadIdx.x & 31u) == 0u)
                    mbar_arrive(&ctl->empty[kb % STAGES]); // one arrival per warp
            };
            if constexpr(sizeof(T) == 4)
            {
                T    avA[COLS], xvA[COLS], avB[COLS], xvB[COLS];
                bool ok = numKB == 0u || fetch(0, avA, xvA);
                for(uint32_t kb = 0; ok && kb < numKB; kb += 2)
                {
                    const bool has1 = kb + 1 < numKB, has2 = kb + 2 < numKB;
                    if(has1 && !fetch(kb + 1, avB, xvB))
                        break;
                    consume(kb, avA, xvA);
                    if(has2 && !fetch(kb + 2, avA, xvA))
                        break;
                    if(has1)
                        consume(kb + 1, avB, xvB);
                }
            }
            else
            {
                // 64-bit elements: two register sets would not fit; one tile at a time
                T av[COLS], xv[COLS];
                for(uint32_t kb = 0; kb < numKB; ++kb)
                {
                    if(!fetch(kb, av, xv))
                        break;
                    consume(kb, av, xv);
                }
            }
            if(row0 + r < m && ctl->abort.flag == 0u)
                yOut[row0 + r] = addRn(mulRn(alpha, acc), mulRn(beta, yIn[row0 + r]));
        }
        __syncthreads();
        if(threadIdx.x == 0 && ctl->abort.flag != 0u && status != nullptr)
        {
            atomicExch(&status[1], ctl->abort.code);
            atomicExch(&status[0], 1u);
        }
    }

    // Same arithmetic with plain loads, for operands TMA cannot address.
    template <typename T>
    __global__ void gemvPlainKernel(uint32_t m, uint32_t k, T const* __restrict__ a,
                                    T const* __restrict__ x, T const* yIn, T* yOut, T alpha, T beta,
                                    uint32_t lda)
    {
        const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
        if(i >= m)
            return;
        T acc = T(0);
        for(uint32_t h = 0; h < k; ++h)
            acc = addRn(acc, mulRn(a[size_t(h) * lda + i], __ldg(x + h)));
        yOut[i] = addRn(mulRn(alpha, acc), mulRn(beta, yIn[i]));
    }

    template <typename T>
    int run(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha, T beta,
            uint32_t lda, cudaStream_t stream)
    {
        // 16-byte asynchronous copies need 16-byte aligned columns
        const bool streamOK = (reinterpret_cast<uintptr_t>(a) % 16 == 0)
                              && ((size_t(lda) * sizeof(T)) % 16 == 0);
        if(!streamOK)
        {
            gemvPlainKernel<T><<<(m + 127) / 128, 128, 0, stream>>>(m, k, a, x, yIn, yOut, alpha,
                                                                  beta, lda);
            return b200wmma::cudaToStatus(cudaGetLastError());
        }
        static bool attrDone[64] = {};
        int         dev          = 0;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev < 0 || dev >= 64 || !attrDone[dev])
        {
            B200WMMA_CUDA_TRY(cudaFuncSetAttribute(gemvStreamKernel<T>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   int(SMEM_BYTES)));
            if(dev >= 0 && dev < 64)
                attrDone[dev] = true;
        }
        return b200wmma::cudaToStatus(b200wmma::launchOverlapped(
            gemvStreamKernel<T>, dim3((m + ROWS - 1) / ROWS), dim3(THREADS), SMEM_BYTES, stream, m,
            k, a, x, yIn, yOut, alpha, beta, lda, b200wmma::deviceStatusWord()));
    }
} // namespace

extern "C" int b200wmma_gemv(int dtype, uint32_t m, uint32_t k, const void* a, const void* x,
                             const void* y_in, void* y_out, double alpha, double beta,
                             uint32_t lda, void* stream)
{
    if(!a || !x || !y_in || !y_out || m == 0 || k == 0 || lda < m)
        return B200WMMA_ERR_INVALID_ARG;
    if(dtype != B200WMMA_F32 && dtype != B200WMMA_F64)
        return B200WMMA_ERR_UNSUPPORTED;
    auto s = static_cast<cudaStream_t>(stream);
    if(dtype == B200WMMA_F32)
        return run<float>(m, k, static_cast<float const*>(a), static_cast<float const*>(x),
                          static_cast<float const*>(y_in), static_cast<float*>(y_out), float(alpha),
                          float(beta), lda, s);
    return run<double>(m, k, static_cast<double const*>(a), static_cast<double const*>(x),
                       static_cast<double const*>(y_in), static_cast<double*>(y_out), alpha, beta,
                       lda, s);
}
