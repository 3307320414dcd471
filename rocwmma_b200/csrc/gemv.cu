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
//   * a block owns ROWS consecutive rows; one warp-elected thread streams
//     ROWS x COLS tiles of A through a ring of shared-memory slots with TMA
//     (cp.async.bulk.tensor, no multicast), full/empty mbarriers per slot;
//   * ROWS compute threads, one per row, read their row's element of each column
//     from the slot (consecutive threads, consecutive addresses) and x[h] by a
//     warp-uniform cached load;
//   * 2 blocks per SM, ~80 KiB of TMA loads in flight per block.
//
// When pointer or leading dimension do not meet TMA's 16-byte rules a plain-load
// kernel with the same summation order is used.
#include "common.cuh"
#include "runtime.cuh"
#include <cstdlib>
#include <cuda.h>
#include <mutex>
#include <rocwmma/rocwmma_block.hpp>

using namespace rocwmma::block;

namespace
{
    constexpr uint32_t TILE_BYTES = 8192; // one ring slot: ROWS x COLS elements
    constexpr uint32_t MAX_STAGES = 26;

    // ROWS = rows per block = compute threads; the contiguous run of one column that a
    // TMA box row fetches is ROWS * sizeof(T) bytes, so taller blocks mean longer DRAM
    // bursts but fewer blocks.
    struct Control
    {
        uint64_t   full[MAX_STAGES];
        uint64_t   empty[MAX_STAGES];
        AbortState abort;
    };
    constexpr uint32_t smemBytes(uint32_t stages)
    {
        return stages * TILE_BYTES + 128 /*alignment slack*/ + uint32_t(sizeof(Control));
    }

    __device__ inline float  mulRn(float a, float b) { return __fmul_rn(a, b); }
    __device__ inline double mulRn(double a, double b) { return __dmul_rn(a, b); }
    __device__ inline float  addRn(float a, float b) { return __fadd_rn(a, b); }
    __device__ inline double addRn(double a, double b) { return __dadd_rn(a, b); }

    template <typename T, uint32_t ROWS, uint32_t STAGES>
    __global__ void __launch_bounds__(ROWS + 32)
        gemvTmaKernel(const __grid_constant__ CUtensorMap tmapA, uint32_t m, uint32_t k,
                      T const* __restrict__ x, T const* yIn, T* yOut, T alpha, T beta,
                      uint32_t* status)
    {
        constexpr uint32_t COLS = TILE_BYTES / (ROWS * sizeof(T)); // 32 (fp32) / 16 (fp64)
        extern __shared__ uint8_t smemRaw[];
        const uint32_t            raw   = smem_addr(smemRaw);
        uint8_t*                  tiles = smemRaw + ((128u - (raw & 127u)) & 127u);
        Control* ctl = reinterpret_cast<Control*>(tiles + STAGES * TILE_BYTES);

        const uint32_t row0   = blockIdx.x * ROWS;
        const uint32_t numKB  = (k + COLS - 1) / COLS;

        if(threadIdx.x == 0)
        {
            for(uint32_t s = 0; s < STAGES; ++s)
            {
                mbar_init(&ctl->full[s], 1);
                mbar_init(&ctl->empty[s], ROWS);
            }
            ctl->abort.flag = 0;
            ctl->abort.code = 0;
            mbar_init_fence();
            tma_prefetch_descriptor(&tmapA);
        }
        __syncthreads();

        if(threadIdx.x >= ROWS)
        {
            // ---- loader warp ----
            if(elect_one())
            {
                uint32_t kb = 0;
                bool     ok = true;
                for(; kb < numKB; ++kb)
                {
                    const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                    if(!mbar_wait(&ctl->empty[s], ph ^ 1u, &ctl->abort, WAIT_STAGE_EMPTY))
                    {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&ctl->full[s], TILE_BYTES);
                    tma_load_2d(tiles + s * TILE_BYTES, &tmapA, &ctl->full[s], int32_t(row0),
                                int32_t(kb * COLS));
                }
                if(!ok)
                {
                    const uint32_t pending = kb < STAGES ? kb : STAGES;
                    for(uint32_t j = 0; j < pending; ++j)
                    {
                        const uint32_t  prev = kb - 1 - j;
                        const long long t0   = clock64();
                        while(!mbar_try_wait(&ctl->full[prev % STAGES], (prev / STAGES) & 1u)
                              && clock64() - t0 < 2000000ll)
                        {
                        }
                    }
                }
            }
        }
        else
        {
            // ---- one row per thread, columns in ascending order ----
            const uint32_t r   = threadIdx.x;
            T              acc = T(0);
            for(uint32_t kb = 0; kb < numKB; ++kb)
            {
                const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                if(!mbar_wait(&ctl->full[s], ph, &ctl->abort, WAIT_STAGE_FULL))
                    break;
                T const*       tile = reinterpret_cast<T const*>(tiles + s * TILE_BYTES);
                const uint32_t h0   = kb * COLS;
                if(h0 + COLS <= k)
                {
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        acc = addRn(acc, mulRn(tile[j * ROWS + r], __ldg(x + h0 + j)));
                }
                else
                {
                    for(uint32_t j = 0; h0 + j < k; ++j)
                        acc = addRn(acc, mulRn(tile[j * ROWS + r], __ldg(x + h0 + j)));
                }
                mbar_arrive(&ctl->empty[s]);
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

    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    EncodeFn encoder()
    {
        static EncodeFn       fn = nullptr;
        static std::once_flag once;
        std::call_once(once, [] {
            void*                           sym = nullptr;
            cudaDriverEntryPointQueryResult q;
            if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q)
                   == cudaSuccess
               && q == cudaDriverEntryPointSuccess)
                fn = reinterpret_cast<EncodeFn>(sym);
            else
                (void)cudaGetLastError();
        });
        return fn;
    }

    template <typename T, uint32_t ROWS, uint32_t STAGES>
    int runTma(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha,
               T beta, uint32_t lda, cudaStream_t stream)
    {
        static_assert(STAGES <= MAX_STAGES, "ring deeper than the control block");
        EncodeFn fn = encoder();
        if(!fn)
            return B200WMMA_ERR_CUDA;
        constexpr uint32_t COLS       = TILE_BYTES / (ROWS * sizeof(T));
        constexpr uint32_t SMEM_BYTES = smemBytes(STAGES);
        constexpr uint32_t THREADS    = ROWS + 32;
        CUtensorMap        map;
        cuuint64_t         dims[2]    = {m, k};
        cuuint64_t         strides[1] = {cuuint64_t(lda) * sizeof(T)};
        cuuint32_t         box[2]     = {ROWS, COLS};
        cuuint32_t         estr[2]    = {1, 1};
        const CUtensorMapDataType dt
            = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT64;
        if(fn(&map, dt, 2, const_cast<T*>(a), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           != CUDA_SUCCESS)
            return B200WMMA_ERR_CUDA;

        static bool attrDone[64] = {};
        int         dev          = 0;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev < 0 || dev >= 64 || !attrDone[dev])
        {
            B200WMMA_CUDA_TRY(cudaFuncSetAttribute(gemvTmaKernel<T, ROWS, STAGES>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   int(SMEM_BYTES)));
            if(dev >= 0 && dev < 64)
                attrDone[dev] = true;
        }
        gemvTmaKernel<T, ROWS, STAGES><<<(m + ROWS - 1) / ROWS, THREADS, SMEM_BYTES, stream>>>(
            map, m, k, x, yIn, yOut, alpha, beta, b200wmma::deviceStatusWord());
        return b200wmma::cudaToStatus(cudaGetLastError());
    }

    template <typename T>
    int run(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha, T beta,
            uint32_t lda, cudaStream_t stream)
    {
        const bool tmaOK = (reinterpret_cast<uintptr_t>(a) % 16 == 0)
                           && ((size_t(lda) * sizeof(T)) % 16 == 0) && m >= 64;
        if(!tmaOK)
        {
            gemvPlainKernel<T><<<(m + 127) / 128, 128, 0, stream>>>(m, k, a, x, yIn, yOut, alpha,
                                                                  beta, lda);
            return b200wmma::cudaToStatus(cudaGetLastError());
        }
        // Rows per block: B200WMMA_GEMV_ROWS overrides (tuning only).
        static const int forced = [] {
            const char* e = getenv("B200WMMA_GEMV_ROWS");
            return e ? atoi(e) : 0;
        }();
        const int sms  = b200wmma::smCount();
        uint32_t  rows = forced ? uint32_t(forced) : 128u;
        if(!forced && m / 128u < uint32_t(sms > 0 ? sms : 1) / 2u)
            rows = 64u; // small problems: more, shorter blocks
        if(rows >= 256u && m >= 256u)
            return runTma<T, 256, 24>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
        if(rows >= 128u && m >= 128u)
            return runTma<T, 128, 12>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
        return runTma<T, 64, 10>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
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
