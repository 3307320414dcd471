// y_out = alpha * A * x + beta * y_in for a column-major A (m x k, leading dimension lda).
//
// The reference sample pushes this through a 16x16x16 tensor-core tile of which one
// column is useful (samples/simple_sgemv.cpp:103-155).  GEMV moves 4 bytes of A per
// 2 flops, so on B200 it is bound by HBM bandwidth and the tensor cores cannot help:
// this kernel streams A with 128-bit loads, consecutive threads on consecutive rows
// (the contiguous direction of a column-major matrix), and splits K over enough
// thread blocks to fill the machine.  Each block writes partial sums for its K slice
// to a scratch array [kSplit][m]; a second small kernel adds the slices in a fixed
// order (so results do not depend on scheduling) and applies alpha and beta.
//
// Arithmetic follows the host routine samples/simple_sgemv.cpp:46-67 except for the
// order of the K summation.
#include "common.cuh"
#include "gemv.cuh"
#include "runtime.cuh"

namespace b200wmma
{
    namespace
    {
        constexpr uint32_t THREADS = 256;
        constexpr uint32_t UNROLL  = 8; // columns in flight per thread

        template <typename T, uint32_t VEC>
        struct alignas(sizeof(T) * VEC) Vec
        {
            T v[VEC];
        };

        // partial[ks][row] = sum over the block's K slice of A[row, h] * x[h]
        template <typename T, uint32_t VEC>
        __global__ void __launch_bounds__(THREADS)
            gemvPartial(uint32_t m, uint32_t k, T const* __restrict__ a, T const* __restrict__ x,
                        T* __restrict__ partial, uint32_t lda, uint32_t kChunk)
        {
            const uint32_t row0 = (blockIdx.x * THREADS + threadIdx.x) * VEC;
            const uint32_t h0   = blockIdx.y * kChunk;
            const uint32_t h1   = min(k, h0 + kChunk);

            __shared__ T xs[1024];
            T            acc[VEC];
#pragma unroll
            for(uint32_t v = 0; v < VEC; ++v)
                acc[v] = T(0);

            for(uint32_t hb = h0; hb < h1; hb += 1024)
            {
                const uint32_t cnt = min(1024u, h1 - hb);
                __syncthreads();
                for(uint32_t i = threadIdx.x; i < cnt; i += THREADS)
                    xs[i] = x[hb + i];
                __syncthreads();
                if(row0 < m)
                {
                    T const* col = a + size_t(hb) * lda + row0;
                    uint32_t i   = 0;
                    for(; i + UNROLL <= cnt; i += UNROLL)
                    {
                        Vec<T, VEC> av[UNROLL];
#pragma unroll
                        for(uint32_t u = 0; u < UNROLL; ++u)
                            av[u] = *reinterpret_cast<Vec<T, VEC> const*>(col + size_t(i + u) * lda);
#pragma unroll
                        for(uint32_t u = 0; u < UNROLL; ++u)
                        {
                            const T xv = xs[i + u];
#pragma unroll
                            for(uint32_t v = 0; v < VEC; ++v)
                                acc[v] += av[u].v[v] * xv;
                        }
                    }
                    for(; i < cnt; ++i)
                    {
                        const Vec<T, VEC> av
                            = *reinterpret_cast<Vec<T, VEC> const*>(col + size_t(i) * lda);
                        const T xv = xs[i];
#pragma unroll
                        for(uint32_t v = 0; v < VEC; ++v)
                            acc[v] += av.v[v] * xv;
                    }
                }
            }
            if(row0 < m)
            {
                Vec<T, VEC> out;
#pragma unroll
                for(uint32_t v = 0; v < VEC; ++v)
                    out.v[v] = acc[v];
                *reinterpret_cast<Vec<T, VEC>*>(partial + size_t(blockIdx.y) * m + row0) = out;
            }
        }

        // y_out[i] = alpha * (partial[0][i] + partial[1][i] + ...) + beta * y_in[i]
        template <typename T>
        __global__ void gemvFinish(uint32_t m, uint32_t kSplit, T const* __restrict__ partial,
                                   T const* yIn, T* yOut, T alpha, T beta)
        {
            const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
            if(i >= m)
                return;
            T acc = T(0);
            for(uint32_t s = 0; s < kSplit; ++s)
                acc += partial[size_t(s) * m + i];
            yOut[i] = alpha * acc + beta * yIn[i];
        }

        template <typename T, uint32_t VEC>
        int launchPartial(uint32_t m, uint32_t k, T const* a, T const* x, T* partial, uint32_t lda,
                          uint32_t kSplit, uint32_t kChunk, cudaStream_t stream)
        {
            dim3 grid((m + THREADS * VEC - 1) / (THREADS * VEC), kSplit);
            gemvPartial<T, VEC><<<grid, THREADS, 0, stream>>>(m, k, a, x, partial, lda, kChunk);
            return cudaToStatus(cudaGetLastError());
        }
    } // namespace

    void gemvPlan(uint32_t m, uint32_t k, size_t elemBytes, int sms, uint32_t* kSplit,
                  uint32_t* kChunk)
    {
        const uint32_t vec       = uint32_t(16 / elemBytes);
        const uint32_t rowBlocks = (m + THREADS * vec - 1) / (THREADS * vec);
        // about four blocks per SM, but never K slices shorter than 64 columns
        uint32_t split = (4u * uint32_t(sms) + rowBlocks - 1) / rowBlocks;
        split          = max(1u, min(split, max(1u, k / 64u)));
        split          = min(split, 1024u);
        *kChunk        = (k + split - 1) / split;
        *kSplit        = (k + *kChunk - 1) / *kChunk;
    }

    template <typename T>
    int gemvRun(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha,
                T beta, uint32_t lda, T* partial, uint32_t kSplit, uint32_t kChunk,
                cudaStream_t stream)
    {
        constexpr uint32_t VEC = 16 / sizeof(T);
        const bool vecOK = (m % VEC == 0) && (lda % VEC == 0)
                           && (reinterpret_cast<uintptr_t>(a) % 16 == 0)
                           && (reinterpret_cast<uintptr_t>(partial) % 16 == 0);
        int rc;
        if(vecOK)
            rc = launchPartial<T, VEC>(m, k, a, x, partial, lda, kSplit, kChunk, stream);
        else
        {
            // scalar rows: the row-block count differs, the K split is reused as is
            rc = launchPartial<T, 1>(m, k, a, x, partial, lda, kSplit, kChunk, stream);
        }
        if(rc != B200WMMA_OK)
            return rc;
        gemvFinish<T><<<(m + 255) / 256, 256, 0, stream>>>(m, kSplit, partial, yIn, yOut, alpha,
                                                          beta);
        return cudaToStatus(cudaGetLastError());
    }

    template int gemvRun<float>(uint32_t, uint32_t, float const*, float const*, float const*,
                                float*, float, float, uint32_t, float*, uint32_t, uint32_t,
                                cudaStream_t);
    template int gemvRun<double>(uint32_t, uint32_t, double const*, double const*, double const*,
                                 double*, double, double, uint32_t, double*, uint32_t, uint32_t,
                                 cudaStream_t);
} // namespace b200wmma

using namespace b200wmma;

extern "C" int b200wmma_gemv(int dtype, uint32_t m, uint32_t k, const void* a, const void* x,
                             const void* y_in, void* y_out, double alpha, double beta,
                             uint32_t lda, void* stream)
{
    if(!a || !x || !y_in || !y_out || m == 0 || k == 0 || lda < m)
        return B200WMMA_ERR_INVALID_ARG;
    if(dtype != B200WMMA_F32 && dtype != B200WMMA_F64)
        return B200WMMA_ERR_UNSUPPORTED;
    const size_t elem = dtypeSize(dtype);
    const int    sms  = smCount();
    if(sms <= 0)
        return B200WMMA_ERR_CUDA;
    uint32_t kSplit = 1, kChunk = k;
    gemvPlan(m, k, elem, sms, &kSplit, &kChunk);
    void* partial = deviceScratch(size_t(kSplit) * m * elem);
    if(!partial)
        return B200WMMA_ERR_CUDA;
    auto s = static_cast<cudaStream_t>(stream);
    if(dtype == B200WMMA_F32)
        return gemvRun<float>(m, k, static_cast<float const*>(a), static_cast<float const*>(x),
                              static_cast<float const*>(y_in), static_cast<float*>(y_out),
                              float(alpha), float(beta), lda, static_cast<float*>(partial), kSplit,
                              kChunk, s);
    return gemvRun<double>(m, k, static_cast<double const*>(a), static_cast<double const*>(x),
                           static_cast<double const*>(y_in), static_cast<double*>(y_out), alpha,
                           beta, lda, static_cast<double*>(partial), kSplit, kChunk, s);
}
