// Builds the reference's OWN sample kernels -- their text unmodified -- against THIS
// repository's rocwmma headers, into oracle/_ref/libref_kernels.so.
//
// TEST INFRASTRUCTURE ONLY.  It answers one question: does a kernel written for rocWMMA
// compile and compute correctly on top of include/rocwmma without being touched?  No
// reference source is copied into this repository: the Makefile slices the kernel part of
// each sample, where it lies in the mounted rocWMMA tree, into a scratch header inside
// oracle/_ref/ (ignored by git), compiles this file against it with nvcc and deletes the
// scratch header.  The slices (file: lines) are
//
//   samples/perf_hgemm.cpp : 193-714   parameters, fragment types, cooperative global -> LDS
//   samples/perf_sgemm.cpp : 193-666   staging, applyTranspose / applyDataLayout, the
//   samples/perf_dgemm.cpp : 193-657   double-buffered macro-tile kernel
//   samples/simple_hgemm.cpp, simple_sgemm.cpp, simple_dgemm.cpp : 81-139   one tile per warp
//   samples/simple_sgemv.cpp, simple_dgemv.cpp : 103-155
//   samples/simple_dlrm.cpp : 184-441  dlrmDotFwd, trilReconstruct, dlrmDotBwd
//
// Everything the slices need besides the rocwmma headers is the handful of names below:
// the samples' own constants (repeated here with the samples' values for a 32-lane warp)
// and HIP's spelling of a dynamic shared-memory declaration.  The launchers repeat the
// samples' launch geometry (perf_hgemm.cpp:811-820, simple_hgemm.cpp:195-200,
// simple_sgemv.cpp:207-212, simple_dlrm.cpp:503-587).
#include <cstdint>
#include <cuda_runtime.h>

#include <rocwmma/rocwmma.hpp>
#include <rocwmma/rocwmma_coop.hpp>
#include <rocwmma/rocwmma_transforms.hpp>

// hip/hip_runtime.h: HIP_DYNAMIC_SHARED(type, var) declares the dynamic LDS array.
#define HIP_DYNAMIC_SHARED(type, var) extern __shared__ type var[];
// HIP accepts __restrict as well as __restrict__; so does nvcc.
using uint = unsigned int;

#define REFK_STR2(x) #x
#define REFK_STR(x) REFK_STR2(x)
#define REFK_SLICE(name) REFK_STR(REFK_SLICE_DIR/name)

namespace
{
    inline int status(cudaError_t e)
    {
        return e == cudaSuccess ? 0 : -4;
    }
    inline unsigned ceilDivU(unsigned a, unsigned b)
    {
        return (a + b - 1) / b;
    }
} // namespace

// ---------------------------------------------------------------------------------------------
// perf_*gemm: the slices are self-contained (they start at `using namespace rocwmma;`).
// ---------------------------------------------------------------------------------------------
namespace ref_perf_hgemm
{
#include REFK_SLICE(perf_hgemm.inc)
} // namespace ref_perf_hgemm
// perf_sgemm.cpp:430-444 compiles its mma_sync loop only under ROCWMMA_ARCH_GFX9 ("SGEMM MMA only
// valid on gfx9 class cards": the other AMD targets have no fp32 matrix instruction).  This
// target has one (float32_t fragments multiply through three TF32 products), so the switch
// is turned on for this slice alone; nothing else in the slice looks at it.
#define ROCWMMA_ARCH_GFX9 1
namespace ref_perf_sgemm
{
#include REFK_SLICE(perf_sgemm.inc)
} // namespace ref_perf_sgemm
#undef ROCWMMA_ARCH_GFX9
namespace ref_perf_dgemm
{
#include REFK_SLICE(perf_dgemm.inc)
} // namespace ref_perf_dgemm

#define REFK_PERF_LAUNCHER(NS, KERNEL, FN)                                                        \
    extern "C" int FN(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,           \
                      const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,           \
                      uint32_t ldd, double alpha, double beta, void* stream)                      \
    {                                                                                             \
        using namespace NS;                                                                       \
        if(m % MACRO_TILE_X || n % MACRO_TILE_Y || k % ROCWMMA_K || k < ROCWMMA_K)                \
            return -1;                                                                            \
        dim3      block(TBLOCK_X, TBLOCK_Y), grid(m / MACRO_TILE_X, n / MACRO_TILE_Y);            \
        const int lds = 2u * sizeof(InputT) * (MACRO_TILE_X + MACRO_TILE_Y) * ROCWMMA_K;          \
        NS::KERNEL<<<grid, block, lds, static_cast<cudaStream_t>(stream)>>>(                      \
            m, n, k, static_cast<InputT const*>(a), static_cast<InputT const*>(b),                \
            static_cast<OutputT const*>(c), static_cast<OutputT*>(d), lda, ldb, ldc, ldd,         \
            ComputeT(alpha), ComputeT(beta));                                                     \
        return status(cudaGetLastError());                                                        \
    }                                                                                             \
    extern "C" void FN##_tile(uint32_t* out4)                                                     \
    {                                                                                             \
        out4[0] = NS::MACRO_TILE_X, out4[1] = NS::MACRO_TILE_Y, out4[2] = NS::ROCWMMA_K;           \
        out4[3] = NS::TBLOCK_X * NS::TBLOCK_Y;                                                     \
    }
REFK_PERF_LAUNCHER(ref_perf_hgemm, gemm_rocwmma_d, refk_perf_hgemm)
REFK_PERF_LAUNCHER(ref_perf_sgemm, sgemm_rocwmma_d, refk_perf_sgemm)
REFK_PERF_LAUNCHER(ref_perf_dgemm, gemm_rocwmma_d, refk_perf_dgemm)

// ---------------------------------------------------------------------------------------------
// simple_*gemm / simple_*gemv: the slices are the kernels only; their constants
// (simple_hgemm.cpp:46-65, simple_sgemv.cpp:68-86) depend on a run-time HIP query in the
// samples, so they are spelled out here for a 32-lane warp.
// ---------------------------------------------------------------------------------------------
#define REFK_SIMPLE_PREAMBLE(TBX_WARPS, TBY)                 \
    using rocwmma::accumulator;                              \
    using rocwmma::col_major;                                \
    using rocwmma::float16_t;                                \
    using rocwmma::float32_t;                                \
    using rocwmma::float64_t;                                \
    using rocwmma::matrix_a;                                 \
    using rocwmma::matrix_b;                                 \
    using rocwmma::row_major;                                \
    const int      ROCWMMA_M = 16;                           \
    const int      ROCWMMA_N = 16;                           \
    const int      ROCWMMA_K = 16;                           \
    const uint32_t WAVE_SIZE = 32;                           \
    const int      T_BLOCK_X = TBX_WARPS * WAVE_SIZE;        \
    const int      T_BLOCK_Y = TBY;

namespace ref_simple_hgemm
{
    REFK_SIMPLE_PREAMBLE(4, 4)
#include REFK_SLICE(simple_hgemm.inc)
} // namespace ref_simple_hgemm
namespace ref_simple_sgemm
{
    REFK_SIMPLE_PREAMBLE(4, 4)
#include REFK_SLICE(simple_sgemm.inc)
} // namespace ref_simple_sgemm
namespace ref_simple_dgemm
{
    REFK_SIMPLE_PREAMBLE(4, 4)
#include REFK_SLICE(simple_dgemm.inc)
} // namespace ref_simple_dgemm
namespace ref_simple_sgemv
{
    REFK_SIMPLE_PREAMBLE(16, 1)
#include REFK_SLICE(simple_sgemv.inc)
} // namespace ref_simple_sgemv
namespace ref_simple_dgemv
{
    REFK_SIMPLE_PREAMBLE(16, 1)
#include REFK_SLICE(simple_dgemv.inc)
} // namespace ref_simple_dgemv

#define REFK_SIMPLE_GEMM(NS, KERNEL, FN, IN_T, OUT_T, COMP_T)                                      \
    extern "C" int FN(uint32_t m, uint32_t n, uint32_t k, const void* a, const void* b,            \
                      const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,            \
                      uint32_t ldd, double alpha, double beta, void* stream)                       \
    {                                                                                              \
        using namespace NS;                                                                        \
        if(m % ROCWMMA_M || n % ROCWMMA_N || k % ROCWMMA_K)                                        \
            return -1;                                                                             \
        dim3 block(T_BLOCK_X, T_BLOCK_Y);                                                          \
        dim3 grid(ceilDivU(m, ROCWMMA_M * T_BLOCK_X / WAVE_SIZE),                                  \
                  ceilDivU(n, ROCWMMA_N * T_BLOCK_Y));                                             \
        NS::KERNEL<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(                         \
            m, n, k, static_cast<IN_T const*>(a), static_cast<IN_T const*>(b),                     \
            static_cast<OUT_T const*>(c), static_cast<OUT_T*>(d), lda, ldb, ldc, ldd,              \
            COMP_T(alpha), COMP_T(beta));                                                          \
        return status(cudaGetLastError());                                                         \
    }
REFK_SIMPLE_GEMM(ref_simple_hgemm, hgemm_rocwmma_d, refk_simple_hgemm, rocwmma::float16_t,
                 rocwmma::float16_t, rocwmma::float32_t)
REFK_SIMPLE_GEMM(ref_simple_sgemm, sgemm_rocwmma_d, refk_simple_sgemm, rocwmma::float32_t,
                 rocwmma::float32_t, rocwmma::float32_t)
REFK_SIMPLE_GEMM(ref_simple_dgemm, dgemm_rocwmma_d, refk_simple_dgemm, rocwmma::float64_t,
                 rocwmma::float64_t, rocwmma::float64_t)

// y = alpha * A x + beta * y, A column-major m x k with lda = m (simple_sgemv.cpp:163-167,
// 207-240: n = 1, ldb = k, ldc = ldd = m).  The sample kernel works on whole 16-column tiles
// (simple_sgemv.cpp:139,145,153), so it reads 16 k elements at x and 16 m elements at yIn
// and writes 16 m elements at yOut: the caller must pass buffers of that size, with the
// vectors in their first k resp. m elements.
#define REFK_SIMPLE_GEMV(NS, KERNEL, FN, T)                                                         \
    extern "C" int FN(uint32_t m, uint32_t k, const void* a, const void* x, const void* yIn,        \
                      void* yOut, double alpha, double beta, void* stream)                          \
    {                                                                                               \
        using namespace NS;                                                                         \
        if(m % ROCWMMA_M || k % ROCWMMA_K)                                                          \
            return -1;                                                                              \
        dim3 block(T_BLOCK_X, T_BLOCK_Y);                                                           \
        dim3 grid(ceilDivU(m, ROCWMMA_M * T_BLOCK_X / WAVE_SIZE), 1);                               \
        NS::KERNEL<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(                          \
            m, 1, k, static_cast<T const*>(a), static_cast<T const*>(x),                            \
            const_cast<T*>(static_cast<T const*>(yIn)), static_cast<T*>(yOut), m, k, m, m,          \
            T(alpha), T(beta));                                                                     \
        return status(cudaGetLastError());                                                          \
    }
REFK_SIMPLE_GEMV(ref_simple_sgemv, sgemv_rocwmma_d, refk_simple_sgemv, float)
REFK_SIMPLE_GEMV(ref_simple_dgemv, dgemv_rocwmma_d, refk_simple_dgemv, double)

// ---------------------------------------------------------------------------------------------
// simple_dlrm: three kernels (simple_dlrm.cpp:184-441); constants simple_dlrm.cpp:57-70.
// ---------------------------------------------------------------------------------------------
namespace ref_simple_dlrm
{
    using rocwmma::accumulator;
    using rocwmma::col_major;
    using rocwmma::float16_t;
    using rocwmma::float32_t;
    using rocwmma::float64_t;
    using rocwmma::matrix_a;
    using rocwmma::matrix_b;
    using rocwmma::row_major;
    using rocwmma::get;
    using rocwmma::make_coord2d;
    using rocwmma::Log2;
    constexpr static const int TILE_DIM  = 16;
    const uint32_t             WAVE_SIZE = 32;
    constexpr static const int T_BLOCK_X = 128;
#include REFK_SLICE(simple_dlrm.inc)
} // namespace ref_simple_dlrm

// acc: float[batch][m * m] scratch of the sample (simple_dlrm.cpp:471-476).
extern "C" int refk_dlrm_fwd(const void* input, void* output, void* acc, uint32_t m, uint32_t k,
                             uint32_t batch, void* stream)
{
    using namespace ref_simple_dlrm;
    if(m % TILE_DIM || k % TILE_DIM)
        return -1;
    dim3 grid(ceilDivU(m, TILE_DIM * T_BLOCK_X / WAVE_SIZE), ceilDivU(m, TILE_DIM), batch);
    dim3 block(T_BLOCK_X);
    dlrmDotFwd<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<float16_t const*>(input), static_cast<float16_t*>(output),
        static_cast<float*>(acc), m, k, batch, m * k, (m * (m - 1)) / 2 + k, m * m);
    return status(cudaGetLastError());
}

// acc: float16_t[batch][m * m] scratch of the sample.  The sample waits on the host between
// the two kernels (simple_dlrm.cpp:559-560); stream order gives the same guarantee.
extern "C" int refk_dlrm_bwd(const void* input, const void* upstream, void* grad, void* mlpGrad,
                             void* acc, uint32_t m, uint32_t k, uint32_t batch, void* stream)
{
    using namespace ref_simple_dlrm;
    if(m % TILE_DIM || k % TILE_DIM)
        return -1;
    auto       s        = static_cast<cudaStream_t>(stream);
    const uint upStride = (m * (m - 1)) / 2 + k;
    dim3       block(T_BLOCK_X);
    dim3       grid(ceilDivU(m * m, T_BLOCK_X), 1, batch);
    trilReconstruct<<<grid, block, 0, s>>>(static_cast<float16_t const*>(upstream),
                                           static_cast<float16_t*>(acc), m, k, batch, upStride,
                                           m * m);
    if(cudaGetLastError() != cudaSuccess)
        return -4;
    grid = dim3(ceilDivU(m, TILE_DIM * T_BLOCK_X / WAVE_SIZE), ceilDivU(k, TILE_DIM), batch);
    dlrmDotBwd<<<grid, block, 0, s>>>(static_cast<float16_t const*>(input),
                                      static_cast<float16_t const*>(upstream),
                                      static_cast<float16_t*>(grad),
                                      static_cast<float16_t*>(mlpGrad),
                                      static_cast<float16_t*>(acc), m, k, batch, m * k, upStride,
                                      m * m);
    return status(cudaGetLastError());
}
