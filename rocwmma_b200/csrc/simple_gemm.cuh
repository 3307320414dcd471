// One-tile-per-warp GEMM written on the fragment API: kernel and launch helpers shared by
// the translation units that instantiate it (simple_gemm.cu: each type's usual BlockK;
// simple_gemm_blockk.cu: the other K extents).
//
// Same algorithm and call sites as the reference's simple GEMM samples
// (samples/simple_hgemm.cpp:81-139; simple_sgemm.cpp:81; simple_dgemm.cpp:81):
// each warp owns one BlockM x BlockN tile of D, walks K in BlockK steps with
// load_matrix_sync / mma_sync, then scales element-wise across two accumulator
// fragments of different types and stores.  The thread block is
// (4 * 32, 4) = 16 warps as in the sample (samples/simple_hgemm.cpp:64-65).
#ifndef ROCWMMA_B200_CSRC_SIMPLE_GEMM_CUH
#define ROCWMMA_B200_CSRC_SIMPLE_GEMM_CUH
#include "common.cuh"
#include <rocwmma/rocwmma.hpp>

namespace b200wmma
{
namespace simple
{
    using namespace rocwmma;

    constexpr uint32_t T_BLOCK_X = 4 * Constants::AMDGCN_WAVE_SIZE;
    constexpr uint32_t T_BLOCK_Y = 4;

    template <typename InT,
              typename OutT,
              typename CompT,
              typename LayoutA,
              typename LayoutB,
              uint32_t BM,
              uint32_t BN,
              uint32_t BK>
    __global__ void __launch_bounds__(T_BLOCK_X* T_BLOCK_Y)
        gemm_simple_d(uint32_t    m,
                      uint32_t    n,
                      uint32_t    k,
                      InT const*  a,
                      InT const*  b,
                      OutT const* c,
                      OutT*       d,
                      uint32_t    lda,
                      uint32_t    ldb,
                      uint32_t    ldc,
                      uint32_t    ldd,
                      CompT       alpha,
                      CompT       beta,
                      layout_t    layoutCD)
    {
        auto fragA   = fragment<matrix_a, BM, BN, BK, InT, LayoutA>();
        auto fragB   = fragment<matrix_b, BM, BN, BK, InT, LayoutB>();
        auto fragC   = fragment<accumulator, BM, BN, BK, OutT>();
        auto fragAcc = fragment<accumulator, BM, BN, BK, CompT>();

        fill_fragment(fragAcc, CompT(0));

        // Tile using a 2D grid: warps along x own tile rows, along y tile columns.
        auto majorWarp = (blockIdx.x * blockDim.x + threadIdx.x) / Constants::AMDGCN_WAVE_SIZE;
        auto minorWarp = (blockIdx.y * blockDim.y + threadIdx.y);

        auto cRow = majorWarp * BM;
        auto cCol = minorWarp * BN;

        if(cRow < m && cCol < n)
        {
            constexpr bool aRow = std::is_same<LayoutA, row_major>::value;
            constexpr bool bRow = std::is_same<LayoutB, row_major>::value;
            for(uint32_t i = 0; i < k; i += BK)
            {
                load_matrix_sync(fragA, a + (aRow ? (cRow * lda + i) : (i * lda + cRow)), lda);
                load_matrix_sync(fragB, b + (bRow ? (i * ldb + cCol) : (i + cCol * ldb)), ldb);
                mma_sync(fragAcc, fragA, fragB, fragAcc);
            }

            const bool     cdRow = (layoutCD == mem_row_major);
            const uint32_t cOff  = cdRow ? (cRow * ldc + cCol) : (cRow + cCol * ldc);
            const uint32_t dOff  = cdRow ? (cRow * ldd + cCol) : (cRow + cCol * ldd);

            load_matrix_sync(fragC, c + cOff, ldc, layoutCD);

            for(uint32_t i = 0; i < fragC.num_elements; ++i)
            {
                // OutputT(alpha * acc + beta * ComputeT(c)), in ComputeT arithmetic
                fragC.x[i] = OutT(alpha * fragAcc.x[i] + beta * CompT(fragC.x[i]));
            }

            store_matrix_sync(d + dOff, fragC, ldd, layoutCD);
        }
    }

    template <typename InT, typename OutT, typename CompT, typename LA, typename LB, uint32_t BM,
              uint32_t BN, uint32_t BK>
    int launch(uint32_t m, uint32_t n, uint32_t k, void const* a, void const* b, void const* c,
               void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha,
               double beta, int layoutCD, cudaStream_t stream)
    {
        if(m % BM || n % BN || k % BK)
            return B200WMMA_ERR_INVALID_ARG;
        dim3 block(T_BLOCK_X, T_BLOCK_Y);
        dim3 grid(ceilDiv(m, BM * T_BLOCK_X / Constants::AMDGCN_WAVE_SIZE),
                  ceilDiv(n, BN * T_BLOCK_Y));
        gemm_simple_d<InT, OutT, CompT, LA, LB, BM, BN, BK><<<grid, block, 0, stream>>>(
            m, n, k, static_cast<InT const*>(a), static_cast<InT const*>(b),
            static_cast<OutT const*>(c), static_cast<OutT*>(d), lda, ldb, ldc, ldd, CompT(alpha),
            CompT(beta), layoutCD == B200WMMA_ROW_MAJOR ? mem_row_major : mem_col_major);
        return b200wmma::cudaToStatus(cudaGetLastError());
    }

    template <typename InT, typename OutT, typename CompT, uint32_t BM, uint32_t BN, uint32_t BK,
              typename... Args>
    int launchLayouts(int la, int lb, Args... args)
    {
        if(la == B200WMMA_ROW_MAJOR && lb == B200WMMA_ROW_MAJOR)
            return launch<InT, OutT, CompT, row_major, row_major, BM, BN, BK>(args...);
        if(la == B200WMMA_ROW_MAJOR && lb == B200WMMA_COL_MAJOR)
            return launch<InT, OutT, CompT, row_major, col_major, BM, BN, BK>(args...);
        if(la == B200WMMA_COL_MAJOR && lb == B200WMMA_ROW_MAJOR)
            return launch<InT, OutT, CompT, col_major, row_major, BM, BN, BK>(args...);
        if(la == B200WMMA_COL_MAJOR && lb == B200WMMA_COL_MAJOR)
            return launch<InT, OutT, CompT, col_major, col_major, BM, BN, BK>(args...);
        return B200WMMA_ERR_INVALID_ARG;
    }


    // Everything a launch needs besides the template parameters.
    struct Args
    {
        uint32_t     m, n, k;
        void const * a, *b, *c;
        void*        d;
        uint32_t     lda, ldb, ldc, ldd;
        double       alpha, beta;
        int          layoutA, layoutB, layoutCD;
        cudaStream_t stream;
    };

    template <typename InT, typename OutT, typename CompT, uint32_t BM, uint32_t BN, uint32_t BK>
    int launchTile(Args const& g)
    {
        return launchLayouts<InT, OutT, CompT, BM, BN, BK>(g.layoutA, g.layoutB, g.m, g.n, g.k, g.a,
                                                           g.b, g.c, g.d, g.lda, g.ldb, g.ldc, g.ldd,
                                                           g.alpha, g.beta, g.layoutCD, g.stream);
    }

    // The type triples of rocWMMA's table (docs/api-reference/api-reference-guide.rst:80-153)
    // that this library builds: F(in code, out code, compute code, InT, OutT, CompT).
#define B200WMMA_SIMPLE_TRIPLES(F)                                                         \
    F(B200WMMA_F16, B200WMMA_F32, B200WMMA_F32, float16_t, float32_t, float32_t)           \
    F(B200WMMA_F16, B200WMMA_F16, B200WMMA_F32, float16_t, float16_t, float32_t)           \
    F(B200WMMA_F16, B200WMMA_F16, B200WMMA_F16, float16_t, float16_t, float16_t)           \
    F(B200WMMA_BF16, B200WMMA_F32, B200WMMA_F32, bfloat16_t, float32_t, float32_t)         \
    F(B200WMMA_BF16, B200WMMA_BF16, B200WMMA_F32, bfloat16_t, bfloat16_t, float32_t)       \
    F(B200WMMA_BF16, B200WMMA_BF16, B200WMMA_BF16, bfloat16_t, bfloat16_t, bfloat16_t)     \
    F(B200WMMA_E4M3, B200WMMA_F32, B200WMMA_F32, float8_t, float32_t, float32_t)           \
    F(B200WMMA_E5M2, B200WMMA_F32, B200WMMA_F32, bfloat8_t, float32_t, float32_t)          \
    F(B200WMMA_I8, B200WMMA_I32, B200WMMA_I32, int8_t, int32_t, int32_t)                   \
    F(B200WMMA_I8, B200WMMA_I8, B200WMMA_I32, int8_t, int8_t, int32_t)                     \
    F(B200WMMA_F32, B200WMMA_F32, B200WMMA_F32, float32_t, float32_t, float32_t)           \
    F(B200WMMA_XF32, B200WMMA_F32, B200WMMA_F32, xfloat32_t, float32_t, float32_t)         \
    F(B200WMMA_F64, B200WMMA_F64, B200WMMA_F64, float64_t, float64_t, float64_t)

    // The usual K extent of a fragment: 16 everywhere except 32x32 tiles of 8-bit types.
    template <typename InT>
    constexpr uint32_t defaultBlockK(uint32_t block)
    {
        return (sizeof(InT) == 1 && block == 32) ? 32u : 16u;
    }

    // Launches with a K extent other than the usual one (simple_gemm_blockk.cu);
    // B200WMMA_ERR_UNSUPPORTED for a combination that is not built.
    int launchOtherBlockK(int in_dtype, int out_dtype, int compute_dtype, int block, int block_k,
                          Args const& g);
} // namespace simple
} // namespace b200wmma
#endif
