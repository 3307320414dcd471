// C launchers of the one-tile-per-warp GEMM (kernel: simple_gemm.cuh), each type's usual
// fragment K extent.
#include "simple_gemm.cuh"

using namespace b200wmma::simple;

namespace
{
    template <typename InT, typename OutT, typename CompT>
    int launchDefault(int block, Args const& g)
    {
        if(block == 16)
            return launchTile<InT, OutT, CompT, 16, 16, 16>(g);
        if(block == 32)
        {
            // 64-bit fragments exist as 16x16 only, as in the reference
            // (test/gemm/gemm_predicates_base.hpp:137-209).
            if constexpr(sizeof(InT) == 8)
                return B200WMMA_ERR_UNSUPPORTED;
            else if constexpr(sizeof(InT) == 1)
                return launchTile<InT, OutT, CompT, 32, 32, 32>(g);
            else
                return launchTile<InT, OutT, CompT, 32, 32, 16>(g);
        }
        return B200WMMA_ERR_UNSUPPORTED;
    }

    // The compute type a (input, output) pair gets when the caller names none.
    int defaultCompute(int in_dtype)
    {
        return in_dtype == B200WMMA_I8 ? B200WMMA_I32
               : in_dtype == B200WMMA_F64 ? B200WMMA_F64
                                          : B200WMMA_F32;
    }
} // namespace

extern "C" int b200wmma_gemm_simple_ex(int in_dtype, int out_dtype, int compute_dtype, uint32_t m,
                                       uint32_t n, uint32_t k, const void* a, const void* b,
                                       const void* c, void* d, uint32_t lda, uint32_t ldb,
                                       uint32_t ldc, uint32_t ldd, double alpha, double beta,
                                       int layout_a, int layout_b, int layout_cd, int block,
                                       int block_k, void* stream)
{
    if(!a || !b || !c || !d || m == 0 || n == 0 || k == 0)
        return B200WMMA_ERR_INVALID_ARG;
    if(layout_cd != B200WMMA_ROW_MAJOR && layout_cd != B200WMMA_COL_MAJOR)
        return B200WMMA_ERR_INVALID_ARG;
    if(compute_dtype < 0)
        compute_dtype = defaultCompute(in_dtype);
    const Args g{m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b,
                 layout_cd, static_cast<cudaStream_t>(stream)};
#define B200WMMA_SIMPLE_CASE(I, O, C, IT, OT, CT)                                    \
    if(in_dtype == I && out_dtype == O && compute_dtype == C)                        \
    {                                                                                \
        if(block_k == 0 || uint32_t(block_k) == defaultBlockK<IT>(uint32_t(block)))  \
            return launchDefault<IT, OT, CT>(block, g);                              \
        return launchOtherBlockK(in_dtype, out_dtype, compute_dtype, block, block_k, g); \
    }
    B200WMMA_SIMPLE_TRIPLES(B200WMMA_SIMPLE_CASE)
#undef B200WMMA_SIMPLE_CASE
    return B200WMMA_ERR_UNSUPPORTED;
}

extern "C" int b200wmma_gemm_simple(int in_dtype, int out_dtype, uint32_t m, uint32_t n,
                                    uint32_t k, const void* a, const void* b, const void* c,
                                    void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                    uint32_t ldd, double alpha, double beta, int layout_a,
                                    int layout_b, int layout_cd, int block, void* stream)
{
    return b200wmma_gemm_simple_ex(in_dtype, out_dtype, -1, m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
                                   alpha, beta, layout_a, layout_b, layout_cd, block, 0, stream);
}
