// The one-tile-per-warp GEMM with fragment K extents other than each type's usual one
// (the reference runs BlockK from the per-type minimum up to 128,
// test/gemm/gemm_common_test_params.hpp:51-121 and
// docs/api-reference/api-reference-guide.rst:80-153).  Built here: 8 (16-bit types: the
// reference's minimum for 32x32 blocks), 16, 32 and 64 for 8- and 16-bit types, 128 as well
// for their 16x16 tiles, 4, 8 and 32 for float32_t / xfloat32_t, 4 and 8 for float64_t.  A translation unit of its own only to keep compile times apart.
#include "simple_gemm.cuh"

namespace b200wmma
{
namespace simple
{
    namespace
    {
        template <typename InT, typename OutT, typename CompT, uint32_t BLOCK>
        int launchK(int block_k, Args const& g)
        {
            if constexpr(sizeof(InT) == 8)
            {
                if constexpr(BLOCK == 16)
                {
                    if(block_k == 4)
                        return launchTile<InT, OutT, CompT, 16, 16, 4>(g);
                    if(block_k == 8)
                        return launchTile<InT, OutT, CompT, 16, 16, 8>(g);
                }
            }
            else if constexpr(sizeof(InT) == 4)
            {
                if(block_k == 4)
                    return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 4>(g);
                if(block_k == 8)
                    return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 8>(g);
                if(block_k == 32)
                    return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 32>(g);
            }
            else
            {
                if constexpr(sizeof(InT) == 2)
                {
                    if(block_k == 8)
                        return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 8>(g);
                }
                if(block_k == 16)
                    return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 16>(g);
                if(block_k == 32)
                    return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 32>(g);
                if(block_k == 64)
                    return launchTile<InT, OutT, CompT, BLOCK, BLOCK, 64>(g);
                if constexpr(BLOCK == 16)
                {
                    if(block_k == 128)
                        return launchTile<InT, OutT, CompT, 16, 16, 128>(g);
                }
            }
            return B200WMMA_ERR_UNSUPPORTED;
        }
    } // namespace

    int launchOtherBlockK(int in_dtype, int out_dtype, int compute_dtype, int block, int block_k,
                          Args const& g)
    {
#define B200WMMA_BLOCKK_CASE(I, O, C, IT, OT, CT)                         \
    if(in_dtype == I && out_dtype == O && compute_dtype == C)             \
    {                                                                     \
        if(block == 16)                                                   \
            return launchK<IT, OT, CT, 16>(block_k, g);                   \
        if(block == 32)                                                   \
            return launchK<IT, OT, CT, 32>(block_k, g);                   \
        return B200WMMA_ERR_UNSUPPORTED;                                  \
    }
        B200WMMA_SIMPLE_TRIPLES(B200WMMA_BLOCKK_CASE)
#undef B200WMMA_BLOCKK_CASE
        return B200WMMA_ERR_UNSUPPORTED;
    }
} // namespace simple
} // namespace b200wmma
