"""Kernel sources for the run-time compilation tests (strings handed to NVRTC)."""

# A GEMM on the fragment API written for these tests: bf16 inputs (A row-major, B
# column-major), fp32 accumulate and fp32 row-major C / D, one 32 x 32 output tile per warp
# built from 32 x 32 x 16 fragments, warps laid out as (blockDim.x / 32) x blockDim.y.
TILE32_BF16_GEMM = r"""
#include <rocwmma/rocwmma.hpp>

namespace w = rocwmma;
constexpr uint32_t TILE = 32, DEPTH = 16;
using FragA = w::fragment<w::matrix_a, TILE, TILE, DEPTH, w::bfloat16_t, w::row_major>;
using FragB = w::fragment<w::matrix_b, TILE, TILE, DEPTH, w::bfloat16_t, w::col_major>;
using FragC = w::fragment<w::accumulator, TILE, TILE, DEPTH, w::float32_t>;

extern "C" __global__ void tile32_gemm(uint32_t rows, uint32_t cols, uint32_t depth,
                                       w::bfloat16_t const* a, w::bfloat16_t const* bT,
                                       w::float32_t const* c, w::float32_t* d, float alpha,
                                       float beta)
{
    const uint32_t warpRow = (blockIdx.x * blockDim.x + threadIdx.x) / w::Constants::AMDGCN_WAVE_SIZE;
    const uint32_t warpCol = blockIdx.y * blockDim.y + threadIdx.y;
    const uint32_t r0 = warpRow * TILE, c0 = warpCol * TILE;
    if(r0 >= rows || c0 >= cols)
        return;
    FragC acc;
    w::fill_fragment(acc, 0.0f);
    for(uint32_t kk = 0; kk < depth; kk += DEPTH)
    {
        FragA fa;
        FragB fb;
        w::load_matrix_sync(fa, a + size_t(r0) * depth + kk, depth);
        w::load_matrix_sync(fb, bT + size_t(c0) * depth + kk, depth);
        w::mma_sync(acc, fa, fb, acc);
    }
    FragC old;
    w::load_matrix_sync(old, c + size_t(r0) * cols + c0, cols, w::mem_row_major);
    for(uint32_t i = 0; i < acc.num_elements; ++i)
        old.x[i] = alpha * acc.x[i] + beta * old.x[i];
    w::store_matrix_sync(d + size_t(r0) * cols + c0, old, cols, w::mem_row_major);
}
"""
