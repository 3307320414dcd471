// Fused DLRM dot-interaction forward and backward for B200.
//
// Reference (paths in the rocWMMA tree): forward samples/simple_dlrm.cpp:184-284,
// backward :290-441, host routines test/reference_impl.hpp:83-179.  The reference
// runs one 16x16 tile per warp with grid.z = batch, writes the m x m product to a
// global scratch array, gathers the triangle from it, and for the backward pass
// launches a separate kernel (plus a host synchronisation) to rebuild the symmetric
// gradient matrix.  Both passes move ~8 bytes per flop-pair of useful work and are
// bound by HBM bandwidth, so here each pass is ONE kernel that touches every input
// and output byte exactly once:
//
//   * a warp owns whole samples, handed out in groups of eight consecutive ones; the
//     packed [k + m(m-1)/2]-wide rows are only 2-byte aligned, so the forward pass stages
//     a row at the offset from a 16-byte boundary that it has in global memory and writes
//     all but its first and last few values with 128-bit stores;
//   * samples stream through a per-warp cp.async ring in shared memory (16-byte pieces into
//     rows padded by 16 bytes, so that ldmatrix is conflict-free).  Bulk copies
//     (cp.async.bulk) per 256-byte row, for the loads or for the gradient, were slower
//     than 16-byte cp.async / 128-bit stores: the copy engine took about 17 cycles per
//     request;
//   * the m x m (forward) and m x k (backward) products run on warp-level tensor-core
//     instructions (mma.sync m16n8k16, fp32 accumulate) with m padded to 32 by a shared
//     row of zeros; nothing is written to global scratch;
//   * forward: X X^T needs only A fragments -- the B operand of block (i, j) is a
//     re-labelling of the A registers of block j; only blocks on or below the diagonal
//     are computed;
//   * backward: the symmetric matrix G is rebuilt in shared memory (stored in fp16 as
//     the host routine does), G X overwrites the sample's own ring slot column block
//     by column block.
//
// Limits: fp16, m <= 32, k a multiple of 16 and <= 256, pointers 16-byte aligned.
#include "common.cuh"
#include "runtime.cuh"
#include <cstdlib>
#include <cuda_fp16.h>

namespace
{
    constexpr uint32_t GROUP      = 8; // samples per aligned group
    constexpr uint32_t MAX_K      = 256;
    constexpr uint32_t G_LD       = 40; // halves per row of the 32x32 G tile (80 bytes)
    // Warps per block.  The backward pass cannot have more (168 registers per thread); the
    // forward pass could (shared memory allows 14 at 27 x 128) but measured best at 11-12:
    // 5.28, 5.68, 5.69, 5.56, 5.39 TB/s with 10, 11, 12, 13, 14 warps.
    constexpr uint32_t MAX_WARPS  = 12;
    constexpr uint32_t ZERO_BYTES = MAX_K * 2 + 16;

    __device__ inline uint32_t smemAddr(void const* p)
    {
        return static_cast<uint32_t>(__cvta_generic_to_shared(p));
    }
    __device__ inline void cpAsync16(uint32_t dst, void const* src)
    {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
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
    __device__ inline void ldmatrixX4(uint32_t (&r)[4], uint32_t addr)
    {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                     : "r"(addr)
                     : "memory");
    }
    __device__ inline void ldmatrixX4Trans(uint32_t (&r)[4], uint32_t addr)
    {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                     : "r"(addr)
                     : "memory");
    }
    __device__ inline void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                    uint32_t a3, uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    // The same with a zero accumulator on input: the first product of a chain needs no
    // cleared registers.
    __device__ inline void mma16816z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                     uint32_t a3, uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    }
    template <bool FIRST>
    __device__ inline void mmaStep(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1)
    {
        if constexpr(FIRST)
            mma16816z(d, a[0], a[1], a[2], a[3], b0, b1);
        else
            mma16816(d, a[0], a[1], a[2], a[3], b0, b1);
    }

    // Predicated shared-memory stores.  Written as predicated instructions on purpose: as
    // `if(p) *ptr = v` the compiler at times emitted a divergent branch with a reconvergence
    // point around every store of an unrolled epilogue, a third more instructions overall.
    __device__ inline void stSharedIf(uint32_t addr, uint32_t v, bool p)
    {
        asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t@q st.shared.b32 [%0], %1;\n\t}"
                     ::"r"(addr), "r"(v), "r"(uint32_t(p))
                     : "memory");
    }
    __device__ inline void stSharedIf(uint32_t addr, __half v, bool p)
    {
        asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t@q st.shared.b16 [%0], %1;\n\t}"
                     ::"r"(addr), "h"(__half_as_ushort(v)), "r"(uint32_t(p))
                     : "memory");
    }

    struct TrueT
    {
        static constexpr bool value = true;
    };
    struct FalseT
    {
        static constexpr bool value = false;
    };

    struct Shape
    {
        uint32_t m, k, batch;
        uint32_t outLen; // k + m(m-1)/2
        uint32_t rowStride; // bytes per staged sample row: 2k + 16
        uint32_t stageBytes; // m * rowStride
        uint32_t numGroups; // ceil(batch / 8)
    };

    // Programmatic dependent launch: block until the previous kernel of the stream has
    // completed, then let the next one be scheduled (it waits at the same place).
    __device__ inline void gridDependencyWait()
    {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    // Work distribution: groups of 8 samples are handed out through one global counter, so
    // a warp that finishes early simply takes the next group (a fixed round-robin deal left
    // the slowest warp one group -- up to 8 % of the run -- behind the rest).  A warp walks
    // its samples as a sequence q = 0, 1, 2, ...; the feed knows the group of the current
    // eight and of the next eight, which is as far ahead as the prefetch looks.
    struct GroupFeed
    {
        unsigned int* counter;
        uint32_t      numGroups;
        uint32_t      lastTicket;
        uint32_t      g0, g1; // groups of q in [base, base + 8) and [base + 8, base + 16)
        uint32_t      base;

        // Every warp of the grid draws tickets until its first one past the end and then
        // stops, so exactly numGroups + (warps of the grid) tickets are drawn per launch.
        // Whoever draws the last one puts the counter back to zero for the launch that
        // uses it next: no memset sits between two kernels of a stream.
        __device__ inline uint32_t fetch(uint32_t lane)
        {
            uint32_t v = 0;
            if(lane == 0)
            {
                v = atomicAdd(counter, 1u);
                if(v == lastTicket)
                    atomicExch(counter, 0u);
            }
            return __shfl_sync(0xffffffffu, v, 0);
        }
        __device__ inline void init(unsigned int* c, uint32_t groups, uint32_t lane)
        {
            counter    = c;
            numGroups  = groups;
            lastTicket = groups + gridDim.x * (blockDim.x / 32u) - 1u;
            base       = 0;
            g0        = fetch(lane);
            g1        = g0 < numGroups ? fetch(lane) : numGroups;
        }
        // Called with q == base + 8: the next eight become the current eight.
        __device__ inline void advance(uint32_t lane)
        {
            g0 = g1;
            g1 = g0 < numGroups ? fetch(lane) : numGroups;
            base += GROUP;
        }
        __device__ inline bool done() const
        {
            return g0 >= numGroups;
        }
        // Sample index of sequence position q (base <= q < base + 16), or ~0u past the end.
        __device__ inline uint32_t sample(uint32_t q) const
        {
            const uint32_t grp = (q - base) < GROUP ? g0 : g1;
            return grp < numGroups ? grp * GROUP + (q % GROUP) : 0xffffffffu;
        }
    };

    // Bytes of the backward pass's triangle table: 4 per entry, rounded up to 16.
    __host__ __device__ inline uint32_t triTableBytes(uint32_t m)
    {
        return (m * (m - 1) / 2 * 4 + 15) / 16 * 16;
    }

    // Forward pass: staging for one packed output row, placed up to 14 bytes into the
    // buffer so that it has the alignment it will have in global memory.
    __host__ __device__ inline uint32_t fwdStagingBytes(uint32_t outLen)
    {
        return (outLen * 2u + 14u + 15u) / 16u * 16u;
    }

    // One warp's ring of staged samples.  A sample is m rows of k halves, contiguous in
    // global memory; in a slot its rows are rowStride bytes apart.  A lane moves the 16-byte
    // pieces lane, lane + 32, ...; the slot offset of piece c needs c / chunksPerRow, which
    // is (c * magic) >> 16 -- exact for c < 2048 and chunksPerRow <= 32 with
    // magic = ceil(65536 / chunksPerRow); a sample has at most 32 * 256 / 8 = 1024 pieces.
    // Every fill is one cp.async group (an empty one past the end of the batch), so that
    // "all but the newest NSTAGES - 2 groups have landed" always means "the oldest slot is
    // full".
    template <uint32_t NSTAGES>
    struct Ring
    {
        uint32_t slot0, stageBytes;
        uint32_t chunksPerRow, magic, rowStride, chunks;

        __device__ inline void init(uint32_t ringAddr, Shape const& sh)
        {
            slot0        = ringAddr;
            stageBytes   = sh.stageBytes;
            chunksPerRow = sh.k / 8;
            magic        = (65536u + chunksPerRow - 1u) / chunksPerRow;
            rowStride    = sh.rowStride;
            chunks       = sh.m * chunksPerRow;
        }
        __device__ inline uint32_t slotAddr(uint32_t s) const
        {
            return slot0 + s * stageBytes;
        }
        // Slot offset of a sample's c-th 16-byte piece.
        __device__ inline uint32_t offset(uint32_t c) const
        {
            const uint32_t row = (c * magic) >> 16;
            return row * rowStride + (c - row * chunksPerRow) * 16u;
        }
        __device__ inline void fill(uint32_t s, __half const* sample, uint32_t lane) const
        {
            uint8_t const* src = reinterpret_cast<uint8_t const*>(sample);
            const uint32_t dst = slotAddr(s);
            for(uint32_t c = lane; c < chunks; c += 32)
                cpAsync16(dst + offset(c), src + size_t(c) * 16);
        }
        // The oldest fill still outstanding has landed, for every lane of the warp.
        __device__ inline void waitOldest() const
        {
            cpAsyncWait<NSTAGES - 2>();
            __syncwarp();
        }
    };

    // =====================================================================================
    // forward
    // =====================================================================================
    template <uint32_t NSTAGES>
    __global__ void __launch_bounds__(MAX_WARPS * 32, 1)
        dlrmFwdKernel(__half const* __restrict__ input, __half* __restrict__ output, Shape sh,
                      unsigned int* counter)
    {
        extern __shared__ __align__(16) uint8_t smem[];
        const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
        const uint32_t g = lane >> 2, t = lane & 3;

        // layout: [zero row][warp 0: ring slots, out staging][warp 1: ...]
        const uint32_t perWarp       = NSTAGES * sh.stageBytes + fwdStagingBytes(sh.outLen);
        uint8_t*       zeroRow       = smem;
        uint8_t*       mine          = smem + ZERO_BYTES + warp * perWarp;
        __half*        outStage      = reinterpret_cast<__half*>(mine + NSTAGES * sh.stageBytes);
        const uint32_t zeroAddr      = smemAddr(zeroRow);

        for(uint32_t i = threadIdx.x; i < ZERO_BYTES / 4; i += blockDim.x)
            reinterpret_cast<uint32_t*>(zeroRow)[i] = 0u;
        Ring<NSTAGES> ring;
        ring.init(smemAddr(mine), sh);
        __syncthreads();

        // Nothing above touches global memory: it may run while the previous kernel of the
        // stream drains.  From here on that kernel's results (and the work counter) are read.
        gridDependencyWait();

        const bool twoM = sh.m > 16;
        GroupFeed  feed;
        feed.init(counter, sh.numGroups, lane);

        // Where this lane's accumulator elements go in a packed output row.  Element pair h
        // of block i sits at row r = 16 mt + g + 8 h, columns c and c + 1 (c = 8 nt + 2 t);
        // only c < r < m is part of the strict lower triangle.  Bits 0-15: index of (r, c)
        // in the row, bit 16 / 17: (r, c) / (r, c + 1) is stored.
        uint32_t triSlot[6][2];
#pragma unroll
        for(uint32_t i = 0; i < 6; ++i)
#pragma unroll
            for(uint32_t h = 0; h < 2; ++h)
            {
                const uint32_t mt = i < 2 ? 0u : 1u;
                const uint32_t nt = i < 2 ? i : i - 2u;
                const uint32_t r  = mt * 16u + g + 8u * h;
                const uint32_t c  = nt * 8u + 2u * t;
                uint32_t       v  = sh.k + r * (r - 1u) / 2u + c;
                if(r < sh.m && c < r)
                    v |= 1u << 16;
                if(r < sh.m && c + 1u < r)
                    v |= 1u << 17;
                triSlot[i][h] = v;
            }

        auto fill = [&](uint32_t q) {
            const uint32_t s = feed.sample(q);
            if(s < sh.batch)
                ring.fill(q % NSTAGES, input + size_t(s) * sh.m * sh.k, lane);
            cpAsyncCommit();
        };
#pragma unroll
        for(uint32_t q = 0; q < NSTAGES - 1; ++q)
            fill(q);

        // ldmatrix row addresses of this lane inside a slot: matrix (lane / 8) of the x4 group
        // is rows (lane/8 & 1) * 8 ..., column block (lane / 16) * 8; rows >= m read zeros.
        const uint32_t lmRow = ((lane >> 3) & 1u) * 8u + (lane & 7u);
        const uint32_t lmCol = (lane >> 4) * 8u;

        for(uint32_t q = 0;; ++q)
        {
            if(q - feed.base == GROUP)
                feed.advance(lane);
            if(feed.done())
                break;
            // sample q has landed, and every lane is done with the slot the next fill overwrites
            ring.waitOldest();
            fill(q + NSTAGES - 1);

            const uint32_t sample = feed.sample(q);
            if(sample < sh.batch)
            {
                const uint32_t slotAddr = ring.slotAddr(q % NSTAGES);
                float          acc[6][4];
                const uint32_t row0 = lmRow, row1 = 16u + lmRow;
                const uint32_t base0 = row0 < sh.m ? slotAddr + row0 * sh.rowStride : zeroAddr;
                const uint32_t base1 = row1 < sh.m ? slotAddr + row1 * sh.rowStride : zeroAddr;
                auto kStep = [&](auto first, uint32_t kk) {
                    constexpr bool FIRST = decltype(first)::value;
                    uint32_t       a[4], b[4];
                    ldmatrixX4(a, base0 + (kk + lmCol) * 2);
                    // blocks (0,0) and (0,1): B operands are A's own registers
                    mmaStep<FIRST>(acc[0], a, a[0], a[2]);
                    mmaStep<FIRST>(acc[1], a, a[1], a[3]);
                    if(twoM)
                    {
                        ldmatrixX4(b, base1 + (kk + lmCol) * 2);
                        mmaStep<FIRST>(acc[2], b, a[0], a[2]);
                        mmaStep<FIRST>(acc[3], b, a[1], a[3]);
                        mmaStep<FIRST>(acc[4], b, b[0], b[2]);
                        mmaStep<FIRST>(acc[5], b, b[1], b[3]);
                    }
                };
                kStep(TrueT{}, 0u);
                for(uint32_t kk = 16; kk < sh.k; kk += 16)
                    kStep(FalseT{}, kk);

                // The packed row of a sample starts on a 2-byte boundary only.  It is staged
                // at the same offset from a 16-byte boundary as it has in global memory, so
                // that all but its first and last few values leave with 128-bit stores.
                const size_t   gByte = size_t(sample) * sh.outLen * 2u;
                const uint32_t shift = uint32_t(gByte) & 15u;
                // row 0 of the sample, then the strict lower triangle
                __half*       dst   = outStage + shift / 2u;
                __half const* row0p = reinterpret_cast<__half const*>(
                    mine + (q % NSTAGES) * sh.stageBytes);
                for(uint32_t j = lane; j < sh.k; j += 32)
                    dst[j] = row0p[j];
                const uint32_t dstAddr = smemAddr(dst);
#pragma unroll
                for(uint32_t i = 0; i < 6; ++i)
#pragma unroll
                    for(uint32_t h = 0; h < 2; ++h)
                    {
                        const uint32_t v = triSlot[i][h], at = dstAddr + (v & 0xffffu) * 2u;
                        stSharedIf(at, __float2half_rn(acc[i][2 * h]), (v >> 16) & 1u);
                        stSharedIf(at + 2u, __float2half_rn(acc[i][2 * h + 1]), (v >> 17) & 1u);
                    }
                __syncwarp();

                // flush: up to 7 single values, 16-byte pieces, up to 7 single values
                uint8_t*       gptr  = reinterpret_cast<uint8_t*>(output) + gByte;
                uint8_t const* sptr  = reinterpret_cast<uint8_t const*>(dst);
                const uint32_t total = sh.outLen * 2u;
                const uint32_t head  = min((16u - shift) & 15u, total);
                const uint32_t body  = (total - head) / 16u;
                const uint32_t tail  = (total - head) % 16u;
                if(lane < head / 2u)
                    reinterpret_cast<__half*>(gptr)[lane] = reinterpret_cast<__half const*>(sptr)[lane];
                for(uint32_t c = lane; c < body; c += 32)
                    reinterpret_cast<uint4*>(gptr + head)[c]
                        = reinterpret_cast<uint4 const*>(sptr + head)[c];
                if(lane < tail / 2u)
                    reinterpret_cast<__half*>(gptr + head + body * 16u)[lane]
                        = reinterpret_cast<__half const*>(sptr + head + body * 16u)[lane];
                // (the next iteration's __syncwarp orders these reads before the next row)
            }
        }
        cpAsyncWait<0>();
    }

    // =====================================================================================
    // backward
    // =====================================================================================
    template <uint32_t NSTAGES>
    __global__ void __launch_bounds__(MAX_WARPS * 32, 1)
        dlrmBwdKernel(__half const* __restrict__ input, __half const* __restrict__ upstream,
                      __half* __restrict__ grad, __half* __restrict__ mlpGrad, Shape sh,
                      unsigned int* counter)
    {
        extern __shared__ __align__(16) uint8_t smem[];
        const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
        const uint32_t g = lane >> 2, t = lane & 3;

        // layout: [zero row][triangle table][warp 0: ring, G][warp 1: ...]
        const uint32_t triCount = sh.m * (sh.m - 1) / 2;
        const uint32_t triBytes = triTableBytes(sh.m);
        const uint32_t gBytes   = 32 * G_LD * 2;
        const uint32_t perWarp  = NSTAGES * sh.stageBytes + gBytes;
        uint8_t*       zeroRow  = smem;
        uint32_t*      tri      = reinterpret_cast<uint32_t*>(smem + ZERO_BYTES);
        uint8_t*       mine     = smem + ZERO_BYTES + triBytes + warp * perWarp;
        __half*        gTile    = reinterpret_cast<__half*>(mine + NSTAGES * sh.stageBytes);
        const uint32_t zeroAddr = smemAddr(zeroRow);
        const uint32_t gAddr    = smemAddr(gTile);

        for(uint32_t i = threadIdx.x; i < ZERO_BYTES / 4; i += blockDim.x)
            reinterpret_cast<uint32_t*>(zeroRow)[i] = 0u;
        // Packed triangle entry idx is G(r, c), c < r, row-major over r: its two places in
        // the G tile, (r, c) in the low and (c, r) in the high 16 bits.
        for(uint32_t r = threadIdx.x; r < sh.m; r += blockDim.x)
            for(uint32_t c = 0; c < r; ++c)
                tri[r * (r - 1) / 2 + c] = (r * G_LD + c) | ((c * G_LD + r) << 16);
        for(uint32_t i = lane; i < 32 * G_LD / 2; i += 32)
            reinterpret_cast<uint32_t*>(gTile)[i] = 0u; // diagonal and padding stay zero
        Ring<NSTAGES> ring;
        ring.init(smemAddr(mine), sh);
        __syncthreads();

        // Nothing above touches global memory: it may run while the previous kernel of the
        // stream drains.  From here on that kernel's results (and the work counter) are read.
        gridDependencyWait();

        const bool twoM = sh.m > 16;
        GroupFeed  feed;
        feed.init(counter, sh.numGroups, lane);

        auto fill = [&](uint32_t q) {
            const uint32_t s = feed.sample(q);
            if(s < sh.batch)
                ring.fill(q % NSTAGES, input + size_t(s) * sh.m * sh.k, lane);
            cpAsyncCommit();
        };

        // The packed upstream row of a sample is only 2-byte aligned, and each value is used
        // once, so it never goes through shared memory: a lane reads its share of the NEXT
        // sample's row (entries lane, lane+32, ... of the first k values and of the triangle)
        // into registers one iteration ahead, so that no instruction of the current sample
        // waits for a load from global memory; a warp-wide 2-byte load covers 64 contiguous
        // bytes.
        constexpr uint32_t TRI_REGS = 16; // ceil(496 / 32) for m = 32
        constexpr uint32_t MLP_REGS = MAX_K / 32;
        __half             triNext[TRI_REGS], mlpNext[MLP_REGS];
        auto prefetchUpstream = [&](uint32_t q) {
            const uint32_t s = feed.sample(q);
            if(s < sh.batch)
            {
                __half const* src = upstream + size_t(s) * sh.outLen;
#pragma unroll
                for(uint32_t i = 0; i < MLP_REGS; ++i)
                {
                    const uint32_t idx = i * 32u + lane;
                    if(idx < sh.k)
                        mlpNext[i] = src[idx];
                }
#pragma unroll
                for(uint32_t i = 0; i < TRI_REGS; ++i)
                {
                    const uint32_t idx = i * 32u + lane;
                    if(idx < triCount)
                        triNext[i] = src[sh.k + idx];
                }
            }
        };

#pragma unroll
        for(uint32_t q = 0; q < NSTAGES - 1; ++q)
            fill(q);
        prefetchUpstream(0);

        const uint32_t lmRow = ((lane >> 3) & 1u) * 8u + (lane & 7u);
        const uint32_t lmCol = (lane >> 4) * 8u;

        for(uint32_t q = 0;; ++q)
        {
            if(q - feed.base == GROUP)
                feed.advance(lane);
            if(feed.done())
                break;
            const uint32_t sample = feed.sample(q);
            if(sample >= sh.batch)
                continue; // padding of the batch's last group; nothing follows it
            ring.waitOldest();
            fill(q + NSTAGES - 1);
            uint8_t*       slotPtr  = mine + (q % NSTAGES) * sh.stageBytes;
            const uint32_t slotAddr = ring.slotAddr(q % NSTAGES);

            // bottom-MLP gradient: the first k upstream values (fetched one iteration ago),
            // copied as they are
            {
                __half* dst = mlpGrad + size_t(sample) * sh.k;
#pragma unroll
                for(uint32_t i = 0; i < MLP_REGS; ++i)
                {
                    const uint32_t idx = i * 32u + lane;
                    if(idx < sh.k)
                        dst[idx] = mlpNext[i];
                }
            }

            // symmetric G (fp16, zero diagonal) from the packed triangle
#pragma unroll
            for(uint32_t i = 0; i < TRI_REGS; ++i)
            {
                const uint32_t idx = i * 32u + lane;
                if(idx < triCount)
                {
                    const uint32_t at = tri[idx];
                    gTile[at & 0xffffu] = triNext[i];
                    gTile[at >> 16]     = triNext[i];
                }
            }
            __syncwarp();
            // the registers are free again: start on the next sample's row
            prefetchUpstream(q + 1);

            // A fragments of G: [mt][kt]
            uint32_t ga[2][2][4];
            ldmatrixX4(ga[0][0], gAddr + (lmRow * G_LD + lmCol) * 2);
            if(twoM)
            {
                ldmatrixX4(ga[0][1], gAddr + (lmRow * G_LD + 16 + lmCol) * 2);
                ldmatrixX4(ga[1][0], gAddr + ((16 + lmRow) * G_LD + lmCol) * 2);
                ldmatrixX4(ga[1][1], gAddr + ((16 + lmRow) * G_LD + 16 + lmCol) * 2);
            }

            // B = X read k-row by k-row (transposing ldmatrix); rows >= m are zeros
            const uint32_t kr0 = lmRow, kr1 = 16u + lmRow;
            const uint32_t xb0 = kr0 < sh.m ? slotAddr + kr0 * sh.rowStride : zeroAddr;
            const uint32_t xb1 = kr1 < sh.m ? slotAddr + kr1 * sh.rowStride : zeroAddr;

            for(uint32_t n0 = 0; n0 < sh.k; n0 += 64)
            {
                const uint32_t pairs = min(4u, (sh.k - n0) / 16u); // 16 columns per ldmatrix.x4
                float          acc[2][8][4];
                // Two passes over the column block, one per half of the k rows, so that the
                // two products that add into one accumulator are sixteen instructions apart.
#pragma unroll
                for(uint32_t p = 0; p < 4; ++p)
                {
                    if(p < pairs)
                    {
                        uint32_t xb[4];
                        ldmatrixX4Trans(xb, xb0 + (n0 + p * 16u + lmCol) * 2u); // k rows 0..15
                        mmaStep<true>(acc[0][2 * p], ga[0][0], xb[0], xb[1]);
                        mmaStep<true>(acc[0][2 * p + 1], ga[0][0], xb[2], xb[3]);
                        if(twoM)
                        {
                            mmaStep<true>(acc[1][2 * p], ga[1][0], xb[0], xb[1]);
                            mmaStep<true>(acc[1][2 * p + 1], ga[1][0], xb[2], xb[3]);
                        }
                    }
                }
                if(twoM)
                {
#pragma unroll
                    for(uint32_t p = 0; p < 4; ++p)
                    {
                        if(p < pairs)
                        {
                            uint32_t xb[4];
                            ldmatrixX4Trans(xb, xb1 + (n0 + p * 16u + lmCol) * 2u); // k rows 16..31
                            mmaStep<false>(acc[0][2 * p], ga[0][1], xb[0], xb[1]);
                            mmaStep<false>(acc[0][2 * p + 1], ga[0][1], xb[2], xb[3]);
                            mmaStep<false>(acc[1][2 * p], ga[1][1], xb[0], xb[1]);
                            mmaStep<false>(acc[1][2 * p + 1], ga[1][1], xb[2], xb[3]);
                        }
                    }
                }
                // This column block of X is not needed any more: overwrite it with the result.
                __syncwarp();
#pragma unroll
                for(uint32_t mt = 0; mt < 2; ++mt)
                {
                    if(mt == 0 || twoM)
                    {
#pragma unroll
                        for(uint32_t h = 0; h < 2; ++h)
                        {
                            const uint32_t r    = mt * 16u + g + 8u * h;
                            const bool     live = r < sh.m;
                            const uint32_t at   = slotAddr + r * sh.rowStride + (n0 + 2u * t) * 2u;
#pragma unroll
                            for(uint32_t nb = 0; nb < 8; ++nb)
                            {
                                if(nb < 2 * pairs)
                                {
                                    const __half2 v = __floats2half2_rn(acc[mt][nb][2 * h],
                                                                        acc[mt][nb][2 * h + 1]);
                                    stSharedIf(at + nb * 16u,
                                               *reinterpret_cast<uint32_t const*>(&v), live);
                                }
                            }
                        }
                    }
                }
            }

            __syncwarp();

            // The result leaves with 128-bit stores (the sample is contiguous in grad).  One
            // bulk copy per 256-byte row instead was slower, as it was for the loads.
            {
                uint4* gdst = reinterpret_cast<uint4*>(grad + size_t(sample) * sh.m * sh.k);
                for(uint32_t c = lane; c < ring.chunks; c += 32)
                    gdst[c] = *reinterpret_cast<uint4 const*>(slotPtr + ring.offset(c));
            }
            // (the next iteration's __syncwarp orders these reads before the slot's refill)
        }
        cpAsyncWait<0>();
    }

    int checkShape(int dtype, void const* p0, void const* p1, uint32_t m, uint32_t k,
                   uint32_t batch, Shape* sh)
    {
        if(!p0 || !p1 || m == 0 || k == 0 || batch == 0)
            return B200WMMA_ERR_INVALID_ARG;
        if(dtype != B200WMMA_F16)
            return B200WMMA_ERR_UNSUPPORTED;
        if(m > 32 || m < 2 || k % 16 != 0 || k > MAX_K)
            return B200WMMA_ERR_UNSUPPORTED;
        sh->m          = m;
        sh->k          = k;
        sh->batch      = batch;
        sh->outLen     = k + m * (m - 1) / 2;
        sh->rowStride  = 2 * k + 16;
        sh->stageBytes = m * sh->rowStride;
        sh->numGroups  = (batch + GROUP - 1) / GROUP;
        return B200WMMA_OK;
    }

    inline bool aligned16(void const* p)
    {
        return reinterpret_cast<uintptr_t>(p) % 16 == 0;
    }

    constexpr uint32_t SMEM_LIMIT = 227 * 1024;

    // Warps per block and ring depth: as many bytes in flight as shared memory allows.
    struct Plan
    {
        uint32_t warps = 0, stages = 0, smemBytes = 0;
    };
    // With one sample per warp every dependent latency inside a sample is hidden only by
    // other warps, so warps count first; a second ring slot is all a warp needs to keep a
    // load in flight while it computes, a third helps when few warps fit.
    // B200WMMA_DLRM_STAGES / B200WMMA_DLRM_WARPS override the choice (tuning only).
    Plan choosePlan(uint32_t fixedBytes, uint32_t stageBytes, uint32_t otherPerWarp,
                    uint32_t maxWarps)
    {
        const char* es = getenv("B200WMMA_DLRM_STAGES");
        const char* ew = getenv("B200WMMA_DLRM_WARPS");
        const uint32_t forceStages = es ? uint32_t(atoi(es)) : 0u;
        const uint32_t forceWarps  = ew ? uint32_t(atoi(ew)) : 0u;
        Plan best;
        for(uint32_t stages = 2; stages <= 3; ++stages)
        {
            if(forceStages && stages != forceStages)
                continue;
            const uint32_t perWarp = stages * stageBytes + otherPerWarp;
            if(fixedBytes + perWarp > SMEM_LIMIT)
                continue;
            uint32_t warps = (SMEM_LIMIT - fixedBytes) / perWarp;
            warps          = warps > maxWarps ? maxWarps : warps;
            if(forceWarps && forceWarps < warps)
                warps = forceWarps;
            // 3 slots only if that costs no warps
            if(warps > best.warps || (warps == best.warps && stages > best.stages))
            {
                best.warps     = warps;
                best.stages    = stages;
                best.smemBytes = fixedBytes + warps * perWarp;
            }
        }
        return best;
    }

    // Opts the kernel in to the large dynamic shared-memory carve-out.
    template <typename KernelT>
    int prepare(KernelT kernel)
    {
        B200WMMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               int(SMEM_LIMIT)));
        return B200WMMA_OK;
    }
} // namespace

extern "C" int b200wmma_dlrm_fwd(int dtype, const void* input, void* output, uint32_t m, uint32_t k,
                                 uint32_t batch, void* stream)
{
    Shape sh;
    int   rc = checkShape(dtype, input, output, m, k, batch, &sh);
    if(rc != B200WMMA_OK)
        return rc;
    if(!aligned16(input) || !aligned16(output))
        return B200WMMA_ERR_ALIGNMENT;
    const Plan plan
        = choosePlan(ZERO_BYTES, sh.stageBytes, fwdStagingBytes(sh.outLen), MAX_WARPS);
    if(plan.warps == 0)
        return B200WMMA_ERR_UNSUPPORTED;
    const int sms = b200wmma::smCount();
    if(sms <= 0)
        return B200WMMA_ERR_CUDA;
    const uint32_t wanted = (sh.numGroups + plan.warps - 1) / plan.warps;
    const uint32_t grid   = wanted < uint32_t(sms) ? wanted : uint32_t(sms);
    auto           s      = static_cast<cudaStream_t>(stream);
    auto           in     = static_cast<__half const*>(input);
    auto           out    = static_cast<__half*>(output);
    unsigned int*  ctr    = b200wmma::launchCounter(s);
    if(!ctr)
        return B200WMMA_ERR_CUDA;
    cudaError_t launchErr = cudaSuccess;
    if(plan.stages == 3)
    {
        if((rc = prepare(dlrmFwdKernel<3>)) != B200WMMA_OK)
            return rc;
        launchErr = b200wmma::launchOverlapped(dlrmFwdKernel<3>, dim3(grid), dim3(plan.warps * 32),
                                               plan.smemBytes, s, in, out, sh, ctr);
    }
    else
    {
        if((rc = prepare(dlrmFwdKernel<2>)) != B200WMMA_OK)
            return rc;
        launchErr = b200wmma::launchOverlapped(dlrmFwdKernel<2>, dim3(grid), dim3(plan.warps * 32),
                                               plan.smemBytes, s, in, out, sh, ctr);
    }
    return b200wmma::cudaToStatus(launchErr);
}

extern "C" int b200wmma_dlrm_bwd(int dtype, const void* input, const void* upstream, void* grad,
                                 void* mlp_grad, uint32_t m, uint32_t k, uint32_t batch,
                                 void* stream)
{
    Shape sh;
    int   rc = checkShape(dtype, input, upstream, m, k, batch, &sh);
    if(rc != B200WMMA_OK)
        return rc;
    if(!grad || !mlp_grad)
        return B200WMMA_ERR_INVALID_ARG;
    if(!aligned16(input) || !aligned16(upstream) || !aligned16(grad) || !aligned16(mlp_grad))
        return B200WMMA_ERR_ALIGNMENT;
    const Plan plan
        = choosePlan(ZERO_BYTES + triTableBytes(m), sh.stageBytes, 32 * G_LD * 2, MAX_WARPS);
    if(plan.warps == 0)
        return B200WMMA_ERR_UNSUPPORTED;
    const int sms = b200wmma::smCount();
    if(sms <= 0)
        return B200WMMA_ERR_CUDA;
    const uint32_t wanted = (sh.numGroups + plan.warps - 1) / plan.warps;
    const uint32_t grid   = wanted < uint32_t(sms) ? wanted : uint32_t(sms);
    auto           s      = static_cast<cudaStream_t>(stream);
    auto           in     = static_cast<__half const*>(input);
    auto           up     = static_cast<__half const*>(upstream);
    auto           g      = static_cast<__half*>(grad);
    auto           mg     = static_cast<__half*>(mlp_grad);
    unsigned int*  ctr    = b200wmma::launchCounter(s);
    if(!ctr)
        return B200WMMA_ERR_CUDA;
    cudaError_t launchErr = cudaSuccess;
    if(plan.stages == 3)
    {
        if((rc = prepare(dlrmBwdKernel<3>)) != B200WMMA_OK)
            return rc;
        launchErr = b200wmma::launchOverlapped(dlrmBwdKernel<3>, dim3(grid), dim3(plan.warps * 32),
                                               plan.smemBytes, s, in, up, g, mg, sh, ctr);
    }
    else
    {
        if((rc = prepare(dlrmBwdKernel<2>)) != B200WMMA_OK)
            return rc;
        launchErr = b200wmma::launchOverlapped(dlrmBwdKernel<2>, dim3(grid), dim3(plan.warps * 32),
                                               plan.smemBytes, s, in, up, g, mg, sh, ctr);
    }
    return b200wmma::cudaToStatus(launchErr);
}
