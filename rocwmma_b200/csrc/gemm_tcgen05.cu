// Block-cooperative GEMM for B200: D = alpha * A * B + beta * C.
//
// Rebuilds the reference's macro-tile GEMM (samples/perf_hgemm.cpp:518-714: 128x128
// macro tile, cooperative global->LDS staging, two LDS buffers, one barrier per
// 16-deep K step) as a persistent, warp-specialised sm_100a kernel:
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A (128 x BK) and
//               B (256 x BK) tiles into a 4-slot shared-memory ring (128-byte
//               swizzle), one mbarrier pair (full/empty) per slot.  No multicast.
//   warp 1      one elected thread issues tcgen05.mma (M=128, N=256) per 32-byte K
//               step; accumulators live in tensor memory, two buffers of 256
//               columns so the epilogue of tile i overlaps the MMAs of tile i+1.
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (one TMEM lane = one output
//               row per thread), alpha/beta in the compute type, conversion, and
//               128-bit stores along the row.
//
// Row-major A / column-major B are "K-major" tensor-core operands (the layout of the
// 8192^3 benchmark configuration); column-major A / row-major B are read in place as
// MN-major operands for 8- and 16-bit types and transposed into scratch first for 32-bit
// ones.  Tiles at the M/N/K edges rely on TMA zero fill for loads and on masks for stores.
//
// Every mbarrier wait is bounded; when one runs out the block raises an abort
// flag, all roles leave their loops, tensor memory is released, and the kernel
// records the event in the library's device status word.
#include "common.cuh"
#include "runtime.cuh"
#include "tile_schedule.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdlib>
#include <cuda_fp16.h>
#include <atomic>
#include <mutex>
#include <rocwmma/rocwmma_block.hpp>

using namespace rocwmma;
using namespace rocwmma::block;
using b200wmma::TileSchedule;

namespace
{
    constexpr uint32_t BM          = 128;
    constexpr uint32_t BN          = 256;
    constexpr uint32_t ROW_BYTES   = 128; // one swizzle row: BK * sizeof(InT)
    constexpr uint32_t STAGES      = 4;
    constexpr uint32_t A_BYTES     = BM * ROW_BYTES; // 16 KiB
    constexpr uint32_t B_BYTES     = BN * ROW_BYTES; // 32 KiB
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t ACC_BUFS    = 2;
    constexpr uint32_t TMEM_COLS   = ACC_BUFS * BN; // 512
    constexpr uint32_t NUM_THREADS = 192;
    constexpr uint32_t EPI_THREADS = 128;
    constexpr uint32_t GROUP_M     = 16; // most tile rows in a raster band (see bandRows)

    struct SharedControl
    {
        uint64_t   full[STAGES];
        uint64_t   empty[STAGES];
        uint64_t   accFull[ACC_BUFS];
        uint64_t   accEmpty[ACC_BUFS];
        uint32_t   tmemBase;
        AbortState abort;
    };
    // Epilogue staging: two buffers of 128 rows x 32 columns (16 KiB for 4-byte outputs),
    // written by the epilogue threads, read by TMA stores.
    constexpr uint32_t STG_BYTES  = 128 * 128;
    constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 2 * STG_BYTES + 1024 /*alignment slack*/
                                    + sizeof(SharedControl) + 64;

    struct GemmParams
    {
        uint32_t    m, n, k;
        void const* c;
        void*       d;
        uint32_t    ldc, ldd;
        double      alpha, beta;
        uint32_t*   status;
        uint32_t    chunkKB; // k-blocks per accumulation chain; 0 = all of K in one chain
        uint32_t    wide; // 1: rows of C and D are 32-byte aligned (256-bit accesses)
        uint32_t    bn; // tile width (columns of D per tile): 256, or less for the pair kernel
        uint32_t    band; // tile rows per raster band (tiles of a band share their rows of A in L2)
        uint32_t    tmaStore; // 1: D leaves through shared memory and TMA stores
        uint32_t    aMN, bMN; // 1: operand is MN-major in memory (A column-major, B row-major)
        uint32_t    sumInTmem; // 1: chunked accumulation keeps its running sum in tensor memory
        uint32_t    wideCols; // pair kernel: tile columns of width bn ...
        uint32_t    tailCols, bnTail; // ... followed by tailCols columns of width bnTail (0: none)
        uint32_t    snake, mirror; // pair kernel: tile order (TileSchedule)
        uint32_t    prefetch; // pair kernel: k-blocks of the first tile to request into L2 early
        uint32_t    l2Hints; // pair kernel: bit 0 = A evict_last, bit 1 = B evict_first, bit 2 = D
                             // (written once) evict_first
        uint32_t    stagedTail; // pair kernel: a block's last tile leaves through the idle ring
        uint32_t    cViaTma; // pair kernel, beta != 0: bit 0 = C comes in through shared memory by
                             // TMA, bit 1 = C and D pass through L2 marked "evict first"
        uint32_t    splitTiles; // pair kernel: tiles of the last wave cut in two along K
        float*      splitWs; // ... their partial accumulators (raw 32-bit values)
        uint32_t*   splitCtr; // ... and one arrival counter per split tile and block of the pair
    };

    // One operand tile for one K block.  K-major: one TMA box of `rows` rows x 128 bytes of
    // K.  MN-major: boxes of BK K-rows x 128 bytes of M/N, one per 128 bytes of the tile's
    // M/N extent, stacked in shared memory.  Returns the bytes that will arrive.
    // `policy`: an L2 eviction policy for the pair form (0: none).
    template <typename InT, bool PAIR>
    __device__ inline uint32_t loadOperandTile(uint8_t* dst, void const* tmap, uint64_t* bar,
                                               uint32_t barClusterAddr, bool mnMajor,
                                               uint32_t mnOrigin, uint32_t rows, uint32_t k0,
                                               uint64_t policy = 0)
    {
        constexpr uint32_t BK = ROW_BYTES / sizeof(InT); // K elements per ring slot
        constexpr uint32_t W  = ROW_BYTES / sizeof(InT); // M/N elements per 128 bytes
        if(!mnMajor)
        {
            if constexpr(PAIR)
            {
                if(policy != 0)
                    tma_load_2d_pair_hint(dst, tmap, barClusterAddr, int32_t(k0), int32_t(mnOrigin),
                                          policy);
                else
                    tma_load_2d_pair(dst, tmap, barClusterAddr, int32_t(k0), int32_t(mnOrigin));
            }
            else
                tma_load_2d(dst, tmap, bar, int32_t(k0), int32_t(mnOrigin));
            return rows * ROW_BYTES;
        }
        const uint32_t atoms = (rows + W - 1) / W;
        for(uint32_t a = 0; a < atoms; ++a)
        {
            uint8_t* d = dst + a * (BK * ROW_BYTES);
            if constexpr(PAIR)
            {
                if(policy != 0)
                    tma_load_2d_pair_hint(d, tmap, barClusterAddr, int32_t(mnOrigin + a * W),
                                          int32_t(k0), policy);
                else
                    tma_load_2d_pair(d, tmap, barClusterAddr, int32_t(mnOrigin + a * W),
                                     int32_t(k0));
            }
            else
                tma_load_2d(d, tmap, bar, int32_t(mnOrigin + a * W), int32_t(k0));
        }
        return atoms * BK * ROW_BYTES;
    }
    template <typename InT>
    __device__ inline uint32_t operandTileBytes(bool mnMajor, uint32_t rows)
    {
        constexpr uint32_t W  = ROW_BYTES / sizeof(InT); // M/N elements per 128 bytes
        constexpr uint32_t BK = ROW_BYTES / sizeof(InT); // K rows per ring slot
        return mnMajor ? ((rows + W - 1) / W) * BK * ROW_BYTES : rows * ROW_BYTES;
    }
    // Shared-memory descriptor of an operand tile at K step `ks` of its ring slot.
    template <typename InT>
    __device__ inline uint64_t operandDesc(uint32_t tileAddr, bool mnMajor, uint32_t ks)
    {
        constexpr uint32_t BK     = ROW_BYTES / sizeof(InT);
        constexpr uint32_t UMMA_K = 32 / sizeof(InT);
        if(!mnMajor)
            return smem_desc_kmajor_sw128(tileAddr + ks * 32u);
        return smem_desc_mnmajor_sw128(tileAddr + ks * (UMMA_K / 8u) * 1024u, BK * ROW_BYTES);
    }


    template <typename T>
    struct KindOf;
    template <>
    struct KindOf<__half>
    {
        static constexpr MmaKind  kind = MmaKind::F16;
        static constexpr uint32_t fmt = FMT_F16, acc = ACC_F32;
    };
    template <>
    struct KindOf<__nv_bfloat16>
    {
        static constexpr MmaKind  kind = MmaKind::F16;
        static constexpr uint32_t fmt = FMT_BF16, acc = ACC_F32;
    };
    template <>
    struct KindOf<float> // xfloat32_t storage
    {
        static constexpr MmaKind  kind = MmaKind::TF32;
        static constexpr uint32_t fmt = FMT_TF32, acc = ACC_F32;
    };
    template <>
    struct KindOf<int8_t>
    {
        static constexpr MmaKind  kind = MmaKind::I8;
        static constexpr uint32_t fmt = FMT_S8, acc = ACC_S32;
    };
    template <>
    struct KindOf<__nv_fp8_e4m3>
    {
        static constexpr MmaKind  kind = MmaKind::F8F6F4;
        static constexpr uint32_t fmt = FMT_E4M3, acc = ACC_F32;
    };

    template <>
    struct KindOf<__nv_fp8_e5m2>
    {
        static constexpr MmaKind  kind = MmaKind::F8F6F4;
        static constexpr uint32_t fmt = FMT_E5M2, acc = ACC_F32;
    };

    __device__ inline void tileCoord(uint32_t t, uint32_t tilesM, uint32_t tilesN, uint32_t band,
                                     uint32_t& tm, uint32_t& tn)
    {
        const uint32_t perGroup = band * tilesN;
        const uint32_t group    = t / perGroup;
        const uint32_t firstM   = group * band;
        const uint32_t rows     = min(tilesM - firstM, band);
        const uint32_t r        = t % perGroup;
        tm                      = firstM + r % rows;
        tn                      = r / rows;
    }

    // alpha * acc + beta * c in the compute type, unfused like the host reference.
    __device__ inline float scaleAdd(float alpha, float acc, float beta, float c)
    {
        return __fadd_rn(__fmul_rn(alpha, acc), __fmul_rn(beta, c));
    }
    __device__ inline int32_t scaleAdd(int32_t alpha, int32_t acc, int32_t beta, int32_t c)
    {
        return alpha * acc + beta * c;
    }

    template <typename OutT>
    __device__ inline float toCompute(OutT v)
    {
        return float(v);
    }
    __device__ inline int32_t toCompute(int32_t v)
    {
        return v;
    }
    template <typename OutT, typename CompT>
    __device__ inline OutT fromCompute(CompT v)
    {
        return OutT(v); // __half(float), __nv_bfloat16(float): round to nearest even
    }

    // How one pass of the epilogue treats the accumulator it just read.  With chunked K
    // accumulation (fp32 outputs only) D doubles as the fp32 running sum between chunks.
    enum EpilogueMode : uint32_t
    {
        EPI_WHOLE  = 0, // D = alpha * acc + beta * C            (K accumulated in one chain)
        EPI_FIRST  = 1, // D = acc                               (first chunk of several)
        EPI_MIDDLE = 2, // D = D + acc
        EPI_LAST   = 3  // D = alpha * (D + acc) + beta * C
    };

    // 16- and 32-byte global accesses.  The 32-byte forms move one whole L2 sector per
    // thread and instruction, which spares L2 the merging of two half-sector writes.
    template <uint32_t BYTES>
    __device__ inline void ldVec(void* dst, void const* src)
    {
        uint32_t* d = static_cast<uint32_t*>(dst);
        if constexpr(BYTES == 32)
            asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]),
                           "=r"(d[6]), "=r"(d[7])
                         : "l"(src));
        else
            asm volatile("ld.global.v4.b32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                         : "l"(src));
    }
    template <uint32_t BYTES>
    __device__ inline void stVec(void* dst, void const* src)
    {
        uint32_t const* v = static_cast<uint32_t const*>(src);
        if constexpr(BYTES == 32)
            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(v[0]),
                         "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
                         "r"(v[7])
                         : "memory");
        else
            asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(v[0]), "r"(v[1]),
                         "r"(v[2]), "r"(v[3])
                         : "memory");
    }

    // stVec with an L2 cache hint (a policy made by createpolicy).
    template <uint32_t BYTES>
    __device__ inline void stVecHint(void* dst, void const* src, uint64_t policy)
    {
        uint32_t const* v = static_cast<uint32_t const*>(src);
        if constexpr(BYTES == 32)
            asm volatile("st.global.L2::cache_hint.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8}, %9;" ::"l"(
                             dst),
                         "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]),
                         "r"(v[6]), "r"(v[7]), "l"(policy)
                         : "memory");
        else
            asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(dst),
                         "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "l"(policy)
                         : "memory");
    }

    // Stores (and optionally reads C for) 32 consecutive columns of one output row.
    template <typename OutT, typename CompT, uint32_t VBYTES>
    __device__ inline void epilogueRowV(uint32_t const (&raw)[32], GemmParams const& p,
                                        CompT alpha, CompT beta, bool useC, uint32_t row,
                                        uint32_t col0, uint32_t mode, float const* dPre,
                                        OutT const* cPre = nullptr)
    {
        constexpr uint32_t VEC = VBYTES / sizeof(OutT); // elements per access
        constexpr bool     CAN_CHUNK
            = std::is_same<OutT, float>::value && std::is_same<CompT, float>::value;
        OutT const*        cRow = static_cast<OutT const*>(p.c) + size_t(row) * p.ldc;
        OutT*              dRow = static_cast<OutT*>(p.d) + size_t(row) * p.ldd;
        const bool         readC = useC && (mode == EPI_WHOLE || mode == EPI_LAST);
        const bool         readD = CAN_CHUNK && (mode == EPI_MIDDLE || mode == EPI_LAST);
        // a large D that is written once (not a running sum) passes through L2 marked
        // "evict first", so that it does not push out operand tiles other blocks come back to
        const bool     hintD = (p.l2Hints & 4u) != 0u && (mode == EPI_WHOLE || mode == EPI_LAST);
        const uint64_t policyD = hintD ? l2_policy_evict_first() : 0;
#pragma unroll
        for(uint32_t v = 0; v < 32 / VEC; ++v)
        {
            const uint32_t col = col0 + v * VEC;
            if(col >= p.n)
                break;
            alignas(32) OutT out[VEC];
            alignas(32) OutT cin[VEC];
            alignas(32) OutT din[VEC];
            const bool       whole = (col + VEC <= p.n);
            if(readC)
            {
                if(cPre != nullptr) // C already fetched by the caller
                {
#pragma unroll
                    for(uint32_t e = 0; e < VEC; ++e)
                        cin[e] = cPre[v * VEC + e];
                }
                else if(whole)
                    ldVec<VBYTES>(cin, cRow + col);
                else
                    for(uint32_t e = 0; e < VEC; ++e)
                        cin[e] = (col + e < p.n) ? cRow[col + e] : OutT(0);
            }
            if(readD)
            {
                if constexpr(CAN_CHUNK)
                {
                    if(dPre != nullptr) // running sum already fetched by the caller
                    {
#pragma unroll
                        for(uint32_t e = 0; e < VEC; ++e)
                            din[e] = dPre[v * VEC + e];
                    }
                    else if(whole)
                        ldVec<VBYTES>(din, dRow + col);
                    else
                        for(uint32_t e = 0; e < VEC; ++e)
                            din[e] = (col + e < p.n) ? dRow[col + e] : OutT(0);
                }
            }
#pragma unroll
            for(uint32_t e = 0; e < VEC; ++e)
            {
                CompT acc;
                if constexpr(std::is_same<CompT, float>::value)
                    acc = __uint_as_float(raw[v * VEC + e]);
                else
                    acc = int32_t(raw[v * VEC + e]);
                if constexpr(CAN_CHUNK)
                {
                    if(readD)
                        acc = __fadd_rn(float(din[e]), acc);
                }
                CompT r;
                if(mode == EPI_FIRST || mode == EPI_MIDDLE)
                    r = acc;
                else if(readC)
                    r = scaleAdd(alpha, acc, beta, CompT(toCompute(cin[e])));
                else if constexpr(std::is_same<CompT, float>::value)
                    r = CompT(__fmul_rn(float(alpha), float(acc)));
                else
                    r = CompT(alpha * acc);
                out[e] = fromCompute<OutT, CompT>(r);
            }
            if(whole)
            {
                if(hintD)
                    stVecHint<VBYTES>(dRow + col, out, policyD);
                else
                    stVec<VBYTES>(dRow + col, out);
            }
            else
                for(uint32_t e = 0; e < VEC; ++e)
                    if(col + e < p.n)
                        dRow[col + e] = out[e];
        }
    }

    template <typename OutT, typename CompT>
    __device__ inline void epilogueRow(uint32_t const (&raw)[32], GemmParams const& p, CompT alpha,
                                       CompT beta, bool useC, uint32_t row, uint32_t col0,
                                       uint32_t mode = EPI_WHOLE, float const* dPre = nullptr,
                                       OutT const* cPre = nullptr)
    {
        if(p.wide) // C and D rows are 32-byte aligned: whole-sector accesses
            epilogueRowV<OutT, CompT, 32>(raw, p, alpha, beta, useC, row, col0, mode, dPre, cPre);
        else
            epilogueRowV<OutT, CompT, 16>(raw, p, alpha, beta, useC, row, col0, mode, dPre, cPre);
    }

    // 32 consecutive values of row `rowPtr` starting at column col0 (zeros outside n).
    template <typename T>
    __device__ inline void loadGroup(T (&dst)[32], T const* rowPtr, uint32_t col0, uint32_t n,
                                     bool rowValid, bool wide)
    {
        constexpr uint32_t V32 = 32u / sizeof(T), V16 = 16u / sizeof(T);
        if(wide && rowValid && col0 + 32u <= n)
        {
#pragma unroll
            for(uint32_t v = 0; v < 32u / V32; ++v)
                ldVec<32>(&dst[v * V32], rowPtr + col0 + v * V32);
            return;
        }
#pragma unroll
        for(uint32_t v = 0; v < 32u / V16; ++v)
        {
            const uint32_t col = col0 + v * V16;
            if(rowValid && col + V16 <= n)
                ldVec<16>(&dst[v * V16], rowPtr + col);
            else
            {
#pragma unroll
                for(uint32_t e = 0; e < V16; ++e)
                    dst[v * V16 + e] = (rowValid && col + e < n) ? rowPtr[col + e] : T(0);
            }
        }
    }

    // 32 consecutive fp32 values of row `rowPtr` starting at column col0 (zeros outside n).
    __device__ inline void loadRunningSum(float (&dst)[32], float const* rowPtr, uint32_t col0,
                                          uint32_t n, bool rowValid, bool wide)
    {
        if(wide && rowValid && col0 + 32u <= n)
        {
#pragma unroll
            for(uint32_t v = 0; v < 4; ++v)
                ldVec<32>(&dst[v * 8u], rowPtr + col0 + v * 8u);
            return;
        }
#pragma unroll
        for(uint32_t v = 0; v < 8; ++v)
        {
            const uint32_t col = col0 + v * 4u;
            if(rowValid && col + 4u <= n)
                ldVec<16>(&dst[v * 4u], rowPtr + col);
            else
            {
#pragma unroll
                for(uint32_t e = 0; e < 4; ++e)
                    dst[v * 4u + e] = (rowValid && col + e < n) ? rowPtr[col + e] : 0.0f;
            }
        }
    }

    // Waits for one accumulator buffer and writes its 128 x 256 values out (one row per
    // thread).  In the chunked modes that add to the running sum kept in D, the sum for the
    // next two 32-column groups is fetched ahead of use -- the first two even before the
    // accumulator is ready -- so that the L2 round trips overlap instead of adding up.
    template <typename OutT, typename CompT>
    __device__ inline bool drainAccumulator(uint64_t* accFullBar, uint32_t accPh,
                                            AbortState* abort, uint32_t taddrRowBase,
                                            GemmParams const& p, CompT alpha, CompT beta,
                                            bool useC, uint32_t row, uint32_t colBase,
                                            uint32_t mode, uint32_t bnTile)
    {
        constexpr bool CAN_CHUNK
            = std::is_same<OutT, float>::value && std::is_same<CompT, float>::value;
        const uint32_t groups = bnTile / 32u; // 32-column groups in this tile
        if constexpr(CAN_CHUNK)
        {
            if(mode == EPI_MIDDLE || mode == EPI_LAST)
            {
                constexpr uint32_t AHEAD = 2;
                float              dq[AHEAD + 1][32];
                float const*       dRow
                    = static_cast<float const*>(p.d) + size_t(row < p.m ? row : 0u) * p.ldd;
                const bool rowValid = row < p.m;
#pragma unroll
                for(uint32_t c = 0; c < AHEAD; ++c)
                    loadRunningSum(dq[c], dRow, colBase + c * 32u, p.n, rowValid, p.wide != 0u);
                if(!mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL))
                    return false;
                tc_fence_after_sync();
#pragma unroll
                for(uint32_t chunk = 0; chunk < BN / 32; ++chunk)
                {
                    if(chunk >= groups)
                        break;
                    if(chunk + AHEAD < BN / 32)
                        loadRunningSum(dq[(chunk + AHEAD) % (AHEAD + 1)], dRow,
                                       colBase + (chunk + AHEAD) * 32u, p.n, rowValid,
                                       p.wide != 0u);
                    uint32_t raw[32];
                    __syncwarp();
                    tmem_load_32x32b_x32(taddrRowBase + chunk * 32u, raw);
                    tmem_load_wait();
                    const uint32_t col0 = colBase + chunk * 32u;
                    if(rowValid && col0 < p.n)
                        epilogueRow<OutT, CompT>(raw, p, alpha, beta, useC, row, col0, mode,
                                                 dq[chunk % (AHEAD + 1)]);
                }
                tc_fence_before_sync();
                return true;
            }
        }
        if(useC && (mode == EPI_WHOLE || mode == EPI_LAST))
        {
            // beta != 0: the rows of C are fetched two 32-column groups ahead of use, the
            // first two before the accumulator is even ready, so that their latency hides
            // behind the wait and behind the groups in front of them (fetched group by group
            // inside the loop they cost 15 % of a 4096^3 bf16 -> fp32 product).
            constexpr uint32_t AHEAD = sizeof(OutT) >= 4 ? 1u : 2u; // 32 registers per group of fp32
            alignas(32) OutT   cq[AHEAD + 1][32];
            const bool         rowValid = row < p.m;
            OutT const*        cRow
                = static_cast<OutT const*>(p.c) + size_t(rowValid ? row : 0u) * p.ldc;
#pragma unroll
            for(uint32_t c = 0; c < AHEAD; ++c)
                loadGroup(cq[c], cRow, colBase + c * 32u, p.n, rowValid, p.wide != 0u);
            if(!mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL))
                return false;
            tc_fence_after_sync();
#pragma unroll
            for(uint32_t chunk = 0; chunk < BN / 32; ++chunk)
            {
                if(chunk >= groups)
                    break;
                if(chunk + AHEAD < BN / 32)
                    loadGroup(cq[(chunk + AHEAD) % (AHEAD + 1)], cRow,
                              colBase + (chunk + AHEAD) * 32u, p.n, rowValid, p.wide != 0u);
                uint32_t raw[32];
                __syncwarp();
                tmem_load_32x32b_x32(taddrRowBase + chunk * 32u, raw);
                tmem_load_wait();
                const uint32_t col0 = colBase + chunk * 32u;
                if(rowValid && col0 < p.n)
                    epilogueRow<OutT, CompT>(raw, p, alpha, beta, useC, row, col0, mode, nullptr,
                                             cq[chunk % (AHEAD + 1)]);
            }
            tc_fence_before_sync();
            return true;
        }
        if(!mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL))
            return false;
        tc_fence_after_sync();
        // Two register sets: the tensor-memory load of the next 32 columns is in flight while
        // the current ones are converted and stored.  Inside a run of tiles the whole drain
        // hides behind the next tile's MMAs; after a block's last tile it is exposed, and
        // a 1024-row shard of an 8-GPU run has only two tiles per pair.
        uint32_t rawA[32], rawB[32];
        auto     emit = [&](uint32_t const (&raw)[32], uint32_t chunk) {
            const uint32_t col0 = colBase + chunk * 32u;
            if(row < p.m && col0 < p.n)
                epilogueRow<OutT, CompT>(raw, p, alpha, beta, useC, row, col0, mode);
            __syncwarp(); // rows masked off above rejoin before the next warp-wide load
        };
        tmem_load_32x32b_x32(taddrRowBase, rawA); // warp-wide
#pragma unroll 1
        for(uint32_t chunk = 0; chunk < groups; chunk += 2)
        {
            tmem_load_wait();
            if(chunk + 1 < groups)
                tmem_load_32x32b_x32(taddrRowBase + (chunk + 1) * 32u, rawB);
            emit(rawA, chunk);
            if(chunk + 1 < groups)
            {
                tmem_load_wait();
                if(chunk + 2 < groups)
                    tmem_load_32x32b_x32(taddrRowBase + (chunk + 2) * 32u, rawA);
                emit(rawB, chunk + 1);
            }
        }
        tc_fence_before_sync();
        return true;
    }

    // ---- chunked accumulation with the running sum in tensor memory --------------------------
    // The pair kernel's two accumulator buffers start at columns 0 and 256 of the 512 the block
    // owns; a tile of bn <= 160 columns leaves [bn, 256) and [256 + bn, 512) unused, which is
    // enough for a third, thread-managed copy of the tile: the running sum over the K chunks.
    // After every chunk but the last the epilogue threads read the fresh accumulator, add it
    // to the sum in fp32 with round-to-nearest and write the sum back with tcgen05.st -- no
    // global traffic; the last chunk goes out through the ordinary row epilogue with the sum
    // as its addend.  A thread only ever touches its own lane, so program order plus the
    // ld / st waits is all the ordering needed.
    __device__ inline uint32_t sumColumn(uint32_t group, uint32_t bn)
    {
        const uint32_t inFirstGap = (256u - bn) / 32u;
        return group < inFirstGap ? bn + 32u * group : 256u + bn + 32u * (group - inFirstGap);
    }

    __device__ inline bool drainAccumulatorToTmemSum(uint64_t* accFullBar, uint32_t accPh,
                                                     AbortState* abort, uint32_t taddrAcc,
                                                     uint32_t taddrLane, GemmParams const& p,
                                                     float alpha, float beta, bool useC,
                                                     uint32_t row, uint32_t colBase, uint32_t mode,
                                                     uint32_t bnTile)
    {
        const uint32_t groups = bnTile / 32u;
        if(mode == EPI_FIRST || mode == EPI_MIDDLE)
        {
            if(!mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL))
                return false;
            tc_fence_after_sync();
#pragma unroll 1
            for(uint32_t g = 0; g < groups; ++g)
            {
                uint32_t raw[32];
                __syncwarp();
                tmem_load_32x32b_x32(taddrAcc + g * 32u, raw);
                if(mode == EPI_MIDDLE)
                {
                    uint32_t sum[32];
                    tmem_load_32x32b_x32(taddrLane + sumColumn(g, bnTile), sum);
                    tmem_load_wait();
#pragma unroll
                    for(uint32_t e = 0; e < 32; ++e)
                        raw[e] = __float_as_uint(
                            __fadd_rn(__uint_as_float(sum[e]), __uint_as_float(raw[e])));
                }
                else
                    tmem_load_wait();
                tmem_store_32x32b_x32(taddrLane + sumColumn(g, bnTile), raw);
            }
            tmem_store_wait();
            tc_fence_before_sync();
            return true;
        }
        // last chunk: D = alpha * (sum + acc) + beta * C.  The sum is added here (the same
        // operations in the same order as the EPI_LAST form of the row epilogue), so that its
        // registers are free before the row leaves.  C is read group by group, not ahead of
        // use: with prefetch buffers on top of the two tensor-memory register sets every
        // fp32-output instantiation of the kernel spilled (3.4 KB of spill stores), which cost
        // the chunk drains -- seven of eight drains per tile -- more than the prefetch saved
        // in the eighth.
        const bool rowValid = row < p.m;
        if(!mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL))
            return false;
        tc_fence_after_sync();
#pragma unroll 1
        for(uint32_t g = 0; g < groups; ++g)
        {
            uint32_t raw[32], sum[32];
            __syncwarp();
            tmem_load_32x32b_x32(taddrAcc + g * 32u, raw);
            tmem_load_32x32b_x32(taddrLane + sumColumn(g, bnTile), sum);
            tmem_load_wait();
#pragma unroll
            for(uint32_t e = 0; e < 32; ++e)
                raw[e] = __float_as_uint(
                    __fadd_rn(__uint_as_float(sum[e]), __uint_as_float(raw[e])));
            const uint32_t col0 = colBase + g * 32u;
            if(rowValid && col0 < p.n)
                epilogueRow<float, float>(raw, p, alpha, beta, useC, row, col0, EPI_WHOLE);
        }
        tc_fence_before_sync();
        return true;
    }

    // ---- epilogue through shared memory and TMA ------------------------------------------
    // One TMEM lane is one output row, so a thread that stores its row straight to global
    // memory touches 32 different cache lines per warp instruction.  Here the 128 epilogue
    // threads instead lay each 32-column group of the tile out in shared memory (in the
    // swizzled order the TMA expects, which also keeps the 16-byte shared stores free of
    // bank conflicts) and one thread hands the 128 x 32 box to a TMA store; rows and columns
    // beyond m and n are clipped by the TMA.  With chunked K accumulation the first chunk is
    // stored and every later chunk is ADDED by a TMA reduction (fp32 adds in L2, round to
    // nearest), so the running sum is never read back.
    template <uint32_t ROW_B>
    __device__ inline uint32_t stagingOffset(uint32_t row, uint32_t chunk)
    {
        if constexpr(ROW_B == 128) // 128-byte swizzle: chunk index ^ (row % 8)
            return row * 128u + ((chunk ^ (row & 7u)) << 4);
        else // 64-byte rows, 64-byte swizzle: chunk index ^ ((row / 2) % 4)
            return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
    }

    template <typename OutT, typename CompT>
    __device__ inline bool drainAccumulatorTma(uint64_t* accFullBar, uint32_t accPh,
                                               AbortState* abort, uint32_t taddrRowBase,
                                               GemmParams const& p, CUtensorMap const* tmapD,
                                               uint8_t* staging, uint32_t& stagedGroups,
                                               CompT alpha, CompT beta, bool useC,
                                               uint32_t rowInTile, uint32_t tileRow0,
                                               uint32_t colBase, uint32_t mode, bool leader,
                                               uint32_t bnTile)
    {
        constexpr uint32_t ROW_B  = 32 * sizeof(OutT); // bytes of one staged row (128 or 64)
        constexpr uint32_t VEC    = 16 / sizeof(OutT); // elements per 16-byte chunk
        constexpr uint32_t CHUNKS = ROW_B / 16;
        const uint32_t     groups = bnTile / 32u;
        const uint32_t     row    = tileRow0 + rowInTile;
        const bool         adds   = (mode == EPI_MIDDLE || mode == EPI_LAST);
        const bool         readC  = useC && !adds && row < p.m;
        OutT const*        cRow   = static_cast<OutT const*>(p.c) + size_t(row) * p.ldc;

        // all 128 epilogue threads must take the same way out: the barriers below have no
        // time limit of their own
        const bool ready = mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL);
        if(!named_barrier_all(1, EPI_THREADS, ready))
            return false;
        tc_fence_after_sync();
        if(adds && leader)
            tma_store_wait_all<0>(); // the previous chunk's stores have been performed
#pragma unroll 1
        for(uint32_t g = 0; g < groups; ++g, ++stagedGroups)
        {
            uint8_t* buf = staging + (stagedGroups & 1u) * STG_BYTES;
            if(leader)
                tma_store_wait_read<1>(); // the store that last used this buffer has read it
            named_barrier(1, EPI_THREADS);
            uint32_t raw[32];
            tmem_load_32x32b_x32(taddrRowBase + g * 32u, raw);
            tmem_load_wait();
            const uint32_t col0 = colBase + g * 32u;
#pragma unroll
            for(uint32_t ch = 0; ch < CHUNKS; ++ch)
            {
                alignas(16) OutT out[VEC];
                alignas(16) OutT cin[VEC];
                const uint32_t   col = col0 + ch * VEC;
                if(readC)
                {
                    if(col + VEC <= p.n)
                        ldVec<16>(cin, cRow + col);
                    else
                        for(uint32_t e = 0; e < VEC; ++e)
                            cin[e] = (col + e < p.n) ? cRow[col + e] : OutT(0);
                }
#pragma unroll
                for(uint32_t e = 0; e < VEC; ++e)
                {
                    CompT acc;
                    if constexpr(std::is_same<CompT, float>::value)
                        acc = __uint_as_float(raw[ch * VEC + e]);
                    else
                        acc = int32_t(raw[ch * VEC + e]);
                    CompT r;
                    if(readC)
                        r = scaleAdd(alpha, acc, beta, CompT(toCompute(cin[e])));
                    else if constexpr(std::is_same<CompT, float>::value)
                        r = CompT(__fmul_rn(float(alpha), float(acc)));
                    else
                        r = CompT(alpha * acc);
                    out[e] = fromCompute<OutT, CompT>(r);
                }
                *reinterpret_cast<uint4*>(buf + stagingOffset<ROW_B>(rowInTile, ch))
                    = *reinterpret_cast<uint4 const*>(out);
            }
            fence_async_shared();
            named_barrier(1, EPI_THREADS);
            if(leader)
            {
                if(adds)
                    tma_reduce_add_2d(tmapD, buf, int32_t(col0), int32_t(tileRow0));
                else
                    tma_store_2d(tmapD, buf, int32_t(col0), int32_t(tileRow0));
                tma_store_commit();
            }
        }
        tc_fence_before_sync();
        return true;
    }

    // ---- beta != 0: C comes in through shared memory as well -------------------------------
    // A row epilogue reads C with one row per thread and can keep one or two 32-column
    // groups of it in flight (registers), so every group costs a memory round trip: the drain
    // of a 128 x 256 fp32 tile took about as long as the tile's MMAs (4096^3 bf16 -> fp32:
    // 3.5 tiles per pair, beta = -1 cost 15 us of 113; 8192^3: 66 us of 776; one tile alone
    // 9 us).  Here one thread asks the TMA for the 128-row x 32-column box of C two groups
    // ahead of its use, into the staging buffer that the TMA store of the group before has
    // just read; the 128 epilogue threads then combine accumulator and C IN PLACE (each
    // thread reads and overwrites the same 16-byte pieces, in the swizzled order both TMA
    // directions use) and the box leaves by a TMA store.  Rows and columns beyond m and n
    // arrive as zeros and are clipped on the way out.  The first two boxes of a tile are
    // requested before the wait for its accumulator.
    template <typename OutT, typename CompT>
    __device__ inline bool drainAccumulatorTmaC(uint64_t* accFullBar, uint32_t accPh,
                                                AbortState* abort, uint32_t taddrRowBase,
                                                CUtensorMap const* tmapC,
                                                CUtensorMap const* tmapD, uint8_t* staging,
                                                uint64_t* cFull, uint32_t& stagedGroups,
                                                CompT alpha, CompT beta, uint32_t rowInTile,
                                                uint32_t tileRow0, uint32_t colBase, bool leader,
                                                uint32_t bnTile, bool hintCD,
                                                uint32_t taddrLane = 0, bool withSum = false)
    {
        constexpr uint32_t ROW_B     = 32 * sizeof(OutT); // bytes of one staged row (128 or 64)
        constexpr uint32_t VEC       = 16 / sizeof(OutT); // elements per 16-byte piece
        constexpr uint32_t CHUNKS    = ROW_B / 16;
        constexpr uint32_t BOX_BYTES = 128 * ROW_B;
        const uint32_t     groups    = bnTile / 32u;
        uint32_t           requested = 0; // leader: boxes of this tile asked for so far
        // C is read once and D written once: both pass through L2 marked "evict first", so
        // that they do not push out the operand tiles that other blocks come back to
        // (B200WMMA_GEMM_CD_HINT=0 leaves them unmarked, for comparison)
        const uint64_t streamPolicy = (leader && hintCD) ? l2_policy_evict_first() : 0;
        auto requestBox = [&](uint32_t g, uint32_t count) {
            const uint32_t b = count & 1u;
            mbar_expect_tx(&cFull[b], BOX_BYTES);
            if(hintCD)
                tma_load_2d_hint(staging + b * STG_BYTES, tmapC, &cFull[b],
                                 int32_t(colBase + g * 32u), int32_t(tileRow0), streamPolicy);
            else
                tma_load_2d(staging + b * STG_BYTES, tmapC, &cFull[b],
                            int32_t(colBase + g * 32u), int32_t(tileRow0));
            ++requested;
        };
        // leaving early: boxes asked for and not yet consumed get a bounded time to land
        auto settle = [&](uint32_t firstGroup, uint32_t firstCount) {
            if(!leader)
                return;
            for(uint32_t g = firstGroup; g < requested; ++g)
            {
                const uint32_t  count = firstCount + (g - firstGroup);
                const long long start = clock64();
                while(!mbar_try_wait(&cFull[count & 1u], (count >> 1) & 1u)
                      && clock64() - start < 2000000ll)
                {
                }
            }
        };
        if(leader)
        {
            tma_store_wait_read<0>(); // the previous tile's stores have read both buffers
            requestBox(0u, stagedGroups);
            if(groups > 1u)
                requestBox(1u, stagedGroups + 1u);
        }
        // all 128 epilogue threads must take the same way out: the barriers below have no
        // time limit of their own
        const bool ready = mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL);
        if(!named_barrier_all(1, EPI_THREADS, ready))
        {
            settle(0u, stagedGroups);
            return false;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for(uint32_t g = 0; g < groups; ++g, ++stagedGroups)
        {
            uint8_t* buf = staging + (stagedGroups & 1u) * STG_BYTES;
            uint32_t raw[32];
            tmem_load_32x32b_x32(taddrRowBase + g * 32u, raw);
            if constexpr(std::is_same<CompT, float>::value)
            {
                // last chunk of a chunked accumulation: the running sum kept in tensor memory
                // (drainAccumulatorToTmemSum) is added first, as the row epilogue does
                if(withSum)
                {
                    uint32_t sum[32];
                    tmem_load_32x32b_x32(taddrLane + sumColumn(g, bnTile), sum);
                    tmem_load_wait();
#pragma unroll
                    for(uint32_t e = 0; e < 32; ++e)
                        raw[e] = __float_as_uint(
                            __fadd_rn(__uint_as_float(sum[e]), __uint_as_float(raw[e])));
                }
            }
            const bool landed = mbar_wait(&cFull[stagedGroups & 1u], (stagedGroups >> 1) & 1u,
                                          abort, WAIT_STAGE_FULL);
            tmem_load_wait();
#pragma unroll
            for(uint32_t ch = 0; ch < CHUNKS; ++ch)
            {
                uint4* piece
                    = reinterpret_cast<uint4*>(buf + stagingOffset<ROW_B>(rowInTile, ch));
                alignas(16) OutT cin[VEC];
                alignas(16) OutT out[VEC];
                *reinterpret_cast<uint4*>(cin) = *piece;
#pragma unroll
                for(uint32_t e = 0; e < VEC; ++e)
                {
                    CompT acc;
                    if constexpr(std::is_same<CompT, float>::value)
                        acc = __uint_as_float(raw[ch * VEC + e]);
                    else
                        acc = int32_t(raw[ch * VEC + e]);
                    out[e] = fromCompute<OutT, CompT>(
                        scaleAdd(alpha, acc, beta, CompT(toCompute(cin[e]))));
                }
                *piece = *reinterpret_cast<uint4 const*>(out);
            }
            fence_async_shared();
            if(!named_barrier_all(1, EPI_THREADS, landed))
            {
                settle(g + 1u, stagedGroups + 1u);
                return false;
            }
            if(leader)
            {
                if(hintCD)
                    tma_store_2d_hint(tmapD, buf, int32_t(colBase + g * 32u), int32_t(tileRow0),
                                      streamPolicy);
                else
                    tma_store_2d(tmapD, buf, int32_t(colBase + g * 32u), int32_t(tileRow0));
                tma_store_commit();
                if(g + 2u < groups)
                {
                    tma_store_wait_read<0>(); // that store has read the buffer: refill it
                    requestBox(g + 2u, stagedGroups + 2u);
                }
            }
        }
        tc_fence_before_sync();
        return true;
    }

    // ---- C on its way to L2 ----------------------------------------------------------------
    // With beta != 0 an epilogue thread reads its row of C once, from DRAM, and a row
    // epilogue can only keep one or two 32-column groups of it in flight (registers): every
    // group then costs a DRAM round trip.  Behind the next tile's MMAs that does not show, but
    // after a block's last tile it does -- 4096^3 bf16 -> fp32 with beta = -1 took 16 us longer
    // than with beta = 0, and 16-bit outputs 8 us.  So each thread asks for its row of the
    // NEXT tile (and, at the start, of its first) to be brought into L2 a whole tile ahead of
    // use; the loads of the epilogue then take an L2 hit each.
    template <typename OutT>
    __device__ inline void prefetchRowOfC(GemmParams const& p, uint32_t row, uint32_t col0,
                                          uint32_t width)
    {
        if(row >= p.m || col0 >= p.n)
            return;
        const uint32_t cols  = (p.n - col0 < width) ? p.n - col0 : width;
        const uint32_t bytes = cols * uint32_t(sizeof(OutT));
        char const*    base
            = reinterpret_cast<char const*>(static_cast<OutT const*>(p.c) + size_t(row) * p.ldc + col0);
        for(uint32_t off = 0; off < bytes; off += 128u)
            prefetch_l2(base + off);
        prefetch_l2(base + bytes - 1u); // a row that does not start on a line boundary
    }

    // ---- half of a tile that was split along K ---------------------------------------------
    // Two pairs each accumulate half of K for the same tile (TileSchedule::splitTiles).  Each
    // block writes its raw 32-bit accumulator to the workspace, makes it visible and takes a
    // ticket from the tile's counter; whoever draws the second ticket adds the other half
    // (read from the workspace past L1) to its own (still in tensor memory) and does the
    // ordinary row epilogue; the first one is done after its write.  Nobody waits for anybody,
    // so nothing can hang, and a two-term fp32 (or int32) sum does not depend on who came
    // last.  The counter is put back to zero by the second arrival.
    // Workspace: [split tile][part][block of the pair][128 rows][256 columns] of 32-bit values.
    template <typename OutT, typename CompT>
    __device__ inline bool drainSplitPart(uint64_t* accFullBar, uint32_t accPh, AbortState* abort,
                                          uint32_t taddrRowBase, GemmParams const& p,
                                          uint32_t* lastFlag, uint32_t splitIndex, uint32_t part,
                                          uint32_t rank, CompT alpha, CompT beta, bool useC,
                                          uint32_t rowInTile, uint32_t row, uint32_t colBase,
                                          bool leader, uint32_t bnTile)
    {
        constexpr uint32_t PLANE  = 128u * 256u; // values of one block's half-accumulator
        const uint32_t     groups = bnTile / 32u;
        uint32_t* mine  = reinterpret_cast<uint32_t*>(p.splitWs)
                         + size_t((splitIndex * 2u + part) * 2u + rank) * PLANE + rowInTile * 256u;
        uint32_t const* theirs = reinterpret_cast<uint32_t const*>(p.splitWs)
                                 + size_t((splitIndex * 2u + (part ^ 1u)) * 2u + rank) * PLANE
                                 + rowInTile * 256u;
        const bool ready = mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL);
        if(!named_barrier_all(1, EPI_THREADS, ready))
            return false;
        tc_fence_after_sync();
#pragma unroll 1
        for(uint32_t h = 0; h < 2u * groups; ++h) // 16 columns at a time
        {
            uint32_t raw[16];
            tmem_load_32x32b_x16(taddrRowBase + h * 16u, raw);
            tmem_load_wait();
#pragma unroll
            for(uint32_t v = 0; v < 2; ++v)
                stVec<32>(mine + h * 16u + v * 8u, &raw[v * 8u]);
        }
        __threadfence(); // this thread's part is visible device-wide before the ticket is drawn
        named_barrier(1, EPI_THREADS);
        if(leader)
        {
            uint32_t* ctr    = p.splitCtr + splitIndex * 2u + rank;
            const uint32_t t = atomicAdd(ctr, 1u);
            if(t == 1u)
                atomicExch(ctr, 0u); // both halves are in: ready for the next launch
            *lastFlag = t;
        }
        named_barrier(1, EPI_THREADS);
        const bool last = (*reinterpret_cast<volatile uint32_t*>(lastFlag) == 1u);
        named_barrier(1, EPI_THREADS); // everybody has read the flag before it is written again
        if(last)
        {
            __threadfence();
#pragma unroll 1
            for(uint32_t g = 0; g < groups; ++g)
            {
                uint32_t raw[32];
                __syncwarp();
                tmem_load_32x32b_x32(taddrRowBase + g * 32u, raw);
                tmem_load_wait();
#pragma unroll
                for(uint32_t h = 0; h < 4; ++h) // the other half, 8 values at a time
                {
                    uint32_t other[8];
#pragma unroll
                    for(uint32_t v = 0; v < 2; ++v)
                        asm volatile("ld.global.cg.v4.b32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(other[v * 4u]), "=r"(other[v * 4u + 1u]),
                                       "=r"(other[v * 4u + 2u]), "=r"(other[v * 4u + 3u])
                                     : "l"(theirs + g * 32u + h * 8u + v * 4u));
#pragma unroll
                    for(uint32_t e = 0; e < 8; ++e)
                    {
                        uint32_t& r = raw[h * 8u + e];
                        if constexpr(std::is_same<CompT, float>::value)
                            r = __float_as_uint(
                                __fadd_rn(__uint_as_float(r), __uint_as_float(other[e])));
                        else
                            r = uint32_t(int32_t(r) + int32_t(other[e]));
                    }
                }
                const uint32_t col0 = colBase + g * 32u;
                if(row < p.m && col0 < p.n)
                    epilogueRow<OutT, CompT>(raw, p, alpha, beta, useC, row, col0, EPI_WHOLE);
            }
        }
        tc_fence_before_sync();
        return true;
    }

    // ---- a block's LAST tile: out through the idle operand ring ---------------------------
    // Inside a run of tiles the epilogue hides behind the next tile's MMAs; after a block's
    // last tile nothing is left to hide it, and a two-wave launch (the 1024-row shard of an
    // 8-GPU run) pays it once per two tiles: 128 rows x 224 columns took 2.6 us through
    // per-thread row stores, which touch 32 different cache lines per warp instruction.
    // When the accumulator of the last tile is complete every MMA of the pair has finished
    // reading shared memory and no load is in flight, so the ring is free: the epilogue
    // threads lay the whole tile out there -- boxes of 128 rows x 128 bytes in the TMA's
    // 128-byte swizzle, which also keeps the 16-byte shared stores free of bank conflicts --
    // with no block-wide barrier between column groups, and one thread hands the boxes to
    // TMA stores, which write whole 128-byte lines.  2-byte outputs whose tile width is an
    // odd multiple of 32 columns end in one box of 64-byte rows (the narrow map).
    // Rows and columns beyond m and n are clipped by the TMA.
    template <typename OutT, typename CompT>
    __device__ inline bool drainLastTileStaged(uint64_t* accFullBar, uint32_t accPh,
                                               AbortState* abort, uint32_t taddrRowBase,
                                               GemmParams const& p, CUtensorMap const* mapWide,
                                               CUtensorMap const* mapNarrow, uint8_t* stage,
                                               CompT alpha, CompT beta, bool useC,
                                               uint32_t rowInTile, uint32_t tileRow0,
                                               uint32_t colBase, bool leader, uint32_t bnTile)
    {
        // The tile is walked 16 columns at a time (two register sets of 16: the next
        // tensor-memory load is in flight while the current columns are converted and staged).
        constexpr uint32_t HALF_B   = 16 * sizeof(OutT); // bytes of 16 columns: 32 or 64
        constexpr uint32_t PER_BOX  = 128 / HALF_B; // 16-column pieces per 128-byte box row
        constexpr uint32_t VEC      = 16 / sizeof(OutT);
        constexpr uint32_t CHUNKS   = HALF_B / 16; // 16-byte chunks per piece: 2 or 4
        constexpr uint32_t BOX_COLS = 128 / sizeof(OutT);
        constexpr uint32_t BOX_B    = 128 * 128;
        const uint32_t     pieces   = bnTile / 16u;
        const uint32_t     wide     = pieces / PER_BOX; // full 128-byte boxes
        const uint32_t     row      = tileRow0 + rowInTile;
        const bool         readC    = useC && row < p.m;
        OutT const*        cRow     = static_cast<OutT const*>(p.c) + size_t(row) * p.ldc;

        const bool ready = mbar_wait(accFullBar, accPh, abort, WAIT_ACC_FULL);
        if(!named_barrier_all(1, EPI_THREADS, ready))
            return false;
        tc_fence_after_sync();
        uint32_t rawA[16], rawB[16];
        auto     emit = [&](uint32_t const (&raw)[16], uint32_t piece) {
            const uint32_t col0 = colBase + piece * 16u;
            const uint32_t box  = piece / PER_BOX;
            uint8_t*       base = stage + box * BOX_B;
#pragma unroll
            for(uint32_t ch = 0; ch < CHUNKS; ++ch)
            {
                alignas(16) OutT out[VEC];
                alignas(16) OutT cin[VEC];
                const uint32_t   col = col0 + ch * VEC;
                if(readC)
                {
                    if(col + VEC <= p.n)
                        ldVec<16>(cin, cRow + col);
                    else
                        for(uint32_t e = 0; e < VEC; ++e)
                            cin[e] = (col + e < p.n) ? cRow[col + e] : OutT(0);
                }
#pragma unroll
                for(uint32_t e = 0; e < VEC; ++e)
                {
                    CompT acc;
                    if constexpr(std::is_same<CompT, float>::value)
                        acc = __uint_as_float(raw[ch * VEC + e]);
                    else
                        acc = int32_t(raw[ch * VEC + e]);
                    CompT r;
                    if(readC)
                        r = scaleAdd(alpha, acc, beta, CompT(toCompute(cin[e])));
                    else if constexpr(std::is_same<CompT, float>::value)
                        r = CompT(__fmul_rn(float(alpha), float(acc)));
                    else
                        r = CompT(alpha * acc);
                    out[e] = fromCompute<OutT, CompT>(r);
                }
                uint32_t off;
                if(box < wide) // 128-byte rows
                    off = stagingOffset<128>(rowInTile, (piece % PER_BOX) * CHUNKS + ch);
                else // the odd last 32 columns of a 2-byte output: 64-byte rows
                    off = stagingOffset<64>(rowInTile, (piece % PER_BOX) * CHUNKS + ch);
                *reinterpret_cast<uint4*>(base + off) = *reinterpret_cast<uint4 const*>(out);
            }
        };
        tmem_load_32x32b_x16(taddrRowBase, rawA); // warp-wide
#pragma unroll 1
        for(uint32_t piece = 0; piece < pieces; piece += 2) // pieces is even: bnTile % 32 == 0
        {
            tmem_load_wait();
            tmem_load_32x32b_x16(taddrRowBase + (piece + 1) * 16u, rawB);
            emit(rawA, piece);
            tmem_load_wait();
            if(piece + 2 < pieces)
                tmem_load_32x32b_x16(taddrRowBase + (piece + 2) * 16u, rawA);
            emit(rawB, piece + 1);
        }
        fence_async_shared();
        named_barrier(1, EPI_THREADS);
        if(leader && tileRow0 < p.m)
        {
            const bool     hintD   = (p.l2Hints & 4u) != 0u;
            const uint64_t policyD = hintD ? l2_policy_evict_first() : 0;
            auto           store   = [&](CUtensorMap const* map, uint8_t* src, uint32_t col) {
                if(hintD)
                    tma_store_2d_hint(map, src, int32_t(col), int32_t(tileRow0), policyD);
                else
                    tma_store_2d(map, src, int32_t(col), int32_t(tileRow0));
            };
            for(uint32_t b = 0; b < wide; ++b)
                if(colBase + b * BOX_COLS < p.n)
                    store(mapWide, stage + b * BOX_B, colBase + b * BOX_COLS);
            if(pieces % PER_BOX != 0u && colBase + wide * BOX_COLS < p.n)
                store(mapNarrow, stage + wide * BOX_B, colBase + wide * BOX_COLS);
            tma_store_commit();
        }
        tc_fence_before_sync();
        return true;
    }

    template <typename InT, typename OutT, typename CompT>
    __global__ void __launch_bounds__(NUM_THREADS, 1)
        gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmapA,
                            const __grid_constant__ CUtensorMap tmapB,
                            const __grid_constant__ CUtensorMap tmapD,
                            const GemmParams                    p)
    {
        constexpr uint32_t BK     = ROW_BYTES / sizeof(InT); // K elements per ring slot
        constexpr uint32_t UMMA_K = 32 / sizeof(InT); // K elements per tcgen05.mma
        const uint32_t IDESC = make_instr_desc(KindOf<InT>::acc, KindOf<InT>::fmt,
                                               KindOf<InT>::fmt, BM, BN, p.aMN, p.bMN);

        extern __shared__ uint8_t smemRaw[];
        const uint32_t            rawAddr = smem_addr(smemRaw);
        uint8_t*       tiles = smemRaw + ((1024u - (rawAddr & 1023u)) & 1023u); // 1024-aligned
        uint8_t*       staging = tiles + STAGES * STAGE_BYTES; // 1024-aligned: tiles are
        SharedControl* ctl
            = reinterpret_cast<SharedControl*>(tiles + STAGES * STAGE_BYTES + 2 * STG_BYTES);

        const uint32_t warp = threadIdx.x / 32;
        const uint32_t lane = threadIdx.x % 32;

        const uint32_t tilesM   = (p.m + BM - 1) / BM;
        const uint32_t tilesN   = (p.n + BN - 1) / BN;
        const uint32_t numTiles = tilesM * tilesN;
        const uint32_t numKB    = (p.k + BK - 1) / BK;
        const uint32_t chunkKB  = p.chunkKB != 0u ? p.chunkKB : numKB; // K blocks per chain
        const uint32_t numChunks = (numKB + chunkKB - 1) / chunkKB;

        if(threadIdx.x == 0)
        {
            for(uint32_t s = 0; s < STAGES; ++s)
            {
                mbar_init(&ctl->full[s], 1);
                mbar_init(&ctl->empty[s], 1);
            }
            for(uint32_t b = 0; b < ACC_BUFS; ++b)
            {
                mbar_init(&ctl->accFull[b], 1);
                mbar_init(&ctl->accEmpty[b], EPI_THREADS);
            }
            ctl->abort.flag = 0;
            ctl->abort.code = 0;
            mbar_init_fence();
            tma_prefetch_descriptor(&tmapA);
            tma_prefetch_descriptor(&tmapB);
            tma_prefetch_descriptor(&tmapD);
        }
        if(warp == 1)
        {
            tmem_alloc(&ctl->tmemBase, TMEM_COLS);
            tmem_relinquish_alloc_permit();
        }
        tc_fence_before_sync();
        __syncthreads();
        tc_fence_after_sync();
        const uint32_t tmemBase = ctl->tmemBase;
        // programmatic dependent launch, as in the pair kernel below: the set-up above may
        // overlap the previous kernel of the stream, global memory is touched only from here
        grid_dependency_wait();
        grid_launch_dependents();

        if(warp == 0)
        {
            // ---------------- TMA producer ----------------
            if(elect_one())
            {
                uint32_t it = 0;
                bool     ok = true;
                for(uint32_t t = blockIdx.x; ok && t < numTiles; t += gridDim.x)
                {
                    uint32_t tm, tn;
                    tileCoord(t, tilesM, tilesN, p.band, tm, tn);
                    for(uint32_t kb = 0; kb < numKB; ++kb, ++it)
                    {
                        const uint32_t s  = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1u;
                        if(!mbar_wait(&ctl->empty[s], ph ^ 1u, &ctl->abort, WAIT_STAGE_EMPTY))
                        {
                            ok = false;
                            break;
                        }
                        uint8_t* slot = tiles + s * STAGE_BYTES;
                        mbar_expect_tx(&ctl->full[s], operandTileBytes<InT>(p.aMN != 0u, BM)
                                                          + operandTileBytes<InT>(p.bMN != 0u, BN));
                        loadOperandTile<InT, false>(slot, &tmapA, &ctl->full[s], 0u, p.aMN != 0u,
                                                    tm * BM, BM, kb * BK);
                        loadOperandTile<InT, false>(slot + A_BYTES, &tmapB, &ctl->full[s], 0u,
                                                    p.bMN != 0u, tn * BN, BN, kb * BK);
                    }
                }
                if(!ok)
                {
                    // Leaving early: give copies already issued a bounded time to land
                    // before the block's shared memory is released.
                    const uint32_t pending = it < STAGES ? it : STAGES;
                    for(uint32_t j = 0; j < pending; ++j)
                    {
                        const uint32_t prev = it - 1 - j;
                        const uint32_t s    = prev % STAGES;
                        const uint32_t ph   = (prev / STAGES) & 1u;
                        const long long start = clock64();
                        while(!mbar_try_wait(&ctl->full[s], ph) && clock64() - start < 2000000ll)
                        {
                        }
                    }
                }
            }
        }
        else if(warp == 1)
        {
            // ---------------- MMA issuer ----------------
            if(elect_one())
            {
                uint32_t it = 0, accIter = 0;
                bool     ok = true;
                for(uint32_t t = blockIdx.x; ok && t < numTiles; t += gridDim.x)
                {
                    // one accumulation chain per chunk of K, alternating TMEM buffers
                    for(uint32_t kb0 = 0; ok && kb0 < numKB; kb0 += chunkKB, ++accIter)
                    {
                        const uint32_t buf   = accIter & 1u;
                        const uint32_t accPh = (accIter >> 1) & 1u;
                        if(!mbar_wait(&ctl->accEmpty[buf], accPh ^ 1u, &ctl->abort,
                                      WAIT_ACC_EMPTY))
                        {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t dTmem = tmemBase + buf * BN;
                        const uint32_t kb1   = min(numKB, kb0 + chunkKB);
                        for(uint32_t kb = kb0; kb < kb1; ++kb, ++it)
                        {
                            const uint32_t s  = it % STAGES;
                            const uint32_t ph = (it / STAGES) & 1u;
                            if(!mbar_wait(&ctl->full[s], ph, &ctl->abort, WAIT_STAGE_FULL))
                            {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t aAddr = smem_addr(tiles + s * STAGE_BYTES);
                            const uint32_t bAddr = aAddr + A_BYTES;
#pragma unroll
                            for(uint32_t ks = 0; ks < BK / UMMA_K; ++ks)
                            {
                                const uint64_t da = operandDesc<InT>(aAddr, p.aMN != 0u, ks);
                                const uint64_t db = operandDesc<InT>(bAddr, p.bMN != 0u, ks);
                                mma_ss<KindOf<InT>::kind>(dTmem, da, db, IDESC,
                                                          (kb > kb0 || ks > 0u) ? 1u : 0u);
                            }
                            mma_commit(&ctl->empty[s]); // slot reusable once these MMAs are done
                        }
                        if(ok)
                            mma_commit(&ctl->accFull[buf]); // this chain is complete
                    }
                }
            }
        }
        else
        {
            // ---------------- epilogue ----------------
            const uint32_t quad  = warp % 4; // TMEM lanes [32*quad, 32*quad+32)
            const CompT    alpha = CompT(p.alpha);
            const CompT    beta  = CompT(p.beta);
            const bool     useC  = (p.beta != 0.0) && (p.c != nullptr);
            uint32_t       accIter = 0, stagedGroups = 0;
            bool           ok      = true;
            for(uint32_t t = blockIdx.x; ok && t < numTiles; t += gridDim.x)
            {
                uint32_t tm, tn;
                tileCoord(t, tilesM, tilesN, p.band, tm, tn);
                const uint32_t row = tm * BM + quad * 32 + lane;
                for(uint32_t ch = 0; ch < numChunks; ++ch, ++accIter)
                {
                    const uint32_t buf   = accIter & 1u;
                    const uint32_t accPh = (accIter >> 1) & 1u;
                    const uint32_t mode = numChunks == 1u       ? EPI_WHOLE
                                          : ch == 0u            ? EPI_FIRST
                                          : ch + 1u < numChunks ? EPI_MIDDLE
                                                                : EPI_LAST;
                    const uint32_t taddr = tmemBase + ((quad * 32u) << 16) + buf * BN;
                    const bool     drained
                        = p.tmaStore
                              ? drainAccumulatorTma<OutT, CompT>(
                                  &ctl->accFull[buf], accPh, &ctl->abort, taddr, p, &tmapD, staging,
                                  stagedGroups, alpha, beta, useC, quad * 32u + lane, tm * BM,
                                  tn * BN, mode, threadIdx.x == 64u, BN)
                              : drainAccumulator<OutT, CompT>(&ctl->accFull[buf], accPh,
                                                              &ctl->abort, taddr, p, alpha, beta,
                                                              useC, row, tn * BN, mode, BN);
                    if(!drained)
                    {
                        ok = false;
                        break;
                    }
                    mbar_arrive(&ctl->accEmpty[buf]);
                }
            }
            if(threadIdx.x == 64u)
                tma_store_wait_all<0>(); // every TMA store of this block has been performed
        }

        // ---------------- teardown ----------------
        tc_fence_before_sync();
        __syncthreads();
        if(warp == 1)
        {
            __syncwarp();
            tc_fence_after_sync();
            tmem_dealloc(tmemBase, TMEM_COLS);
        }
        if(threadIdx.x == 0 && ctl->abort.flag != 0u && p.status != nullptr)
        {
            atomicExch(&p.status[1], ctl->abort.code);
            atomicExch(&p.status[0], 1u);
        }
    }

    // =====================================================================================
    // CTA-pair variant: a cluster of two blocks (the two SMs of a TPC) computes a
    // 256 x 256 tile with tcgen05.mma.cta_group::2.  Block r of the pair loads rows
    // [128 r, 128 r + 128) of the A tile and of the B tile into its OWN shared memory
    // (plain TMA loads; nothing is multicast), the even block issues the M = 256 MMAs
    // for both, and each block's tensor core leaves its 128 accumulator rows in its own
    // TMEM.  Per block and K step that is 32 KiB of operands instead of 48 KiB, which
    // buys a 6-slot ring and a third less L2 -> shared-memory traffic per flop.
    //
    // Barriers: the leader's full[s] collects the bytes of BOTH blocks (the peer's TMA
    // signals it remotely); empty[s] and accFull[b] are completed in both blocks by one
    // multicast tcgen05.commit; the leader's accEmpty[b] counts the epilogue threads of
    // both blocks.
    // =====================================================================================
    constexpr uint32_t P_TILE_M      = 256; // rows per pair
    constexpr uint32_t P_STAGES      = 6;
    constexpr uint32_t P_A_BYTES     = 128 * ROW_BYTES; // 16 KiB: this block's rows of A
    constexpr uint32_t P_B_BYTES     = 128 * ROW_BYTES; // 16 KiB: this block's half of B
    constexpr uint32_t P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;

    struct PairControl
    {
        uint64_t   full[P_STAGES];
        uint64_t   empty[P_STAGES];
        uint64_t   accFull[ACC_BUFS];
        uint64_t   accEmpty[ACC_BUFS];
        uint64_t   cFull[2]; // epilogue: a box of C has landed in staging buffer 0 / 1
        uint32_t   tmemBase;
        uint32_t   splitLast; // epilogue: this block arrived last at a split tile
        AbortState abort;
    };
    constexpr uint32_t P_SMEM_BYTES
        = P_STAGES * P_STAGE_BYTES + 2 * STG_BYTES + 1024 + sizeof(PairControl) + 64;

    template <typename InT, typename OutT, typename CompT>
    __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
        gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmapA,
                                 const __grid_constant__ CUtensorMap tmapB,
                                 const __grid_constant__ CUtensorMap tmapBTail,
                                 const __grid_constant__ CUtensorMap tmapD,
                                 const __grid_constant__ CUtensorMap tmapDWide,
                                 const __grid_constant__ CUtensorMap tmapC,
                                 const GemmParams                    p)
    {
        constexpr uint32_t BK     = ROW_BYTES / sizeof(InT);
        constexpr uint32_t UMMA_K = 32 / sizeof(InT);
        // The tile width is chosen per launch (a multiple of 32 up to 256); it is the N of the
        // MMA instruction.  A launch may use a second, narrower width for the right-hand
        // columns of the output (TileSchedule); tmapBTail is B's tensor map with that box.
        const uint32_t bn    = p.bn;
        const uint32_t IDESC = make_instr_desc(KindOf<InT>::acc, KindOf<InT>::fmt,
                                               KindOf<InT>::fmt, P_TILE_M, bn, p.aMN, p.bMN);
        const uint32_t IDESC_TAIL
            = make_instr_desc(KindOf<InT>::acc, KindOf<InT>::fmt, KindOf<InT>::fmt, P_TILE_M,
                              p.bnTail != 0u ? p.bnTail : bn, p.aMN, p.bMN);
        // bytes per K block and block: its 128 rows of A and its half of the B tile
        const uint32_t aSlotBytes = operandTileBytes<InT>(p.aMN != 0u, 128u);

        extern __shared__ uint8_t smemRaw[];
        const uint32_t            rawAddr = smem_addr(smemRaw);
        uint8_t*     tiles = smemRaw + ((1024u - (rawAddr & 1023u)) & 1023u);
        uint8_t*     staging = tiles + P_STAGES * P_STAGE_BYTES;
        PairControl* ctl
            = reinterpret_cast<PairControl*>(tiles + P_STAGES * P_STAGE_BYTES + 2 * STG_BYTES);

        const uint32_t warp   = threadIdx.x / 32;
        const uint32_t lane   = threadIdx.x % 32;
        const uint32_t rank   = cluster_cta_rank(); // 0 = leader of the pair
        const uint32_t pairId = blockIdx.x / 2;
        const uint32_t nPairs = gridDim.x / 2;

        const uint32_t tilesM   = (p.m + P_TILE_M - 1) / P_TILE_M;
        const uint32_t numKB    = (p.k + BK - 1) / BK;
        const uint32_t chunkKB  = p.chunkKB != 0u ? p.chunkKB : numKB; // K blocks per chain
        const uint32_t numChunks = (numKB + chunkKB - 1) / chunkKB;
        const TileSchedule sched{tilesM, p.wideCols, p.tailCols, bn,       p.bnTail,
                                 p.band, nPairs,     p.snake,    p.mirror, p.splitTiles};

        if(threadIdx.x == 0)
        {
            for(uint32_t s = 0; s < P_STAGES; ++s)
            {
                mbar_init(&ctl->full[s], 1);
                mbar_init(&ctl->empty[s], 1);
            }
            for(uint32_t b = 0; b < ACC_BUFS; ++b)
            {
                mbar_init(&ctl->accFull[b], 1);
                mbar_init(&ctl->accEmpty[b], 2 * EPI_THREADS);
            }
            mbar_init(&ctl->cFull[0], 1);
            mbar_init(&ctl->cFull[1], 1);
            ctl->abort.flag = 0;
            ctl->abort.code = 0;
            mbar_init_fence();
            tma_prefetch_descriptor(&tmapA);
            tma_prefetch_descriptor(&tmapB);
            tma_prefetch_descriptor(&tmapBTail);
            tma_prefetch_descriptor(&tmapC);
            tma_prefetch_descriptor(&tmapD);
            tma_prefetch_descriptor(&tmapDWide);
        }
        // First half of the pair's start-up barrier: this block's mbarriers exist (thread 0
        // released them above, before its own arrival).  The wait comes after the rest of the
        // set-up, which so overlaps the barrier's latency (measured: a back-to-back
        // arrive + wait at this point cost 1.8 us of every launch).
        __syncwarp();
        cluster_arrive_relaxed();
        if(threadIdx.x == 64u && p.prefetch != 0u)
        {
            // The operands of this block's first ring slots are requested into L2 while the
            // set-up below (and, under programmatic dependent launch, the previous kernel's
            // tail) is still running.  An L2 prefetch reads nothing into the SM, and L2 is
            // where a later write by the previous kernel lands too, so this is safe before
            // griddepcontrol.wait even when A or B is that kernel's output.
            uint32_t tm, col0, width, part, ways, splitIndex;
            if(sched.getItem(pairId, 0, tm, col0, width, part, ways, splitIndex))
            {
                const void*    mapB = width == bn ? static_cast<void const*>(&tmapB)
                                                  : static_cast<void const*>(&tmapBTail);
                const int32_t  rowA = int32_t(tm * P_TILE_M + rank * 128u);
                const int32_t  rowB = int32_t(col0 + rank * (width / 2u));
                const uint32_t kb0  = part * numKB / ways;
                const uint32_t nkb  = kb0 + (p.prefetch < numKB ? p.prefetch : numKB);
                for(uint32_t kb = kb0; kb < nkb && kb < numKB; ++kb)
                {
                    if(p.aMN == 0u)
                        tma_prefetch_l2_2d(&tmapA, int32_t(kb * BK), rowA);
                    if(p.bMN == 0u)
                        tma_prefetch_l2_2d(mapB, int32_t(kb * BK), rowB);
                }
            }
        }
        if(warp == 1)
        {
            tmem_alloc_pair(&ctl->tmemBase, TMEM_COLS);
            tmem_relinquish_alloc_permit_pair();
        }
        tc_fence_before_sync();
        __syncthreads();
        cluster_wait(); // both blocks' barriers exist before anything signals them remotely
        tc_fence_after_sync();
        const uint32_t tmemBase = ctl->tmemBase;
        // Programmatic dependent launch: everything above (barriers, tensor-memory
        // allocation, descriptor prefetch) touches no global data and may run while the
        // previous kernel of the stream drains; from here on its results are needed (A, B or C
        // may be its output, D its input).  The next kernel of the stream may be scheduled as
        // soon as every block of this one has got this far: it waits at the same place.
        grid_dependency_wait();
        grid_launch_dependents();

        if(warp == 0)
        {
            // ---------------- TMA producer (both blocks) ----------------
            if(elect_one())
            {
                uint32_t it = 0;
                bool     ok = true;
                // A column tile of B is used by the pairs of one wave and then not before the
                // next raster band (or the next launch): a B too large to stay in L2 anyway is
                // fetched "evict first", so that its stream does not push the rows of A, which
                // every wave of a band comes back to, and the freshly written D out of L2.
                // Measured (20 launches back to back after an idle gap, same box, alternating
                // runs): 8192^3 751.7 -> 739.2 us, 4096-row shard 374.6 -> 366.5, 2048 rows
                // 186.9 -> 182.6, 1024 rows 97.1 -> 95.2; 4096^3 unchanged.  Marking A
                // "evict last" as well changes nothing measurable (bit 0).
                const uint64_t policyA = (p.l2Hints & 1u) ? l2_policy_evict_last() : 0;
                const uint64_t policyB = (p.l2Hints & 2u) ? l2_policy_evict_first() : 0;
                for(uint32_t i = 0; ok; ++i)
                {
                    uint32_t tm, col0, width, part, ways, splitIndex;
                    if(!sched.getItem(pairId, i, tm, col0, width, part, ways, splitIndex))
                        break;
                    const int32_t  rowA = int32_t(tm * P_TILE_M + rank * 128u);
                    const int32_t  rowB = int32_t(col0 + rank * (width / 2u));
                    const void*    mapB = width == bn ? static_cast<void const*>(&tmapB)
                                                      : static_cast<void const*>(&tmapBTail);
                    const uint32_t pairSlotBytes
                        = aSlotBytes + operandTileBytes<InT>(p.bMN != 0u, width / 2u);
                    // this item's k-blocks: all of them, or its half of a split tile
                    const uint32_t kbBegin = part * numKB / ways, kbEnd = (part + 1u) * numKB / ways;
                    for(uint32_t kb = kbBegin; kb < kbEnd; ++kb, ++it)
                    {
                        const uint32_t s  = it % P_STAGES;
                        const uint32_t ph = (it / P_STAGES) & 1u;
                        if(!mbar_wait(&ctl->empty[s], ph ^ 1u, &ctl->abort, WAIT_STAGE_EMPTY))
                        {
                            ok = false;
                            break;
                        }
                        uint8_t* slot = tiles + s * P_STAGE_BYTES;
                        if(rank == 0)
                            mbar_expect_tx(&ctl->full[s], 2u * pairSlotBytes); // both blocks
                        const uint32_t leaderFull = map_to_cta(smem_addr(&ctl->full[s]), 0);
                        loadOperandTile<InT, true>(slot, &tmapA, nullptr, leaderFull, p.aMN != 0u,
                                                   uint32_t(rowA), 128u, kb * BK, policyA);
                        loadOperandTile<InT, true>(slot + P_A_BYTES, mapB, nullptr, leaderFull,
                                                   p.bMN != 0u, uint32_t(rowB), width / 2u,
                                                   kb * BK, policyB);
                    }
                }
            }
        }
        else if(warp == 1)
        {
            // ---------------- MMA issuer (leader block only) ----------------
            if(rank == 0 && elect_one())
            {
                uint32_t it = 0, accIter = 0;
                bool     ok = true;
                for(uint32_t i = 0; ok; ++i)
                {
                    uint32_t tm, col0, width, part, ways, splitIndex;
                    if(!sched.getItem(pairId, i, tm, col0, width, part, ways, splitIndex))
                        break;
                    const uint32_t idesc   = width == bn ? IDESC : IDESC_TAIL;
                    const uint32_t kbBegin = part * numKB / ways, kbEnd = (part + 1u) * numKB / ways;
                    for(uint32_t kb0 = kbBegin; ok && kb0 < kbEnd; kb0 += chunkKB, ++accIter)
                    {
                        const uint32_t buf   = accIter & 1u;
                        const uint32_t accPh = (accIter >> 1) & 1u;
                        if(!mbar_wait(&ctl->accEmpty[buf], accPh ^ 1u, &ctl->abort,
                                      WAIT_ACC_EMPTY))
                        {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t dTmem = tmemBase + buf * BN;
                        const uint32_t kb1   = min(kbEnd, kb0 + chunkKB);
                        for(uint32_t kb = kb0; kb < kb1; ++kb, ++it)
                        {
                            const uint32_t s  = it % P_STAGES;
                            const uint32_t ph = (it / P_STAGES) & 1u;
                            if(!mbar_wait(&ctl->full[s], ph, &ctl->abort, WAIT_STAGE_FULL))
                            {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t aAddr = smem_addr(tiles + s * P_STAGE_BYTES);
                            const uint32_t bAddr = aAddr + P_A_BYTES;
#pragma unroll
                            for(uint32_t ks = 0; ks < BK / UMMA_K; ++ks)
                            {
                                const uint64_t da = operandDesc<InT>(aAddr, p.aMN != 0u, ks);
                                const uint64_t db = operandDesc<InT>(bAddr, p.bMN != 0u, ks);
                                mma_ss_pair<KindOf<InT>::kind>(dTmem, da, db, idesc,
                                                               (kb > kb0 || ks > 0u) ? 1u : 0u);
                            }
                            mma_commit_pair(&ctl->empty[s], 0x3); // frees the slot in both blocks
                        }
                        if(ok)
                            mma_commit_pair(&ctl->accFull[buf], 0x3);
                    }
                }
            }
        }
        else
        {
            // ---------------- epilogue (both blocks, own 128 rows) ----------------
            const uint32_t quad  = warp % 4;
            const CompT    alpha = CompT(p.alpha);
            const CompT    beta  = CompT(p.beta);
            const bool     useC  = (p.beta != 0.0) && (p.c != nullptr);
            uint32_t       accIter = 0, stagedGroups = 0;
            bool           ok      = true;
            for(uint32_t i = 0; ok; ++i)
            {
                uint32_t tm, col0, width, part, ways, splitIndex;
                if(!sched.getItem(pairId, i, tm, col0, width, part, ways, splitIndex))
                    break;
                const uint32_t row = tm * P_TILE_M + rank * 128u + quad * 32u + lane;
                uint32_t       tmNext, colNext, widthNext, partNext, waysNext, splitNext;
                const bool     hasNext = sched.getItem(pairId, i + 1u, tmNext, colNext, widthNext,
                                                       partNext, waysNext, splitNext);
                if(useC && p.cViaTma == 0u)
                {
                    if(i == 0u)
                        prefetchRowOfC<OutT>(p, row, col0, width);
                    if(hasNext)
                        prefetchRowOfC<OutT>(
                            p, tmNext * P_TILE_M + rank * 128u + quad * 32u + lane, colNext,
                            widthNext);
                }
                // (with beta != 0 the last tile keeps the row epilogue, whose loads of C run
                // ahead of their use; the staged form reads C where it needs it)
                const bool stagedTail = p.stagedTail != 0u && numChunks == 1u && ways == 1u
                                        && !useC && !hasNext;
                for(uint32_t ch = 0; ch < numChunks; ++ch, ++accIter)
                {
                    const uint32_t buf   = accIter & 1u;
                    const uint32_t accPh = (accIter >> 1) & 1u;
                    const uint32_t mode = numChunks == 1u       ? EPI_WHOLE
                                          : ch == 0u            ? EPI_FIRST
                                          : ch + 1u < numChunks ? EPI_MIDDLE
                                                                : EPI_LAST;
                    const uint32_t taddrLane = tmemBase + ((quad * 32u) << 16);
                    const uint32_t taddr     = taddrLane + buf * BN;
                    bool           drained;
                    if(ways > 1u)
                    {
                        // half of a split tile: see drainSplitPart
                        drained = drainSplitPart<OutT, CompT>(
                            &ctl->accFull[buf], accPh, &ctl->abort, taddr, p, &ctl->splitLast,
                            splitIndex, part, rank, alpha, beta, useC, quad * 32u + lane, row, col0,
                            threadIdx.x == 64u, width);
                    }
                    else if(p.cViaTma != 0u && useC && numChunks == 1u)
                    {
                        drained = drainAccumulatorTmaC<OutT, CompT>(
                            &ctl->accFull[buf], accPh, &ctl->abort, taddr, &tmapC, &tmapD, staging,
                            ctl->cFull, stagedGroups, alpha, beta, quad * 32u + lane,
                            tm * P_TILE_M + rank * 128u, col0, threadIdx.x == 64u, width,
                            (p.cViaTma & 2u) != 0u);
                    }
                    else if(stagedTail)
                    {
                        // this block's last tile: the ring is idle, see drainLastTileStaged
                        drained = drainLastTileStaged<OutT, CompT>(
                            &ctl->accFull[buf], accPh, &ctl->abort, taddr, p, &tmapDWide, &tmapD,
                            tiles, alpha, beta, useC, quad * 32u + lane,
                            tm * P_TILE_M + rank * 128u, col0, threadIdx.x == 64u, width);
                    }
                    else if constexpr(std::is_same<OutT, float>::value
                                      && std::is_same<CompT, float>::value)
                    {
                        if(p.sumInTmem && numChunks > 1u && mode == EPI_LAST && useC
                           && p.cViaTma != 0u)
                            drained = drainAccumulatorTmaC<OutT, CompT>(
                                &ctl->accFull[buf], accPh, &ctl->abort, taddr, &tmapC, &tmapD,
                                staging, ctl->cFull, stagedGroups, alpha, beta, quad * 32u + lane,
                                tm * P_TILE_M + rank * 128u, col0, threadIdx.x == 64u, width,
                                (p.cViaTma & 2u) != 0u, taddrLane, true);
                        else if(p.sumInTmem && numChunks > 1u)
                            drained = drainAccumulatorToTmemSum(&ctl->accFull[buf], accPh,
                                                                &ctl->abort, taddr, taddrLane, p,
                                                                alpha, beta, useC, row, col0, mode,
                                                                width);
                        else
                            drained = p.tmaStore
                                          ? drainAccumulatorTma<OutT, CompT>(
                                              &ctl->accFull[buf], accPh, &ctl->abort, taddr, p,
                                              &tmapD, staging, stagedGroups, alpha, beta, useC,
                                              quad * 32u + lane, tm * P_TILE_M + rank * 128u, col0,
                                              mode, threadIdx.x == 64u, width)
                                          : drainAccumulator<OutT, CompT>(
                                              &ctl->accFull[buf], accPh, &ctl->abort, taddr, p,
                                              alpha, beta, useC, row, col0, mode, width);
                    }
                    else
                        drained = p.tmaStore
                                      ? drainAccumulatorTma<OutT, CompT>(
                                          &ctl->accFull[buf], accPh, &ctl->abort, taddr, p, &tmapD,
                                          staging, stagedGroups, alpha, beta, useC,
                                          quad * 32u + lane, tm * P_TILE_M + rank * 128u, col0,
                                          mode, threadIdx.x == 64u, width)
                                      : drainAccumulator<OutT, CompT>(&ctl->accFull[buf], accPh,
                                                                      &ctl->abort, taddr, p, alpha,
                                                                      beta, useC, row, col0, mode,
                                                                      width);
                    if(!drained)
                    {
                        ok = false;
                        break;
                    }
                    mbar_arrive_cluster(map_to_cta(smem_addr(&ctl->accEmpty[buf]), 0));
                }
            }
            if(threadIdx.x == 64u)
            {
                // Shared memory must outlive the TMA stores' reads of it.  The staged last
                // tile waits for exactly that (the writes themselves complete with the grid);
                // the chunked-accumulation path has waited for its stores to be performed.
                if(p.stagedTail != 0u && numChunks == 1u)
                    tma_store_wait_read<0>();
                else
                    tma_store_wait_all<0>();
            }
        }

        // ---------------- teardown ----------------
        tc_fence_before_sync();
        __syncthreads();
        // neither block leaves while the other may still signal it (nothing to order: relaxed)
        cluster_arrive_relaxed();
        cluster_wait();
        if(warp == 1)
        {
            __syncwarp();
            tc_fence_after_sync();
            tmem_dealloc_pair(tmemBase, TMEM_COLS);
        }
        if(threadIdx.x == 0 && ctl->abort.flag != 0u && p.status != nullptr)
        {
            atomicExch(&p.status[1], ctl->abort.code);
            atomicExch(&p.status[0], 1u);
        }
    }

    // ---- host side -----------------------------------------------------------------
    using b200wmma::EncodeFn;
    inline EncodeFn encoder()
    {
        return b200wmma::tensorMapEncoder();
    }

    // Tensor map of the row-major output: rows x cols elements, `ld` apart; box = 32 columns
    // (128 or 64 bytes, swizzled accordingly) x 128 rows.
    // boxCols * elemBytes is 64 or 128 bytes, which is also the swizzle span.
    int makeOutputMap(CUtensorMap* map, CUtensorMapDataType dt, size_t elemBytes, void* base,
                      uint32_t rows, uint32_t cols, uint32_t ld, uint32_t boxCols = 32)
    {
        EncodeFn fn = encoder();
        if(!fn)
            return B200WMMA_ERR_CUDA;
        cuuint64_t dims[2]    = {cols, rows};
        cuuint64_t strides[1] = {cuuint64_t(ld) * elemBytes};
        cuuint32_t box[2]     = {boxCols, 128};
        cuuint32_t estr[2]    = {1, 1};
        CUresult   r = fn(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        boxCols * elemBytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                                   : CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? B200WMMA_OK : B200WMMA_ERR_CUDA;
    }

    template <typename OutT>
    CUtensorMapDataType outputMapType()
    {
        if(std::is_same<OutT, __half>::value)
            return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        if(std::is_same<OutT, __nv_bfloat16>::value)
            return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        if(std::is_same<OutT, int32_t>::value)
            return CU_TENSOR_MAP_DATA_TYPE_INT32;
        return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    }

    // Tensor map of a K-major operand: `rows` rows of `k` elements, `ld` elements apart;
    // box = one 128-byte swizzle row wide, boxRows tall.
    int makeOperandMap(CUtensorMap* map, CUtensorMapDataType dt, size_t elemBytes, void const* base,
                       uint32_t rows, uint32_t k, uint32_t ld, uint32_t boxRows)
    {
        EncodeFn fn = encoder();
        if(!fn)
            return B200WMMA_ERR_CUDA;
        cuuint64_t dims[2]    = {k, rows};
        cuuint64_t strides[1] = {cuuint64_t(ld) * elemBytes};
        cuuint32_t box[2]     = {cuuint32_t(ROW_BYTES / elemBytes), boxRows};
        cuuint32_t estr[2]    = {1, 1};
        CUresult   r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? B200WMMA_OK : B200WMMA_ERR_CUDA;
    }

    // Tensor map of an MN-major operand (column-major A or row-major B): `k` rows of `mn`
    // contiguous elements, `ld` apart; box = 128 bytes of M/N x one ring slot of K rows.
    int makeOperandMapMN(CUtensorMap* map, CUtensorMapDataType dt, size_t elemBytes,
                         void const* base, uint32_t mn, uint32_t k, uint32_t ld)
    {
        EncodeFn fn = encoder();
        if(!fn)
            return B200WMMA_ERR_CUDA;
        cuuint64_t dims[2]    = {mn, k};
        cuuint64_t strides[1] = {cuuint64_t(ld) * elemBytes};
        cuuint32_t box[2]     = {cuuint32_t(ROW_BYTES / elemBytes), cuuint32_t(ROW_BYTES / elemBytes)};
        cuuint32_t estr[2]    = {1, 1};
        CUresult   r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? B200WMMA_OK : B200WMMA_ERR_CUDA;
    }

    // The pair kernel is the default whenever a 256-row tile makes sense; the environment
    // variable B200WMMA_GEMM_PAIR=0 selects the single-block kernel (for comparison).
    bool pairEnabled()
    {
        static const bool on = [] {
            const char* e = getenv("B200WMMA_GEMM_PAIR");
            return !(e && e[0] == '0');
        }();
        return on;
    }

    template <typename KernelT>
    int optInSharedMemory(KernelT kernel, uint32_t bytes, bool (&done)[64])
    {
        static std::mutex           attrMutex;
        std::lock_guard<std::mutex> lock(attrMutex);
        int                         dev = 0;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev < 0 || dev >= 64 || !done[dev])
        {
            // the opt-in shared-memory size is a per-device property of the kernel
            B200WMMA_CUDA_TRY(cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
            if(dev >= 0 && dev < 64)
                done[dev] = true;
        }
        return B200WMMA_OK;
    }

    // `status`: device word that records a bounded wait giving up (may be nullptr).
    // Tile rows per raster band.  Tiles are walked band by band, column by column inside a
    // band, so the rows of A that a band needs stay in L2 while B streams past.  Measured on
    // 8192^3: with 64 MB of A per band (16 tile rows of fp16) DRAM traffic is 3.5 x the
    // algorithmic bytes; 32 MB per band is 0.7 % faster there (less energy under the power
    // cap), while 8-bit inputs and 4096-deep problems -- 32 MB per band at 16 rows -- lose
    // 2 % with 8 rows.  Hence: about 32 MB of A per band, between 4 and 16 tile rows.
    inline uint32_t bandRows(uint32_t k, size_t elemBytes)
    {
        const size_t perTileRow = size_t(P_TILE_M) * k * elemBytes;
        size_t       rows       = perTileRow ? (size_t(32) << 20) / perTileRow : GROUP_M;
        rows                    = rows < 4 ? 4 : rows;
        return uint32_t(rows > GROUP_M ? GROUP_M : rows);
    }

    template <typename InT, typename OutT, typename CompT>
    int launchWithStatus(CUtensorMapDataType dt, uint32_t m, uint32_t n, uint32_t k,
                         void const* a, void const* b, void const* c, void* d, uint32_t lda,
                         uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta,
                         cudaStream_t stream, uint32_t* status, bool aMN = false,
                         bool bMN = false)
    {
        const int sms = b200wmma::smCount();
        if(sms <= 0)
            return B200WMMA_ERR_CUDA;
        // xf32 -> fp32: the tensor core's fp32 accumulator truncates when it aligns addends, a
        // bias that grows with the length of the accumulation chain (measured: 5e-4 in the
        // parity metric after 4096 terms).  Chains are therefore cut every 512 elements of K
        // and the partial sums are added in fp32 with round-to-nearest by the epilogue, using
        // D as the running sum.  Not possible in place (c == d with beta != 0).
        uint32_t chunkKB = 0;
        if(std::is_same<InT, float>::value && std::is_same<OutT, float>::value
           && !(beta != 0.0 && c == d))
        {
            constexpr uint32_t kbPerChunk = 512u / (ROW_BYTES / uint32_t(sizeof(InT)));
            if((k + ROW_BYTES / sizeof(InT) - 1) / (ROW_BYTES / sizeof(InT)) > kbPerChunk)
                chunkKB = kbPerChunk;
        }
        auto aligned32 = [](void const* ptr, uint32_t ld, size_t elem) {
            return (reinterpret_cast<uintptr_t>(ptr) % 32) == 0 && (size_t(ld) * elem) % 32 == 0;
        };
        const uint32_t wide = aligned32(d, ldd, sizeof(OutT))
                                      && (beta == 0.0 || c == nullptr
                                          || aligned32(c, ldc, sizeof(OutT)))
                                  ? 1u
                                  : 0u;
        // B200WMMA_GEMM_BAND overrides the raster band height (tuning only)
        static const uint32_t bandEnv = [] {
            const char* e = getenv("B200WMMA_GEMM_BAND");
            return e ? uint32_t(atoi(e)) : 0u;
        }();
        // Two epilogues.  "rows": every thread stores its own output row (256-bit accesses).
        // "tma": the tile goes through shared memory and leaves by TMA stores / reduce-adds.
        // Measured on 8192^3 fp16 they are equal (the epilogue hides behind the next tile's
        // MMAs either way); with chunked accumulation, where the epilogue runs once per 512
        // elements of K, the TMA form is 1.4x faster because the running sum is added in L2
        // instead of being read back.  TMA stores write whole 16-byte pieces, so they are
        // only used when a row of D ends on a 16-byte boundary (otherwise bytes between n
        // and ldd could be touched).  B200WMMA_GEMM_EPILOGUE=rows|tma forces one (tuning).
        static const int epilogueEnv = [] {
            const char* e = getenv("B200WMMA_GEMM_EPILOGUE");
            return !e ? 0 : (e[0] == 'r' ? 1 : (e[0] == 't' ? 2 : 0));
        }();
        const bool tmaSafe = (size_t(n) * sizeof(OutT)) % 16 == 0;
        bool       useTma  = chunkKB != 0u;
        if(epilogueEnv == 1)
            useTma = false;
        if(epilogueEnv == 2)
            useTma = true;
        useTma = useTma && tmaSafe;
        GemmParams  p{m,    n,      k,       c,    d,  ldc, ldd, alpha, beta,
                     status, chunkKB, wide, BN, bandEnv ? bandEnv : bandRows(k, sizeof(InT)),
                     useTma ? 1u : 0u,
                     aMN ? 1u : 0u,      bMN ? 1u : 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, nullptr, nullptr};
        CUtensorMap mapA, mapB, mapD;
        {
            int rcD = makeOutputMap(&mapD, outputMapType<OutT>(), sizeof(OutT), d, m, n, ldd);
            if(rcD != B200WMMA_OK)
                return rcD;
        }

        // One tile row of at most 128 rows (a skinny product) is bound by how fast one SM can
        // pull its operands, not by the tensor cores: 128 x 8192 x 8192 as 32 single-block
        // tiles of 128 x 256 keeps 32 SMs busy for 57 us.  The pair kernel with 128-wide tiles
        // spreads the same columns of B over 128 SMs (the second block of each pair gets rows
        // past m, which the TMA fills with zeros without reading memory).
        // B200WMMA_GEMM_SKINNY=0 keeps such products on the single-block kernel (comparison).
        static const bool skinnyEnv = [] {
            const char* e = getenv("B200WMMA_GEMM_SKINNY");
            return !(e && e[0] == '0');
        }();
        const bool skinny = skinnyEnv && m <= BM && n >= 4u * 128u;
        if(pairEnabled() && (m > BM || skinny) && sms >= 2)
        {
            // Tile widths.  A tile costs its width plus a fixed part (A is loaded per tile
            // whatever its width, so narrow tiles pay more L2 traffic per flop; measured:
            // 128-wide tiles lose at 4096^3), and a launch takes as long as its busiest pair.
            // Candidates: one width for the whole output (256, 224 or 192 columns).  8192^2 and
            // 4096^2 keep 256; the 2048- and 1024-row shards of a 4- or 8-GPU run of 8192^3
            // come out at 224, which turns 3.46 resp. 1.73 waves into 4 resp. 2 full ones.
            // The kernel can also follow its wide tile columns with 128-wide ones that fill the
            // last, partial wave (TileSchedule; B200WMMA_GEMM_TAIL=1).  That is off by default
            // because it measured slower: a 4096^2 output (256 tiles on 74 pairs, 3.46 waves)
            // as 13 wide + 6 narrow tile columns ran 3 % slower than 16 wide ones -- the last
            // wave's 34 tiles already run faster than a full wave (less contention, higher
            // clock), and narrow tiles cost more than their width suggests.
            const uint32_t pairsMax = uint32_t(sms / 2);
            const uint32_t tilesM   = (m + P_TILE_M - 1) / P_TILE_M;
            // B200WMMA_GEMM_BN forces one width, B200WMMA_GEMM_TMEMSUM=0 keeps the running sum
            // of chunked accumulation in D (tuning / comparison only)
            static const uint32_t bnEnv = [] {
                const char* e = getenv("B200WMMA_GEMM_BN");
                const uint32_t v = e ? uint32_t(atoi(e)) : 0u;
                return (v >= 128 && v <= 256 && v % 32 == 0) ? v : 0u;
            }();
            static const bool tmemSumEnv = [] {
                const char* e = getenv("B200WMMA_GEMM_TMEMSUM");
                return !(e && e[0] == '0');
            }();
            // Chunked accumulation: tiles of at most 160 columns leave room in tensor memory
            // for the running sum, which takes the chunks' read-modify-write of D (an L2 round
            // trip per 512 elements of K) out of the picture.  Measured on xf32 4096^3: 446
            // TFLOP/s with the sum in D (256-wide tiles, TMA reduce-add), 572 with the sum in
            // tensor memory (160-wide tiles); one unbroken chain runs at 588 with 160-wide and
            // 692 with 256-wide tiles, so what is left is the narrower tile, not the chunks.
            const bool tmemSum = chunkKB != 0u && tmemSumEnv;
            if(tmemSum)
            {
                p.sumInTmem = 1u;
                p.tmaStore  = 0u;
            }
            // Less than one wave of the widest tiles: narrower ones down to 128 columns put
            // more SMs to work.
            const uint32_t widest   = tmemSum ? 160u : 256u;
            const bool     subWave  = tilesM * ((n + widest - 1) / widest) < pairsMax;
            const uint32_t narrowest = (tmemSum || subWave) ? 128u : 192u;
            // Tiles of a last wave that is less than half full can be cut in two along K
            // (TileSchedule::splitTiles, drainSplitPart): 256 tiles on 74 pairs then take 3.5
            // waves instead of 4.  Only with one accumulation chain per tile, a workspace to
            // meet in (the allocation-free entry point has none) and K deep enough to halve.
            // OFF unless B200WMMA_GEMM_SPLIT=1: it measured SLOWER on this part -- 4096^3
            // bf16 -> f32 112.8 -> 119.0 us, fp16 96.0 -> 103.0, int8 50.1 -> 65.6 (same box,
            // alternating runs).  Under the 1 kW cap a half-empty last wave is not idle time
            // to be filled: the SMs that have run out let the others clock higher, so wave
            // quantisation costs 4096^3 about 5 %, not the 13.5 % its tile count suggests, and
            // the trip through the workspace costs more than that.
            const char* splitEnv   = getenv("B200WMMA_GEMM_SPLIT");
            const bool  splitAllowed = (splitEnv && splitEnv[0] == '1') && chunkKB == 0u
                                      && status != nullptr
                                      && (k + ROW_BYTES / sizeof(InT) - 1) / (ROW_BYTES / sizeof(InT)) >= 8u;
            auto splitCount = [&](uint32_t tiles) -> uint32_t {
                if(!splitAllowed || tiles <= pairsMax)
                    return 0u;
                const uint32_t rem = tiles % pairsMax;
                return (rem != 0u && 2u * rem <= pairsMax) ? rem : 0u;
            };
            auto makespan = [&](uint32_t bnW, uint32_t wideCols, uint32_t tailCols, uint32_t bnT) {
                const uint32_t total = tilesM * (wideCols + tailCols);
                const uint32_t pairs = total < pairsMax ? total : pairsMax;
                if(tailCols == 0u && splitCount(total) != 0u)
                    // whole waves, then half a tile plus the fix-up through the workspace
                    return (total / pairsMax) * (bnW + 64u) + (bnW + 64u) / 2u + 24u;
                TileSchedule   sc{tilesM, wideCols, tailCols, bnW, bnT, GROUP_M, pairs, 0u, 0u};
                uint32_t       worst = 0;
                for(uint32_t pr = 0; pr < pairs; ++pr)
                {
                    uint32_t load = 0, tm, col0, width;
                    for(uint32_t i = 0; sc.get(pr, i, tm, col0, width); ++i)
                        load += width + 64u;
                    worst = load > worst ? load : worst;
                }
                return worst;
            };
            uint32_t bn = widest, wideCols = (n + widest - 1) / widest, tailCols = 0, bnTail = 0;
            if(bnEnv != 0u && !(tmemSum && bnEnv > 160u))
            {
                bn       = bnEnv;
                wideCols = (n + bn - 1) / bn;
            }
            else if(n <= widest)
            {
                // narrower than one tile: no wider than needed (multiples of 32)
                bn       = n <= 128u ? 128u : (n + 31u) / 32u * 32u;
                wideCols = 1;
            }
            else
            {
                uint32_t best = 0xffffffffu;
                for(uint32_t cand = widest; cand >= narrowest; cand -= 32)
                {
                    const uint32_t cols = (n + cand - 1) / cand;
                    const uint32_t cost = makespan(cand, cols, 0, 0);
                    if(cost < best)
                        best = cost, bn = cand, wideCols = cols, tailCols = 0, bnTail = 0;
                }
                // wide columns, then 128-wide ones over what is left (tuning switch, see above)
                const char* tailEnv = getenv("B200WMMA_GEMM_TAIL");
                if(widest > 128u && tailEnv && tailEnv[0] == '1')
                {
                    const uint32_t full = n / widest;
                    for(uint32_t wc = full > 6u ? full - 6u : 1u; wc <= full; ++wc)
                    {
                        const uint32_t left = n - wc * widest;
                        if(left == 0u)
                            continue;
                        const uint32_t tc   = (left + 127u) / 128u;
                        const uint32_t cost = makespan(widest, wc, tc, 128u);
                        if(cost + cost / 50u < best)
                            best = cost, bn = widest, wideCols = wc, tailCols = tc, bnTail = 128u;
                    }
                }
            }
            p.bn       = bn;
            p.wideCols = wideCols;
            p.tailCols = tailCols;
            p.bnTail   = bnTail;
            if(tailCols == 0u)
            {
                const uint32_t split = splitCount(tilesM * wideCols);
                if(split != 0u && split * 2u <= 256u)
                {
                    // per split tile: 2 halves x 2 blocks x 128 rows x 256 columns x 4 bytes
                    uint32_t* ctr = nullptr;
                    void*     ws  = b200wmma::splitWorkspace(size_t(split) * 4u * 128u * 256u * 4u, &ctr);
                    if(ws != nullptr)
                    {
                        p.splitTiles = split;
                        p.splitWs    = static_cast<float*>(ws);
                        p.splitCtr   = ctr;
                    }
                }
            }
            // Tile order (TileSchedule).  B200WMMA_GEMM_ORDER = digits "smp" (snake, mirror on
            // alternate launches, k-blocks prefetched into L2), e.g. "000" for the plain
            // order; tuning and comparison only.
            static const char* orderEnv = getenv("B200WMMA_GEMM_ORDER");
            const bool snakeOn    = !(orderEnv && orderEnv[0] == '0');
            const bool mirrorOn   = !(orderEnv && orderEnv[0] && orderEnv[1] == '0');
            const uint32_t prefKB = (orderEnv && orderEnv[0] && orderEnv[1] && orderEnv[2] >= '0'
                                     && orderEnv[2] <= '9')
                                        ? uint32_t(orderEnv[2] - '0')
                                        : P_STAGES;
            p.snake    = snakeOn ? 1u : 0u;
            p.prefetch = prefKB;
            {
                // B200WMMA_GEMM_L2HINT=0..7 forces the cache hints (bit 0: A, bit 1: B, bit 2: D;
                // comparison)
                const char* hintEnv = getenv("B200WMMA_GEMM_L2HINT");
                const bool  streams = size_t(n) * k * sizeof(InT) > (size_t(48) << 20);
                const bool  bigD    = size_t(m) * n * sizeof(OutT) >= (size_t(32) << 20);
                p.l2Hints = hintEnv ? uint32_t(hintEnv[0] - '0') & 7u
                                    : (streams ? 2u : 0u) | (bigD ? 4u : 0u);
            }
            if(mirrorOn)
            {
                // Launches alternate between the forward and the mirrored order, so that each
                // starts on the operands its predecessor left in L2 (the usual case being the
                // same B, or the same A and B, launch after launch).  The result does not
                // depend on the order.
                static std::atomic<uint32_t> launchParity[64];
                int                          dev = 0;
                if(cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64)
                    p.mirror = launchParity[dev].fetch_add(1u, std::memory_order_relaxed) & 1u;
                else
                    (void)cudaGetLastError();
            }
            int rc = aMN ? makeOperandMapMN(&mapA, dt, sizeof(InT), a, m, k, lda)
                         : makeOperandMap(&mapA, dt, sizeof(InT), a, m, k, lda, 128);
            if(rc != B200WMMA_OK)
                return rc;
            rc = bMN ? makeOperandMapMN(&mapB, dt, sizeof(InT), b, n, k, ldb)
                     : makeOperandMap(&mapB, dt, sizeof(InT), b, n, k, ldb, bn / 2);
            if(rc != B200WMMA_OK)
                return rc;
            // B again with the box of a narrow tile (K-major boxes are half a tile high; the
            // MN-major box does not depend on the tile width)
            CUtensorMap mapBTail = mapB;
            if(bnTail != 0u && !bMN)
            {
                rc = makeOperandMap(&mapBTail, dt, sizeof(InT), b, n, k, ldb, bnTail / 2);
                if(rc != B200WMMA_OK)
                    return rc;
            }
            // The last tile of every block leaves through the idle operand ring and TMA stores
            // of 128-byte rows (drainLastTileStaged) when TMA stores are safe for D -- they
            // write whole 16-byte pieces, so a row of D must end on a 16-byte boundary -- K
            // is accumulated in one chain and the output is a 16-bit type (1024-row shard of
            // 8192^3 fp16: 92.85 -> 92.6 us; with 128 KB of 32-bit output per block to stage
            // it is the slower form, int8 -> int32 4096^3 50.7 -> 52.2 us).
            // B200WMMA_GEMM_STAGED_TAIL=0 switches it off.
            static const bool stagedEnv = [] {
                const char* e = getenv("B200WMMA_GEMM_STAGED_TAIL");
                return !(e && e[0] == '0');
            }();
            CUtensorMap mapDWide = mapD;
            if(stagedEnv && tmaSafe && chunkKB == 0u && epilogueEnv == 0 && sizeof(OutT) == 2)
            {
                p.stagedTail = 1u;
                if(sizeof(OutT) == 2)
                {
                    rc = makeOutputMap(&mapDWide, outputMapType<OutT>(), sizeof(OutT), d, m, n,
                                       ldd, 64);
                    if(rc != B200WMMA_OK)
                        return rc;
                }
            }
            // beta == 0: every tile but a block's last leaves through the staging buffers and
            // TMA stores of whole 128-byte (64-byte) rows rather than by per-thread row
            // stores.  The two measure alike where the MMAs of a tile outlast its drain
            // (8192^3 fp16); where they do not -- int8 -> int32 at K = 4096 has 8.6 us of MMAs
            // per tile and 128 KB to write per block -- the row stores are the slower and the
            // more fragile form (50.7 -> 57.6 us after unrelated changes to the kernel moved
            // its code around; 50.8 us through TMA before and after).
            if(tmaSafe && epilogueEnv == 0 && chunkKB == 0u && (beta == 0.0 || c == nullptr))
                p.tmaStore = 1u;
            // beta != 0 with K accumulated in one chain: C is fetched by TMA as well
            // (drainAccumulatorTmaC) when both C and D meet the TMA's alignment rules.
            // B200WMMA_GEMM_CTMA=0 keeps the row epilogue for C (comparison).
            static const bool cTmaEnv = [] {
                const char* e = getenv("B200WMMA_GEMM_CTMA");
                return !(e && e[0] == '0');
            }();
            CUtensorMap mapC = mapD;
            if(cTmaEnv && beta != 0.0 && c != nullptr && (chunkKB == 0u || p.sumInTmem != 0u)
               && tmaSafe
               && epilogueEnv == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0
               && (size_t(ldc) * sizeof(OutT)) % 16 == 0)
            {
                rc = makeOutputMap(&mapC, outputMapType<OutT>(), sizeof(OutT),
                                   const_cast<void*>(c), m, n, ldc);
                if(rc != B200WMMA_OK)
                    return rc;
                static const bool cdHintEnv = [] {
                    const char* e = getenv("B200WMMA_GEMM_CD_HINT");
                    return !(e && e[0] == '0');
                }();
                p.cViaTma = cdHintEnv ? 3u : 1u;
            }
            auto        kernel = gemm_tcgen05_pair_kernel<InT, OutT, CompT>;
            static bool done[64] = {};
            rc = optInSharedMemory(kernel, P_SMEM_BYTES, done);
            if(rc != B200WMMA_OK)
                return rc;
            const uint32_t tiles = tilesM * (wideCols + tailCols) + p.splitTiles; // work items
            const uint32_t pairs = tiles < pairsMax ? tiles : pairsMax;
            return b200wmma::cudaToStatus(b200wmma::launchOverlapped(
                kernel, dim3(2 * pairs), dim3(NUM_THREADS), P_SMEM_BYTES, stream, mapA, mapB,
                mapBTail, mapD, mapDWide, mapC, p));
        }

        int rc = aMN ? makeOperandMapMN(&mapA, dt, sizeof(InT), a, m, k, lda)
                     : makeOperandMap(&mapA, dt, sizeof(InT), a, m, k, lda, BM);
        if(rc != B200WMMA_OK)
            return rc;
        rc = bMN ? makeOperandMapMN(&mapB, dt, sizeof(InT), b, n, k, ldb)
                 : makeOperandMap(&mapB, dt, sizeof(InT), b, n, k, ldb, BN);
        if(rc != B200WMMA_OK)
            return rc;
        auto        kernel = gemm_tcgen05_kernel<InT, OutT, CompT>;
        static bool done[64] = {};
        rc = optInSharedMemory(kernel, SMEM_BYTES, done);
        if(rc != B200WMMA_OK)
            return rc;
        const uint32_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
        const uint32_t grid  = tiles < uint32_t(sms) ? tiles : uint32_t(sms);
        return b200wmma::cudaToStatus(b200wmma::launchOverlapped(
            kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, mapA, mapB, mapD, p));
    }

    template <typename InT, typename OutT, typename CompT>
    int launch(CUtensorMapDataType dt, uint32_t m, uint32_t n, uint32_t k, void const* a,
               void const* b, void const* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
               uint32_t ldd, double alpha, double beta, cudaStream_t stream, bool aMN, bool bMN)
    {
        return launchWithStatus<InT, OutT, CompT>(dt, m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
                                                  alpha, beta, stream,
                                                  b200wmma::deviceStatusWord(), aMN, bMN);
    }

    // out[c][r] = in[r][c]: turns an MN-major operand into the K-major form the
    // tensor-core path reads.  rows x cols elements, 32x32 tiles through shared memory.
    template <typename T>
    __global__ void transposeKernel(T const* __restrict__ in, T* __restrict__ out, uint32_t rows,
                                    uint32_t cols, uint32_t ldIn, uint32_t ldOut)
    {
        __shared__ T   tile[32][33];
        const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
        for(uint32_t j = threadIdx.y; j < 32; j += blockDim.y)
        {
            const uint32_t r = r0 + j, c = c0 + threadIdx.x;
            if(r < rows && c < cols)
                tile[j][threadIdx.x] = in[size_t(r) * ldIn + c];
        }
        __syncthreads();
        for(uint32_t j = threadIdx.y; j < 32; j += blockDim.y)
        {
            const uint32_t c = c0 + j, r = r0 + threadIdx.x;
            if(r < rows && c < cols)
                out[size_t(c) * ldOut + r] = tile[threadIdx.x][j];
        }
    }

    template <typename T>
    int transposeInto(T const* in, T* out, uint32_t rows, uint32_t cols, uint32_t ldIn,
                      uint32_t ldOut, cudaStream_t stream)
    {
        dim3 block(32, 8);
        dim3 grid((cols + 31) / 32, (rows + 31) / 32);
        transposeKernel<T><<<grid, block, 0, stream>>>(in, out, rows, cols, ldIn, ldOut);
        return b200wmma::cudaToStatus(cudaGetLastError());
    }

    inline uint32_t roundUp(uint32_t v, uint32_t m)
    {
        return (v + m - 1) / m * m;
    }

    // Every layout combination is read in place: a row-major A / column-major B tile is
    // K-major for the tensor core, a column-major A / row-major B tile MN-major; the TMA box
    // shape and the shared-memory and instruction descriptors follow the layout.
    template <typename InT, typename OutT, typename CompT>
    int run(CUtensorMapDataType dt, uint32_t m, uint32_t n, uint32_t k, void const* a,
            void const* b, void const* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
            uint32_t ldd, double alpha, double beta, int layoutA, int layoutB, cudaStream_t stream)
    {
        bool aMN = layoutA == B200WMMA_COL_MAJOR;
        bool bMN = layoutB == B200WMMA_ROW_MAJOR;
        if constexpr(sizeof(InT) == 4)
        {
            // 32-bit (tf32) operands are fed K-major only: with the MN-major descriptors that
            // work for 8- and 16-bit types the tensor core returned zeros for kind::tf32
            // (it wants a different swizzle atom for 32-bit transposes).  Column-major A /
            // row-major B are therefore transposed into a per-device scratch buffer first.
            if(aMN || bMN)
            {
                constexpr uint32_t E16    = 16 / sizeof(InT);
                const uint32_t     kPad   = roundUp(k, E16);
                const size_t       aBytes = aMN ? size_t(m) * kPad * sizeof(InT) : 0;
                const size_t       bBytes = bMN ? size_t(n) * kPad * sizeof(InT) : 0;
                const size_t       aPad   = (aBytes + 255) / 256 * 256;
                uint8_t* scratch = static_cast<uint8_t*>(b200wmma::deviceScratch(aPad + bBytes));
                if(!scratch)
                    return B200WMMA_ERR_CUDA;
                if(aMN)
                {
                    if(lda < m)
                        return B200WMMA_ERR_INVALID_ARG;
                    int rc = transposeInto(static_cast<InT const*>(a),
                                           reinterpret_cast<InT*>(scratch), k, m, lda, kPad, stream);
                    if(rc != B200WMMA_OK)
                        return rc;
                    a   = scratch;
                    lda = kPad;
                    aMN = false;
                }
                if(bMN)
                {
                    if(ldb < n)
                        return B200WMMA_ERR_INVALID_ARG;
                    int rc = transposeInto(static_cast<InT const*>(b),
                                           reinterpret_cast<InT*>(scratch + aPad), k, n, ldb, kPad,
                                           stream);
                    if(rc != B200WMMA_OK)
                        return rc;
                    b   = scratch + aPad;
                    ldb = kPad;
                    bMN = false;
                }
            }
        }
        auto misaligned = [](void const* ptr, uint32_t ld, size_t elem) {
            return (reinterpret_cast<uintptr_t>(ptr) % 16) != 0 || (size_t(ld) * elem) % 16 != 0;
        };
        if(misaligned(a, lda, sizeof(InT)) || misaligned(b, ldb, sizeof(InT))
           || misaligned(d, ldd, sizeof(OutT)) || (beta != 0.0 && misaligned(c, ldc, sizeof(OutT))))
            return B200WMMA_ERR_ALIGNMENT;
        if(lda < (aMN ? m : k) || ldb < (bMN ? n : k) || ldd < n || (beta != 0.0 && ldc < n))
            return B200WMMA_ERR_INVALID_ARG;
        return launch<InT, OutT, CompT>(dt, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,
                                        stream, aMN, bMN);
    }

    // ---- float32_t: full fp32 products from three TF32 products ------------------------------
    // The tensor core has no fp32 operand format.  x = hi + lo with hi = tf32(x) and
    // lo = tf32(x - hi) keeps 21 of x's 24 significand bits, and
    //     A B  ~  Ahi Bhi + Alo Bhi + Ahi Blo            (the lo x lo term, 2^-22 relative, dropped)
    // -- the same split mma_sync uses for float32_t fragments.  Here it is three runs of the
    // xf32 kernel over split copies of the operands: D = alpha Ahi Bhi + beta C, then twice
    // D += alpha (correction term).  The main term uses the chunked accumulation of the xf32
    // path; the corrections are 2^-11 of it, so a single chain is accurate enough for them.
    // The split pass also brings column-major A / row-major B into K-major order.
    __device__ inline float tf32Round(float v)
    {
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
        return __uint_as_float(u);
    }

    // in: `rows` x `cols` values, element (r, c) at in[r * ldIn + c]; TRANSPOSE writes element
    // (r, c) to out[c * ldOut + r], otherwise to out[r * ldOut + c].
    template <bool TRANSPOSE>
    __global__ void splitTf32Kernel(float const* __restrict__ in, float* __restrict__ hi,
                                    float* __restrict__ lo, uint32_t rows, uint32_t cols,
                                    uint32_t ldIn, uint32_t ldOut)
    {
        __shared__ float tileHi[32][33], tileLo[32][33];
        const uint32_t   c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
        for(uint32_t j = threadIdx.y; j < 32; j += blockDim.y)
        {
            const uint32_t r = r0 + j, c = c0 + threadIdx.x;
            if(r < rows && c < cols)
            {
                const float v = in[size_t(r) * ldIn + c];
                const float h = tf32Round(v);
                const float l = tf32Round(v - h);
                if constexpr(TRANSPOSE)
                {
                    tileHi[j][threadIdx.x] = h;
                    tileLo[j][threadIdx.x] = l;
                }
                else
                {
                    hi[size_t(r) * ldOut + c] = h;
                    lo[size_t(r) * ldOut + c] = l;
                }
            }
        }
        if constexpr(TRANSPOSE)
        {
            __syncthreads();
            for(uint32_t j = threadIdx.y; j < 32; j += blockDim.y)
            {
                const uint32_t c = c0 + j, r = r0 + threadIdx.x;
                if(r < rows && c < cols)
                {
                    hi[size_t(c) * ldOut + r] = tileHi[threadIdx.x][j];
                    lo[size_t(c) * ldOut + r] = tileLo[threadIdx.x][j];
                }
            }
        }
    }

    int splitTf32(float const* in, float* hi, float* lo, uint32_t rows, uint32_t cols,
                  uint32_t ldIn, uint32_t ldOut, bool transpose, cudaStream_t stream)
    {
        dim3 block(32, 8);
        dim3 grid((cols + 31) / 32, (rows + 31) / 32);
        if(transpose)
            splitTf32Kernel<true><<<grid, block, 0, stream>>>(in, hi, lo, rows, cols, ldIn, ldOut);
        else
            splitTf32Kernel<false><<<grid, block, 0, stream>>>(in, hi, lo, rows, cols, ldIn, ldOut);
        return b200wmma::cudaToStatus(cudaGetLastError());
    }

    int runF32(uint32_t m, uint32_t n, uint32_t k, void const* a, void const* b, void const* c,
               void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha,
               double beta, int layoutA, int layoutB, cudaStream_t stream)
    {
        const bool aMN = layoutA == B200WMMA_COL_MAJOR, bMN = layoutB == B200WMMA_ROW_MAJOR;
        auto       misaligned = [](void const* ptr, uint32_t ld) {
            return (reinterpret_cast<uintptr_t>(ptr) % 16) != 0 || (size_t(ld) * 4) % 16 != 0;
        };
        if(misaligned(d, ldd) || (beta != 0.0 && misaligned(c, ldc)))
            return B200WMMA_ERR_ALIGNMENT;
        if(lda < (aMN ? m : k) || ldb < (bMN ? n : k) || ldd < n || (beta != 0.0 && ldc < n))
            return B200WMMA_ERR_INVALID_ARG;
        const uint32_t kPad   = roundUp(k, 4);
        const size_t   aElems = (size_t(m) * kPad + 63) / 64 * 64; // keeps every part 256-byte aligned
        const size_t   bElems = (size_t(n) * kPad + 63) / 64 * 64;
        float* scratch = static_cast<float*>(b200wmma::deviceScratch((2 * aElems + 2 * bElems) * 4));
        if(!scratch)
            return B200WMMA_ERR_CUDA;
        float *aHi = scratch, *aLo = aHi + aElems, *bHi = aLo + aElems, *bLo = bHi + bElems;
        // A is m x k: row-major = K-major already; column-major is k rows of m values.
        int rc = aMN ? splitTf32(static_cast<float const*>(a), aHi, aLo, k, m, lda, kPad, true, stream)
                     : splitTf32(static_cast<float const*>(a), aHi, aLo, m, k, lda, kPad, false,
                                 stream);
        if(rc != B200WMMA_OK)
            return rc;
        // B is k x n: column-major = n rows of k values = K-major; row-major is k rows of n.
        rc = bMN ? splitTf32(static_cast<float const*>(b), bHi, bLo, k, n, ldb, kPad, true, stream)
                 : splitTf32(static_cast<float const*>(b), bHi, bLo, n, k, ldb, kPad, false, stream);
        if(rc != B200WMMA_OK)
            return rc;
        const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        rc = launch<float, float, float>(dt, m, n, k, aHi, bHi, c, d, kPad, kPad, ldc, ldd, alpha,
                                         beta, stream, false, false);
        if(rc != B200WMMA_OK)
            return rc;
        rc = launch<float, float, float>(dt, m, n, k, aLo, bHi, d, d, kPad, kPad, ldd, ldd, alpha, 1.0,
                                         stream, false, false);
        if(rc != B200WMMA_OK)
            return rc;
        return launch<float, float, float>(dt, m, n, k, aHi, bLo, d, d, kPad, kPad, ldd, ldd, alpha,
                                           1.0, stream, false, false);
    }
} // namespace

namespace b200wmma
{
    // Implemented in gemm_f64.cu
    int gemmF64(uint32_t m, uint32_t n, uint32_t k, double const* a, double const* b,
                double const* c, double* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                double alpha, double beta, int layoutA, int layoutB, cudaStream_t stream);
} // namespace b200wmma

extern "C" int b200wmma_gemm(int in_dtype, int out_dtype, uint32_t m, uint32_t n, uint32_t k,
                             const void* a, const void* b, const void* c, void* d, uint32_t lda,
                             uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta,
                             int layout_a, int layout_b, void* stream)
{
    if(!a || !b || !d || m == 0 || n == 0 || k == 0)
        return B200WMMA_ERR_INVALID_ARG;
    if(beta != 0.0 && !c)
        return B200WMMA_ERR_INVALID_ARG;
    if((layout_a != B200WMMA_ROW_MAJOR && layout_a != B200WMMA_COL_MAJOR)
       || (layout_b != B200WMMA_ROW_MAJOR && layout_b != B200WMMA_COL_MAJOR))
        return B200WMMA_ERR_INVALID_ARG;
    auto s = static_cast<cudaStream_t>(stream);
#define B200WMMA_GEMM_CASE(I, O, IT, OT, CT, TM)                                              \
    if(in_dtype == I && out_dtype == O)                                                       \
        return run<IT, OT, CT>(TM, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta,      \
                               layout_a, layout_b, s);
    B200WMMA_GEMM_CASE(B200WMMA_F16, B200WMMA_F16, __half, __half, float,
                       CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
    B200WMMA_GEMM_CASE(B200WMMA_F16, B200WMMA_F32, __half, float, float,
                       CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
    B200WMMA_GEMM_CASE(B200WMMA_BF16, B200WMMA_F32, __nv_bfloat16, float, float,
                       CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
    B200WMMA_GEMM_CASE(B200WMMA_BF16, B200WMMA_BF16, __nv_bfloat16, __nv_bfloat16, float,
                       CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
    B200WMMA_GEMM_CASE(B200WMMA_XF32, B200WMMA_F32, float, float, float,
                       CU_TENSOR_MAP_DATA_TYPE_FLOAT32)
    B200WMMA_GEMM_CASE(B200WMMA_I8, B200WMMA_I32, int8_t, int32_t, int32_t,
                       CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_GEMM_CASE(B200WMMA_E4M3, B200WMMA_BF16, __nv_fp8_e4m3, __nv_bfloat16, float,
                       CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_GEMM_CASE(B200WMMA_E4M3, B200WMMA_F32, __nv_fp8_e4m3, float, float,
                       CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_GEMM_CASE(B200WMMA_E5M2, B200WMMA_BF16, __nv_fp8_e5m2, __nv_bfloat16, float,
                       CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_GEMM_CASE(B200WMMA_E5M2, B200WMMA_F32, __nv_fp8_e5m2, float, float,
                       CU_TENSOR_MAP_DATA_TYPE_UINT8)
#undef B200WMMA_GEMM_CASE
    if(in_dtype == B200WMMA_F32 && out_dtype == B200WMMA_F32)
        return runF32(m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, layout_a, layout_b, s);
    if(in_dtype == B200WMMA_F64 && out_dtype == B200WMMA_F64)
        return b200wmma::gemmF64(m, n, k, static_cast<double const*>(a),
                                 static_cast<double const*>(b), static_cast<double const*>(c),
                                 static_cast<double*>(d), lda, ldb, ldc, ldd, alpha, beta, layout_a,
                                 layout_b, s);
    return B200WMMA_ERR_UNSUPPORTED;
}

extern "C" int b200wmma_gemm_host(int in_dtype, int out_dtype, uint32_t m, uint32_t n, uint32_t k,
                                  const void* a, const void* b, const void* c, void* d,
                                  uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                                  double alpha, double beta, int layout_a, int layout_b,
                                  void* stream)
{
    if(!a || !b || !d || m == 0 || n == 0 || k == 0 || (beta != 0.0 && !c))
        return B200WMMA_ERR_INVALID_ARG;
    if((layout_a != B200WMMA_ROW_MAJOR && layout_a != B200WMMA_COL_MAJOR)
       || (layout_b != B200WMMA_ROW_MAJOR && layout_b != B200WMMA_COL_MAJOR))
        return B200WMMA_ERR_INVALID_ARG; // the copy sizes below depend on the layouts
    const size_t inB = b200wmma::dtypeSize(in_dtype), outB = b200wmma::dtypeSize(out_dtype);
    if(inB == 0 || outB == 0)
        return B200WMMA_ERR_UNSUPPORTED;
    // staging buffers, copy streams and events exist once per device: one call at a time
    std::mutex* hostCall = b200wmma::hostCallMutex();
    if(!hostCall)
        return B200WMMA_ERR_CUDA;
    std::lock_guard<std::mutex> hostLock(*hostCall);
    auto         s      = static_cast<cudaStream_t>(stream);
    const size_t aBytes = size_t(layout_a == B200WMMA_ROW_MAJOR ? m : k) * lda * inB;
    const size_t bBytes = size_t(layout_b == B200WMMA_ROW_MAJOR ? k : n) * ldb * inB;
    const size_t cBytes = beta != 0.0 ? size_t(m) * ldc * outB : 0;
    const size_t dBytes = size_t(m) * ldd * outB;
    void*        dA     = b200wmma::stagingBuffer(0, aBytes);
    void*        dB     = b200wmma::stagingBuffer(1, bBytes);
    void*        dC     = cBytes ? b200wmma::stagingBuffer(2, cBytes) : nullptr;
    void*        dD     = b200wmma::stagingBuffer(3, dBytes);
    if(!dA || !dB || !dD || (cBytes && !dC))
        return B200WMMA_ERR_CUDA;
    // Pipelined form (A row-major): B goes first, then A (and C) in row slabs on a copy
    // stream; the GEMM of slab i runs as soon as slab i has landed, and its rows of D return
    // on a second copy stream while later slabs are still arriving.  The transfer of the
    // inputs is the critical path; compute and the D copies hide behind it.
    b200wmma::HostPipe* pipe = b200wmma::hostPipe();
    if(pipe && layout_a == B200WMMA_ROW_MAJOR && m >= 1024)
    {
        const uint32_t nChunks   = 8;
        const uint32_t chunkRows = ((m + nChunks - 1) / nChunks + 255) / 256 * 256;
        B200WMMA_CUDA_TRY(cudaEventRecord(pipe->start, s));
        B200WMMA_CUDA_TRY(cudaStreamWaitEvent(pipe->h2d, pipe->start, 0));
        B200WMMA_CUDA_TRY(cudaStreamWaitEvent(pipe->d2h, pipe->start, 0));
        B200WMMA_CUDA_TRY(cudaMemcpyAsync(dB, b, bBytes, cudaMemcpyHostToDevice, pipe->h2d));
        B200WMMA_CUDA_TRY(cudaEventRecord(pipe->bReady, pipe->h2d));
        B200WMMA_CUDA_TRY(cudaStreamWaitEvent(s, pipe->bReady, 0));
        uint32_t chunk = 0;
        for(uint32_t r0 = 0; r0 < m; r0 += chunkRows, ++chunk)
        {
            const uint32_t rows = (m - r0) < chunkRows ? (m - r0) : chunkRows;
            const size_t   aOff = size_t(r0) * lda * inB, cOff = size_t(r0) * ldc * outB;
            const size_t   dOff = size_t(r0) * ldd * outB;
            B200WMMA_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(dA) + aOff,
                                              static_cast<uint8_t const*>(a) + aOff,
                                              size_t(rows) * lda * inB, cudaMemcpyHostToDevice,
                                              pipe->h2d));
            if(cBytes)
                B200WMMA_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(dC) + cOff,
                                                  static_cast<uint8_t const*>(c) + cOff,
                                                  size_t(rows) * ldc * outB,
                                                  cudaMemcpyHostToDevice, pipe->h2d));
            B200WMMA_CUDA_TRY(cudaEventRecord(pipe->in[chunk], pipe->h2d));
            B200WMMA_CUDA_TRY(cudaStreamWaitEvent(s, pipe->in[chunk], 0));
            int rc = b200wmma_gemm(in_dtype, out_dtype, rows, n, k,
                                   static_cast<uint8_t*>(dA) + aOff, dB,
                                   cBytes ? static_cast<uint8_t*>(dC) + cOff : nullptr,
                                   static_cast<uint8_t*>(dD) + dOff, lda, ldb, ldc, ldd, alpha,
                                   beta, layout_a, layout_b, stream);
            if(rc != B200WMMA_OK)
                return rc;
            B200WMMA_CUDA_TRY(cudaEventRecord(pipe->out[chunk], s));
            B200WMMA_CUDA_TRY(cudaStreamWaitEvent(pipe->d2h, pipe->out[chunk], 0));
            B200WMMA_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(d) + dOff,
                                              static_cast<uint8_t*>(dD) + dOff,
                                              size_t(rows) * ldd * outB, cudaMemcpyDeviceToHost,
                                              pipe->d2h));
        }
        B200WMMA_CUDA_TRY(cudaStreamSynchronize(pipe->d2h));
        B200WMMA_CUDA_TRY(cudaStreamSynchronize(s));
        return B200WMMA_OK;
    }

    B200WMMA_CUDA_TRY(cudaMemcpyAsync(dA, a, aBytes, cudaMemcpyHostToDevice, s));
    B200WMMA_CUDA_TRY(cudaMemcpyAsync(dB, b, bBytes, cudaMemcpyHostToDevice, s));
    if(cBytes)
        B200WMMA_CUDA_TRY(cudaMemcpyAsync(dC, c, cBytes, cudaMemcpyHostToDevice, s));
    int rc = b200wmma_gemm(in_dtype, out_dtype, m, n, k, dA, dB, dC, dD, lda, ldb, ldc, ldd, alpha,
                           beta, layout_a, layout_b, stream);
    if(rc != B200WMMA_OK)
        return rc;
    B200WMMA_CUDA_TRY(cudaMemcpyAsync(d, dD, dBytes, cudaMemcpyDeviceToHost, s));
    B200WMMA_CUDA_TRY(cudaStreamSynchronize(s));
    return B200WMMA_OK;
}


// =========================================================================================
// GEMM for callers that must not allocate
// =========================================================================================
namespace
{
    // Transposition scratch that is part of the library image instead of coming from
    // cudaMalloc.  Every GPU that loads this library carries these 8 MiB until the process
    // exits, whether or not the entry point below is ever called.
    constexpr size_t NOALLOC_SCRATCH_BYTES = size_t(8) << 20;
    static __device__ __align__(256) uint8_t g_noallocScratch[NOALLOC_SCRATCH_BYTES];

    // In host code `g_noallocScratch` is only a handle for the symbol; the address a kernel
    // can use is asked from the runtime once per device and remembered here.
    std::mutex g_noallocMutex;
    uint8_t*   g_noallocAddress[64] = {};

    int noallocScratch(uint8_t** out)
    {
        int dev = -1;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev < 0 || dev >= 64)
            return B200WMMA_ERR_CUDA;
        std::lock_guard<std::mutex> lock(g_noallocMutex);
        if(!g_noallocAddress[dev])
        {
            void* p = nullptr;
            B200WMMA_CUDA_TRY(cudaGetSymbolAddress(&p, g_noallocScratch));
            if(!p)
                return B200WMMA_ERR_CUDA;
            g_noallocAddress[dev] = static_cast<uint8_t*>(p);
        }
        *out = g_noallocAddress[dev];
        return B200WMMA_OK;
    }

    template <typename InT, typename OutT, typename CompT>
    int runNoAlloc(CUtensorMapDataType dt, uint32_t m, uint32_t n, uint32_t k, void const* a,
                   void const* b, void const* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                   uint32_t ldd, double alpha, double beta, int layoutA, int layoutB,
                   cudaStream_t stream)
    {
        constexpr uint32_t E16 = 16 / sizeof(InT);
        // Every argument is checked before anything is enqueued: the transposition pass
        // below reads a and b with the caller's leading dimensions.
        auto misaligned = [](void const* ptr, uint32_t ld, size_t elem) {
            return (reinterpret_cast<uintptr_t>(ptr) % 16) != 0 || (size_t(ld) * elem) % 16 != 0;
        };
        const bool aT = layoutA == B200WMMA_COL_MAJOR, bT = layoutB == B200WMMA_ROW_MAJOR;
        if(lda < (aT ? m : k) || ldb < (bT ? n : k) || ldd < n || (beta != 0.0 && ldc < n))
            return B200WMMA_ERR_INVALID_ARG;
        // operands that are transposed are read with ordinary loads and need no alignment
        if((!aT && misaligned(a, lda, sizeof(InT))) || (!bT && misaligned(b, ldb, sizeof(InT)))
           || misaligned(d, ldd, sizeof(OutT)) || (beta != 0.0 && misaligned(c, ldc, sizeof(OutT))))
            return B200WMMA_ERR_ALIGNMENT;
        if(aT || bT)
        {
            const uint32_t kPad   = roundUp(k, E16);
            const size_t   aBytes = layoutA == B200WMMA_COL_MAJOR ? size_t(m) * kPad * sizeof(InT) : 0;
            const size_t   bBytes = layoutB == B200WMMA_ROW_MAJOR ? size_t(n) * kPad * sizeof(InT) : 0;
            const size_t   aPad   = (aBytes + 255) / 256 * 256;
            if(aPad + bBytes > NOALLOC_SCRATCH_BYTES)
                return B200WMMA_ERR_TOO_LARGE;
            uint8_t* scratch = nullptr;
            int      rc      = noallocScratch(&scratch);
            if(rc != B200WMMA_OK)
                return rc;
            // The array still holds whatever the previous call left there.  Nothing has to
            // be cleared: every element inside the [rows x k] extents the tensor maps cover
            // is rewritten below, and the row padding beyond k is never read.
            if(layoutA == B200WMMA_COL_MAJOR)
            {
                rc = transposeInto(static_cast<InT const*>(a), reinterpret_cast<InT*>(scratch), k,
                                   m, lda, kPad, stream);
                if(rc != B200WMMA_OK)
                    return rc;
                a   = scratch;
                lda = kPad;
            }
            if(layoutB == B200WMMA_ROW_MAJOR)
            {
                rc = transposeInto(static_cast<InT const*>(b),
                                   reinterpret_cast<InT*>(scratch + aPad), k, n, ldb, kPad, stream);
                if(rc != B200WMMA_OK)
                    return rc;
                b   = scratch + aPad;
                ldb = kPad;
            }
        }
        // No status word: the library's one comes from cudaMalloc.
        return launchWithStatus<InT, OutT, CompT>(dt, m, n, k, a, b, c, d, lda, ldb, ldc, ldd,
                                                  alpha, beta, stream, nullptr);
    }
} // namespace

extern "C" int b200wmma_gemm_noalloc(int in_dtype, int out_dtype, uint32_t m, uint32_t n,
                                     uint32_t k, const void* a, const void* b, const void* c,
                                     void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                     uint32_t ldd, double alpha, double beta, int layout_a,
                                     int layout_b, void* stream)
{
    if(!a || !b || !d || m == 0 || n == 0 || k == 0)
        return B200WMMA_ERR_INVALID_ARG;
    if(beta != 0.0 && !c)
        return B200WMMA_ERR_INVALID_ARG;
    if((layout_a != B200WMMA_ROW_MAJOR && layout_a != B200WMMA_COL_MAJOR)
       || (layout_b != B200WMMA_ROW_MAJOR && layout_b != B200WMMA_COL_MAJOR))
        return B200WMMA_ERR_INVALID_ARG;
    auto s = static_cast<cudaStream_t>(stream);
#define B200WMMA_NOALLOC_CASE(I, O, IT, OT, CT, TM)                                            \
    if(in_dtype == I && out_dtype == O)                                                        \
        return runNoAlloc<IT, OT, CT>(TM, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, beta, \
                                      layout_a, layout_b, s);
    B200WMMA_NOALLOC_CASE(B200WMMA_F16, B200WMMA_F16, __half, __half, float,
                          CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
    B200WMMA_NOALLOC_CASE(B200WMMA_F16, B200WMMA_F32, __half, float, float,
                          CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
    B200WMMA_NOALLOC_CASE(B200WMMA_BF16, B200WMMA_F32, __nv_bfloat16, float, float,
                          CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
    B200WMMA_NOALLOC_CASE(B200WMMA_BF16, B200WMMA_BF16, __nv_bfloat16, __nv_bfloat16, float,
                          CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
    B200WMMA_NOALLOC_CASE(B200WMMA_XF32, B200WMMA_F32, float, float, float,
                          CU_TENSOR_MAP_DATA_TYPE_FLOAT32)
    B200WMMA_NOALLOC_CASE(B200WMMA_I8, B200WMMA_I32, int8_t, int32_t, int32_t,
                          CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_NOALLOC_CASE(B200WMMA_E4M3, B200WMMA_BF16, __nv_fp8_e4m3, __nv_bfloat16, float,
                          CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_NOALLOC_CASE(B200WMMA_E4M3, B200WMMA_F32, __nv_fp8_e4m3, float, float,
                          CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_NOALLOC_CASE(B200WMMA_E5M2, B200WMMA_BF16, __nv_fp8_e5m2, __nv_bfloat16, float,
                          CU_TENSOR_MAP_DATA_TYPE_UINT8)
    B200WMMA_NOALLOC_CASE(B200WMMA_E5M2, B200WMMA_F32, __nv_fp8_e5m2, float, float,
                          CU_TENSOR_MAP_DATA_TYPE_UINT8)
#undef B200WMMA_NOALLOC_CASE
    return B200WMMA_ERR_UNSUPPORTED;
}
