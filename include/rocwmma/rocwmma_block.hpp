// Block-cooperative extension of the fragment API for B200 (sm_100a).
//
// The per-warp API (rocwmma.hpp) keeps accumulators in registers.  Blackwell's
// 5th-generation tensor cores are instead driven per thread block: one thread
// issues tcgen05.mma on operand tiles that the Tensor Memory Accelerator (TMA)
// staged in shared memory, and the accumulator lives in tensor memory (TMEM).
// This header holds the device-side building blocks for kernels of that kind:
// mbarrier pipeline primitives with BOUNDED waits, TMA tile loads, TMEM
// allocation, tcgen05.mma / commit / ld wrappers, and the shared-memory and
// instruction descriptors they take.
//
// It plays the role of the reference's cooperative global->LDS staging
// (rocwmma_coop.hpp, samples/perf_hgemm.cpp:592-685), redone for the hardware.
// No load here uses cluster multicast; the only multicast is the completion signal of
// tcgen05.commit for CTA pairs.
//
// Every wait gives up after a time limit, raises a block-wide abort flag and
// returns false; callers leave their loops, release what they hold and return,
// so that a protocol error surfaces as a status code instead of a hung GPU.
#ifndef ROCWMMA_B200_BLOCK_API_HPP
#define ROCWMMA_B200_BLOCK_API_HPP

#include "internal/config.hpp"
#include "internal/types.hpp"

namespace rocwmma
{
    namespace block
    {
        // ---- addresses ------------------------------------------------------------
        ROCWMMA_DEVICE inline uint32_t smem_addr(void const* p)
        {
            return static_cast<uint32_t>(__cvta_generic_to_shared(p));
        }

        ROCWMMA_DEVICE inline bool elect_one()
        {
            uint32_t pred = 0;
            asm volatile("{\n\t"
                         ".reg .pred P;\n\t"
                         "elect.sync _|P, 0xffffffff;\n\t"
                         "selp.u32 %0, 1, 0, P;\n\t"
                         "}"
                         : "=r"(pred));
            return pred != 0;
        }

        // ---- mbarrier -------------------------------------------------------------
        ROCWMMA_DEVICE inline void mbar_init(uint64_t* bar, uint32_t count)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)),
                         "r"(count)
                         : "memory");
        }
        // Makes freshly initialised barriers visible to the async (TMA / tensor
        // core) proxy.
        ROCWMMA_DEVICE inline void mbar_init_fence()
        {
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        ROCWMMA_DEVICE inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                             smem_addr(bar)),
                         "r"(bytes)
                         : "memory");
        }
        ROCWMMA_DEVICE inline void mbar_arrive(uint64_t* bar)
        {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar))
                         : "memory");
        }
        ROCWMMA_DEVICE inline bool mbar_try_wait(uint64_t* bar, uint32_t parity)
        {
            uint32_t done;
            asm volatile("{\n\t"
                         ".reg .pred P;\n\t"
                         "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, P;\n\t"
                         "}"
                         : "=r"(done)
                         : "r"(smem_addr(bar)), "r"(parity)
                         : "memory");
            return done != 0;
        }

        // Non-blocking form: reports whether the phase has completed and returns at once
        // (mbarrier.try_wait may suspend the thread for a system-dependent time, microseconds,
        // when it has not).  For polls whose outcome is only looked at later.
        ROCWMMA_DEVICE inline bool mbar_test_wait(uint64_t* bar, uint32_t parity)
        {
            uint32_t done;
            asm volatile("{\n\t"
                         ".reg .pred P;\n\t"
                         "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, P;\n\t"
                         "}"
                         : "=r"(done)
                         : "r"(smem_addr(bar)), "r"(parity)
                         : "memory");
            return done != 0;
        }

        // Codes recorded next to the abort flag: which kind of wait ran out.
        enum WaitCode : uint32_t
        {
            WAIT_STAGE_EMPTY = 1, // loader waiting for the MMA to release a ring slot
            WAIT_STAGE_FULL  = 2, // MMA issuer waiting for TMA data
            WAIT_ACC_EMPTY   = 3, // MMA issuer waiting for the epilogue to drain TMEM
            WAIT_ACC_FULL    = 4, // epilogue waiting for the MMAs of a tile
            WAIT_DRAIN       = 5, // leaving: waiting for own TMA copies still in flight
            WAIT_PEER        = 6  // CTA-pair handshake
        };

        // Block-wide abort state in shared memory.
        struct AbortState
        {
            volatile uint32_t flag;
            volatile uint32_t code;
        };

        // ~2 s at B200 clocks; a healthy pipeline wait lasts microseconds.
        constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;

        // Waits until the phase with the given parity of `bar` has completed.
        // Returns false if the block is aborting or the time limit passed (in which
        // case it raises the abort flag itself).
        ROCWMMA_DEVICE inline bool
            mbar_wait(uint64_t* bar, uint32_t parity, AbortState* abort, uint32_t code,
                      long long limit = WAIT_LIMIT_CYCLES)
        {
            if(mbar_try_wait(bar, parity))
                return true;
            const long long start = clock64();
            uint32_t        spins = 0;
            while(true)
            {
                if(mbar_try_wait(bar, parity))
                    return true;
                if((++spins & 63u) == 0u)
                {
                    if(abort->flag != 0u)
                        return false;
                    if(clock64() - start > limit)
                    {
                        abort->code = code;
                        abort->flag = 1u;
                        __threadfence_block();
                        return false;
                    }
                }
            }
        }

        // ---- TMA (cp.async.bulk.tensor), no multicast --------------------------------
        ROCWMMA_DEVICE inline void tma_prefetch_descriptor(void const* tensorMap)
        {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensorMap))
                         : "memory");
        }
        // Asks for the 128-byte line that holds `addr` to be brought into L2 (no register
        // result, nothing to wait for).
        ROCWMMA_DEVICE inline void prefetch_l2(void const* addr)
        {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(addr) : "memory");
        }
        // Asks for the box at (x, y) of `tensorMap` to be brought into L2 (no shared-memory
        // destination, no completion to wait for).  Same alignment rule for x as a load.
        ROCWMMA_DEVICE inline void tma_prefetch_l2_2d(void const* tensorMap, int32_t x, int32_t y)
        {
            asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(
                             reinterpret_cast<uint64_t>(tensorMap)),
                         "r"(x), "r"(y)
                         : "memory");
        }
        // Loads the box of `tensorMap` whose innermost coordinate is x (elements;
        // x * element size must be a multiple of 16 bytes) and outer coordinate y
        // into shared memory at dst, signalling `bar` with the byte count.
        ROCWMMA_DEVICE inline void tma_load_2d(void* dst, void const* tensorMap, uint64_t* bar,
                                               int32_t x, int32_t y)
        {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                         " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_addr(dst)),
                         "l"(reinterpret_cast<uint64_t>(tensorMap)), "r"(smem_addr(bar)), "r"(x),
                         "r"(y)
                         : "memory");
        }

        // One-dimensional form: the box starting at element x (x * element size a multiple of
        // 16 bytes).
        ROCWMMA_DEVICE inline void tma_load_1d(void* dst, void const* tensorMap, uint64_t* bar,
                                               int32_t x)
        {
            asm volatile("cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes"
                         " [%0], [%1, {%3}], [%2];" ::"r"(smem_addr(dst)),
                         "l"(reinterpret_cast<uint64_t>(tensorMap)), "r"(smem_addr(bar)), "r"(x)
                         : "memory");
        }

        // ---- untiled bulk copies (cp.async.bulk): contiguous bytes, no tensor map ----------
        // Both addresses 16-byte aligned, `bytes` a multiple of 16.
        // Global -> this block's shared memory; `bar` receives complete_tx(bytes).
        ROCWMMA_DEVICE inline void bulk_load(uint32_t dstSmemAddr, void const* src, uint32_t bytes,
                                             uint32_t barSmemAddr)
        {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes"
                         " [%0], [%1], %2, [%3];" ::"r"(dstSmemAddr),
                         "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(barSmemAddr)
                         : "memory");
        }
        // Shared -> global, completion tracked by the issuing thread's bulk groups
        // (tma_store_commit / tma_store_wait_read / tma_store_wait_all below).
        ROCWMMA_DEVICE inline void bulk_store(void* dst, uint32_t srcSmemAddr, uint32_t bytes)
        {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                             reinterpret_cast<uint64_t>(dst)),
                         "r"(srcSmemAddr), "r"(bytes)
                         : "memory");
        }
        // One arrival on `bar` that also announces `bytes` of complete_tx still to come
        // (bytes may be 0).  Address form of mbar_expect_tx.
        ROCWMMA_DEVICE inline void mbar_arrive_expect_tx(uint32_t barSmemAddr, uint32_t bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barSmemAddr),
                         "r"(bytes)
                         : "memory");
        }

        // ---- TMA stores (shared -> global), bulk-group completion ----------------------------
        // Generic-proxy writes to shared memory must be fenced before the async proxy reads them.
        ROCWMMA_DEVICE inline void fence_async_shared()
        {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        // Writes the box at (x, y) of `tensorMap` from shared memory; parts of the box outside
        // the tensor are dropped.  x * element size must be a multiple of 16 bytes, x, y >= 0.
        ROCWMMA_DEVICE inline void tma_store_2d(void const* tensorMap, void const* src, int32_t x,
                                                int32_t y)
        {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::
                             "l"(reinterpret_cast<uint64_t>(tensorMap)),
                         "r"(smem_addr(src)), "r"(x), "r"(y)
                         : "memory");
        }
        // tma_store_2d with an L2 cache hint (a policy from l2_policy_evict_first / _last).
        ROCWMMA_DEVICE inline void tma_store_2d_hint(void const* tensorMap, void const* src,
                                                     int32_t x, int32_t y, uint64_t policy)
        {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint"
                         " [%0, {%2, %3}], [%1], %4;" ::"l"(reinterpret_cast<uint64_t>(tensorMap)),
                         "r"(smem_addr(src)), "r"(x), "r"(y), "l"(policy)
                         : "memory");
        }
        // Same, but adds the box to global memory (element type of the tensor map; the adds
        // are performed by the L2, round to nearest for fp32).
        ROCWMMA_DEVICE inline void tma_reduce_add_2d(void const* tensorMap, void const* src,
                                                     int32_t x, int32_t y)
        {
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::
                             "l"(reinterpret_cast<uint64_t>(tensorMap)),
                         "r"(smem_addr(src)), "r"(x), "r"(y)
                         : "memory");
        }
        ROCWMMA_DEVICE inline void tma_store_commit()
        {
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        // Waits until at most N of this thread's bulk groups have not yet READ their shared
        // memory source (the source may then be overwritten).
        template <int N>
        ROCWMMA_DEVICE inline void tma_store_wait_read()
        {
            asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
        }
        // Waits until at most N of this thread's bulk groups are still incomplete (their global
        // writes performed).
        template <int N>
        ROCWMMA_DEVICE inline void tma_store_wait_all()
        {
            asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
        }
        // Barrier among `count` threads that also ANDs a predicate over them: every
        // participant gets true only if all passed true.
        ROCWMMA_DEVICE inline bool named_barrier_all(uint32_t id, uint32_t count, bool pred)
        {
            uint32_t r;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %3, 0;\n\t"
                         "bar.red.and.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(r)
                         : "r"(id), "r"(count), "r"(uint32_t(pred))
                         : "memory");
            return r != 0u;
        }
        // Barrier among `count` threads of the block (id 1..15; 0 is __syncthreads).
        ROCWMMA_DEVICE inline void named_barrier(uint32_t id, uint32_t count)
        {
            asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
        }

        // ---- tensor memory ----------------------------------------------------------
        // One full warp allocates `columns` (power of two, 32..512) TMEM columns; the
        // base address is written to *slot in shared memory.
        ROCWMMA_DEVICE inline void tmem_alloc(uint32_t* slot, uint32_t columns)
        {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_addr(slot)),
                         "r"(columns)
                         : "memory");
        }
        ROCWMMA_DEVICE inline void tmem_relinquish_alloc_permit()
        {
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        ROCWMMA_DEVICE inline void tmem_dealloc(uint32_t base, uint32_t columns)
        {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base),
                         "r"(columns)
                         : "memory");
        }
        ROCWMMA_DEVICE inline void tc_fence_before_sync()
        {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        ROCWMMA_DEVICE inline void tc_fence_after_sync()
        {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }

        // ---- descriptors -------------------------------------------------------------
        // Shared-memory matrix descriptor for a K-major operand tile written by TMA
        // with the 128-byte swizzle: rows are 128 bytes wide, groups of 8 rows are
        // 1024 bytes apart.  `addr` is the shared-memory byte address of the tile (or
        // of a 32-byte K step inside its first row); the tile base must be
        // 1024-byte aligned.
        ROCWMMA_DEVICE inline uint64_t smem_desc_kmajor_sw128(uint32_t addr)
        {
            uint64_t d = 0;
            d |= uint64_t((addr & 0x3ffffu) >> 4); // start address, 16-byte units
            d |= uint64_t(1) << 16; // leading-dimension byte offset (unused with swizzle)
            d |= uint64_t(1024u >> 4) << 32; // stride between 8-row groups
            d |= uint64_t(1) << 46; // descriptor version for sm_100
            d |= uint64_t(2) << 61; // layout: 128-byte swizzle
            return d;
        }

        // Descriptor for an MN-major operand tile (the M or N index is contiguous in memory:
        // a column-major A or a row-major B) written by TMA with the 128-byte swizzle as
        // blocks of [K rows][128 bytes of M/N]: 8 K rows form a 1024-byte group, consecutive
        // groups follow each other, and `mnAtomStride` bytes separate the blocks that hold
        // the next 128 bytes of M/N.  `addr` is the tile base plus the K groups already
        // consumed.
        ROCWMMA_DEVICE inline uint64_t smem_desc_mnmajor_sw128(uint32_t addr, uint32_t mnAtomStride)
        {
            uint64_t d = 0;
            d |= uint64_t((addr & 0x3ffffu) >> 4);
            d |= uint64_t((mnAtomStride >> 4) & 0x3fffu) << 16; // leading-dimension byte offset
            d |= uint64_t(1024u >> 4) << 32; // stride between 8-row K groups
            d |= uint64_t(1) << 46;
            d |= uint64_t(2) << 61;
            return d;
        }

        enum class MmaKind : uint32_t
        {
            F16, // fp16 or bf16 inputs, fp32 accumulate
            TF32,
            I8,
            F8F6F4
        };
        // Operand format codes of the instruction descriptor.
        constexpr uint32_t FMT_F16 = 0, FMT_BF16 = 1, FMT_TF32 = 2;
        constexpr uint32_t FMT_E4M3 = 0, FMT_E5M2 = 1;
        constexpr uint32_t FMT_U8 = 0, FMT_S8 = 1;
        constexpr uint32_t ACC_F16 = 0, ACC_F32 = 1, ACC_S32 = 2;

        // 32-bit instruction descriptor: accumulator format, A/B formats, operand majors
        // (0 = K-major, 1 = MN-major), tile M x N.
        ROCWMMA_HOST_DEVICE constexpr uint32_t
            make_instr_desc(uint32_t accFmt, uint32_t aFmt, uint32_t bFmt, uint32_t m, uint32_t n,
                            uint32_t aMnMajor = 0, uint32_t bMnMajor = 0)
        {
            return (accFmt << 4) | (aFmt << 7) | (bFmt << 10) | (aMnMajor << 15)
                   | (bMnMajor << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
        }

        // D[tmem] (+)= A[smem] * B[smem].  Issued by ONE thread.
        template <MmaKind Kind>
        ROCWMMA_DEVICE inline void mma_ss(uint32_t dTmem, uint64_t descA, uint64_t descB,
                                          uint32_t idesc, uint32_t accumulate)
        {
            if constexpr(Kind == MmaKind::F16)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
            else if constexpr(Kind == MmaKind::TF32)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
            else if constexpr(Kind == MmaKind::I8)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
            else
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
        }

        // Makes `bar` complete one arrival when all tcgen05.mma issued so far by this
        // thread have finished (implies tcgen05.fence::before_thread_sync).
        ROCWMMA_DEVICE inline void mma_commit(uint64_t* bar)
        {
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                             "r"(smem_addr(bar))
                         : "memory");
        }

        // =============================================================================
        // CTA pairs (cta_group::2): two thread blocks of a cluster, on the two SMs of
        // one TPC, drive ONE tcgen05.mma of M = 256.  Each block stages its own 128
        // rows of A and its own half of the B tile (plain TMA loads into its own
        // shared memory -- no multicast), the even block of the pair issues the MMA,
        // and each block's tensor core writes its 128 accumulator rows to its own TMEM.
        // =============================================================================
        ROCWMMA_DEVICE inline uint32_t cluster_cta_rank()
        {
            uint32_t r;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
            return r;
        }
        // Shared-memory address of the same variable in block `rank` of the cluster.
        ROCWMMA_DEVICE inline uint32_t map_to_cta(uint32_t smemAddr, uint32_t rank)
        {
            uint32_t r;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
            return r;
        }
        ROCWMMA_DEVICE inline void cluster_sync()
        {
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
        // The two halves of a cluster barrier, to be used as a pair with independent work in
        // between.  The arrival orders nothing by itself: what the other block must see
        // (freshly initialised mbarriers) has to be released before it, as mbar_init_fence()
        // does.  Every thread of the block executes both, warps converged.
        ROCWMMA_DEVICE inline void cluster_arrive_relaxed()
        {
            asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        }
        ROCWMMA_DEVICE inline void cluster_wait()
        {
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
        // Programmatic dependent launch.  A kernel launched with the stream-serialization
        // attribute may start while the previous kernel of its stream still runs;
        // grid_dependency_wait() returns once that kernel has completed and its writes are
        // visible (at once if there is no such kernel or the attribute was not given).
        // grid_launch_dependents() lets the next kernel of the stream be scheduled when every
        // block of this grid has called it or exited.
        ROCWMMA_DEVICE inline void grid_dependency_wait()
        {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        }
        ROCWMMA_DEVICE inline void grid_launch_dependents()
        {
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
        // Arrive on an mbarrier that may live in the other block of the pair
        // (`clusterAddr` from map_to_cta).
        ROCWMMA_DEVICE inline void mbar_arrive_cluster(uint32_t clusterAddr)
        {
            asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                             clusterAddr)
                         : "memory");
        }
        // TMA tile load issued by either block of a pair: data lands in the issuing
        // block's shared memory, the byte count is signalled on `barClusterAddr`, which
        // may be the pair leader's barrier.
        ROCWMMA_DEVICE inline void tma_load_2d_pair(void* dst, void const* tensorMap,
                                                    uint32_t barClusterAddr, int32_t x, int32_t y)
        {
            asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global"
                         ".mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                             smem_addr(dst)),
                         "l"(reinterpret_cast<uint64_t>(tensorMap)), "r"(barClusterAddr), "r"(x),
                         "r"(y)
                         : "memory");
        }
        ROCWMMA_DEVICE inline void tmem_alloc_pair(uint32_t* slot, uint32_t columns)
        {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_addr(slot)),
                         "r"(columns)
                         : "memory");
        }
        ROCWMMA_DEVICE inline void tmem_relinquish_alloc_permit_pair()
        {
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        }
        ROCWMMA_DEVICE inline void tmem_dealloc_pair(uint32_t base, uint32_t columns)
        {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base),
                         "r"(columns)
                         : "memory");
        }
        // Pair MMA (M = 256 over both blocks).  Issued by ONE thread of the even block.
        template <MmaKind Kind>
        ROCWMMA_DEVICE inline void mma_ss_pair(uint32_t dTmem, uint64_t descA, uint64_t descB,
                                               uint32_t idesc, uint32_t accumulate)
        {
            if constexpr(Kind == MmaKind::F16)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
            else if constexpr(Kind == MmaKind::TF32)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
            else if constexpr(Kind == MmaKind::I8)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
            else
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(
                                 dTmem),
                             "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                             : "memory");
        }
        // L2 eviction policies for loads that carry a cache hint: lines fetched with
        // `evict_last` are kept in preference to others (an operand many blocks come back to),
        // lines fetched with `evict_first` are the first to go (an operand that streams past).
        ROCWMMA_DEVICE inline uint64_t l2_policy_evict_last()
        {
            uint64_t p;
            asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
            return p;
        }
        ROCWMMA_DEVICE inline uint64_t l2_policy_evict_first()
        {
            uint64_t p;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
            return p;
        }
        // tma_load_2d with an L2 cache hint (a policy from the functions above).
        ROCWMMA_DEVICE inline void tma_load_2d_hint(void* dst, void const* tensorMap, uint64_t* bar,
                                                    int32_t x, int32_t y, uint64_t policy)
        {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                         ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_addr(dst)),
                         "l"(reinterpret_cast<uint64_t>(tensorMap)), "r"(smem_addr(bar)), "r"(x),
                         "r"(y), "l"(policy)
                         : "memory");
        }
        // tma_load_2d_pair with an L2 cache hint (a policy from the functions above).
        ROCWMMA_DEVICE inline void tma_load_2d_pair_hint(void* dst, void const* tensorMap,
                                                         uint32_t barClusterAddr, int32_t x,
                                                         int32_t y, uint64_t policy)
        {
            asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global"
                         ".mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(
                             smem_addr(dst)),
                         "l"(reinterpret_cast<uint64_t>(tensorMap)), "r"(barClusterAddr), "r"(x),
                         "r"(y), "l"(policy)
                         : "memory");
        }
        // Completion of all pair MMAs issued so far arrives (one count) on the barrier at
        // the same shared-memory offset in every block named in ctaMask.
        ROCWMMA_DEVICE inline void mma_commit_pair(uint64_t* bar, uint16_t ctaMask)
        {
            // clang-format off
            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                         :: "r"(smem_addr(bar)), "h"(ctaMask) : "memory");
            // clang-format on
        }

        // Reads 32 consecutive 32-bit columns of this thread's TMEM lane
        // (lane = 32 * (warp % 4) + laneid).  Warp-wide.
        ROCWMMA_DEVICE inline void tmem_load_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
        {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
                "[%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                  "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                  "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
                  "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                  "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                  "=r"(r[30]), "=r"(r[31])
                : "r"(taddr)
                : "memory");
        }
        // Same for 16 columns.
        ROCWMMA_DEVICE inline void tmem_load_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
        {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                  "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                  "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
        }
        ROCWMMA_DEVICE inline void tmem_load_wait()
        {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
        // Writes 32 consecutive 32-bit columns of this thread's TMEM lane.  Warp-wide.
        ROCWMMA_DEVICE inline void tmem_store_32x32b_x32(uint32_t taddr, uint32_t const (&r)[32])
        {
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                :
                : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
                  "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
                  "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
                  "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
                  "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
                  "r"(r[31])
                : "memory");
        }
        ROCWMMA_DEVICE inline void tmem_store_wait()
        {
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
    } // namespace block
} // namespace rocwmma

#endif // ROCWMMA_B200_BLOCK_API_HPP
