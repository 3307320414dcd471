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
//   * a block owns 64 consecutive rows (32 when the matrix has so few rows that 64-row
//     blocks would leave most SMs idle: a row shard of a many-GPU run); one producer thread
//     streams ROWS-row x 32-column tiles of A through a shared-memory ring (12 slots of
//     8 KiB, or 24 of 4 KiB) with one TMA tile load each, full/empty mbarriers per slot; the
//     32 values of x that belong to a tile travel in the same slot (a second, one-dimensional
//     TMA load), so that no compute thread ever waits on a global load (with x read straight
//     from global memory the kernel was bound by that latency, 3.8 TB/s).  (The first form of
//     this loader, four warps issuing 16-byte cp.async copies, held a block to ~25 GB/s
//     whatever the grid: the SM tracks only so many outstanding load sectors, and 80 KiB in
//     flight needed far more.  One TMA request moves a whole tile.)
//   * one compute thread per row reads its row's element of each column from the slot
//     (consecutive threads, consecutive addresses) and x[h] by warp-uniform vector loads;
//     its loop is software-pipelined three tiles deep (see the compute branch), so that the
//     only thing on the critical path is the chain of dependent additions the ordered sum
//     consists of: 4 cycles per column, ~35 us for 16384 columns whatever the row count;
//   * 2 blocks per SM, 80 KiB of loads in flight per block.
//
// When A, x or the leading dimension are not 16-byte multiples (TMA cannot address them) a
// plain-load kernel with the same summation order is used.
#include "common.cuh"
#include "runtime.cuh"
#include <cuda.h>
#include <rocwmma/rocwmma_block.hpp>

using namespace rocwmma::block;

namespace
{
    constexpr uint32_t COLS_BYTES = 128; // the columns of a tile: 128 bytes of x (32 fp32, 16 fp64)
    constexpr uint32_t LTHREADS   = 32; // the producer warp (one elected thread issues)

    // Geometry of one instantiation: ROWS rows per block (one compute thread per row), STAGES
    // ring slots of one tile (ROWS rows x 128 bytes' worth of columns) plus its x values.
    template <typename T, uint32_t ROWS_, uint32_t STAGES_>
    struct Geometry
    {
        static constexpr uint32_t ROWS       = ROWS_;
        static constexpr uint32_t STAGES     = STAGES_;
        static constexpr uint32_t COLS       = COLS_BYTES / sizeof(T);
        static constexpr uint32_t TILE_BYTES = ROWS * COLS * sizeof(T);
        static constexpr uint32_t XSEG_BYTES = COLS_BYTES;
        static constexpr uint32_t SLOT_BYTES = TILE_BYTES + XSEG_BYTES;
        static constexpr uint32_t THREADS    = ROWS + LTHREADS;
        struct Control
        {
            uint64_t   full[STAGES];
            uint64_t   empty[STAGES];
            AbortState abort;
        };
        static constexpr uint32_t SMEM_BYTES
            = STAGES * SLOT_BYTES + 128 /*alignment slack*/ + sizeof(Control);
    };

    __device__ inline float  mulRn(float a, float b) { return __fmul_rn(a, b); }
    __device__ inline double mulRn(double a, double b) { return __dmul_rn(a, b); }
    __device__ inline float  addRn(float a, float b) { return __fadd_rn(a, b); }
    __device__ inline double addRn(double a, double b) { return __dadd_rn(a, b); }

    template <typename T, uint32_t N>
    struct alignas(sizeof(T) * N) Vec
    {
        T v[N];
    };

    template <typename T, uint32_t ROWS, uint32_t STAGES>
    __global__ void __launch_bounds__(ROWS + LTHREADS, 2)
        gemvStreamKernel(const __grid_constant__ CUtensorMap tmapA,
                         const __grid_constant__ CUtensorMap tmapX, uint32_t m, uint32_t k,
                         T const* yIn, T* yOut, T alpha, T beta, uint32_t* status)
    {
        using G = Geometry<T, ROWS, STAGES>;
        using Control = typename G::Control;
        constexpr uint32_t COLS       = G::COLS; // 32 (fp32) / 16 (fp64)
        constexpr uint32_t TILE_BYTES = G::TILE_BYTES;
        constexpr uint32_t SLOT_BYTES = G::SLOT_BYTES;
        constexpr uint32_t XV         = 16 / sizeof(T);
        extern __shared__ uint8_t smemRaw[];
        const uint32_t            raw   = smem_addr(smemRaw);
        uint8_t*                  tiles = smemRaw + ((128u - (raw & 127u)) & 127u);
        Control* ctl = reinterpret_cast<Control*>(tiles + STAGES * SLOT_BYTES);

        const uint32_t row0  = blockIdx.x * ROWS;
        const uint32_t numKB = (k + COLS - 1) / COLS;

        if(threadIdx.x == 0)
        {
            for(uint32_t s = 0; s < STAGES; ++s)
            {
                mbar_init(&ctl->full[s], 1);
                mbar_init(&ctl->empty[s], ROWS); // every compute thread arrives for itself
            }
            ctl->abort.flag = 0;
            ctl->abort.code = 0;
            mbar_init_fence();
            tma_prefetch_descriptor(&tmapA);
            tma_prefetch_descriptor(&tmapX);
        }
        __syncthreads();
        // the barriers are set up while the previous kernel of the stream drains; A, x and y
        // may be its output
        grid_dependency_wait();
        grid_launch_dependents();

        if(threadIdx.x >= ROWS)
        {
            // ---- producer: one thread, two TMA loads per tile ----
            // Rows beyond m and columns beyond k are filled with zeros by the TMA (and still
            // counted in the bytes the barrier expects).
            if(elect_one())
            {
                uint32_t kb = 0;
                for(; kb < numKB; ++kb)
                {
                    const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                    if(!mbar_wait(&ctl->empty[s], ph ^ 1u, &ctl->abort, WAIT_STAGE_EMPTY))
                        break;
                    uint8_t* slot = tiles + s * SLOT_BYTES;
                    mbar_expect_tx(&ctl->full[s], SLOT_BYTES);
                    tma_load_2d(slot, &tmapA, &ctl->full[s], int32_t(row0), int32_t(kb * COLS));
                    tma_load_1d(slot + TILE_BYTES, &tmapX, &ctl->full[s], int32_t(kb * COLS));
                }
                if(kb < numKB)
                {
                    // Leaving early: give copies already issued a bounded time to land before
                    // the block's shared memory is released.
                    const uint32_t pending = kb < STAGES ? kb : STAGES;
                    for(uint32_t j = 0; j < pending; ++j)
                    {
                        const uint32_t prev = kb - 1 - j;
                        const long long start = clock64();
                        while(!mbar_try_wait(&ctl->full[prev % STAGES], (prev / STAGES) & 1u)
                              && clock64() - start < 2000000ll)
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
            // x values of tile kb (from the slot)
            auto xValues = [&](uint32_t kb, T (&xv)[COLS]) {
                const uint32_t    s = kb % STAGES;
                Vec<T, XV> const* xs
                    = reinterpret_cast<Vec<T, XV> const*>(tiles + s * SLOT_BYTES + TILE_BYTES);
#pragma unroll
                for(uint32_t j = 0; j < COLS; j += XV)
                {
                    const Vec<T, XV> q = xs[j / XV]; // same address in every lane: broadcast
#pragma unroll
                    for(uint32_t e = 0; e < XV; ++e)
                        xv[j + e] = q.v[e];
                }
            };
            if constexpr(sizeof(T) == 4)
            {
                // The ordered sum is a chain of dependent additions, 4 cycles each: 128 cycles
                // per tile that nothing can shorten.  Everything else a tile needs -- 32
                // shared-memory loads of A, 8 of x, 32 multiplications, a barrier poll and a
                // barrier arrival -- is taken off that chain by working on three tiles at
                // once: while the products of tile t are added, the values of tile t + 1
                // (already in registers) are multiplied and tile t + 2 is polled for and
                // loaded.  A warp issues in order, so what matters is where each result is
                // first USED: the poll of tile t + 2 is issued before the chain and its outcome
                // tested after it, the loaded values are first touched one step later.  Written
                // as one unrolled loop body, additions and multiplications interleave.
                // (Fetching a whole tile and then adding it cost ~550 cycles per tile, most of
                // them latency of the barrier poll and its dependent branch, not arithmetic: a
                // block streamed at 25 GB/s whatever the grid, and a 2048-row shard took as
                // long as the whole matrix.)
                // A slot goes back to the producer once its values have been multiplied.
                // The last tile may be partial: its columns beyond k must not enter the sum
                // (adding +0 could turn a -0 into +0), so it takes a guarded path of its own.
                const uint32_t numFull = k / COLS; // tiles made of COLS valid columns
                bool           ok      = true;
                // Ring positions are carried along instead of being derived from the tile
                // number each time (a division by a slot count that is no power of two is a
                // chain of dependent integer operations, and this warp issues in order).
                struct RingPos
                {
                    uint32_t slot, phase;
                    __device__ void advance()
                    {
                        if(++slot == STAGES)
                        {
                            slot = 0;
                            phase ^= 1u;
                        }
                    }
                };
                RingPos toLoad{0u, 0u}, toRelease{0u, 0u};
                // raw values of the tile in slot `s` (A and x) -> registers
                auto loadTile = [&](uint32_t s, T (&av)[COLS], T (&xv)[COLS]) {
                    T const*          tile = reinterpret_cast<T const*>(tiles + s * SLOT_BYTES);
                    Vec<T, XV> const* xs   = reinterpret_cast<Vec<T, XV> const*>(
                        tiles + s * SLOT_BYTES + TILE_BYTES);
#pragma unroll
                    for(uint32_t j = 0; j < COLS; j += XV)
                    {
                        const Vec<T, XV> q = xs[j / XV]; // same address in every lane: broadcast
#pragma unroll
                        for(uint32_t e = 0; e < XV; ++e)
                            xv[j + e] = q.v[e];
                    }
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        av[j] = tile[j * ROWS + r];
                };
                // Every lane arrives for itself (the barrier counts ROWS arrivals): a lane's
                // arrival follows its own reads of the slot in program order, so no warp-wide
                // synchronisation -- another instruction with a branch's latency -- is needed.
                auto releaseSlot = [&]() {
                    mbar_arrive(&ctl->empty[toRelease.slot]);
                    toRelease.advance();
                };
                // One steady-state step for tile t: adds the products `pCur` of tile t;
                // multiplies the raw values of tile t + 1 into `pNext` and releases that tile's
                // slot; loads tile t + 2 into `aNew`, `xNew`; polls for a tile four further on.
                // The loads and the poll sit inside the unrolled loop, between additions, so that
                // their issue slots and latencies fall into the gaps of the 4-cycle chain; what
                // they return is first used one step (the poll: one trip of four steps) later.
                // Branches are what a lone warp cannot hide (~40 cycles each, measured), so a
                // step has none: arrival of the four tiles a trip loads is established once,
                // before the trip, from the polls of the trip before.
                RingPos toPoll{0u, 0u};
                auto    step = [&](T const (&pCur)[COLS], T (&pNext)[COLS], T const (&aNext)[COLS],
                                T const (&xNext)[COLS], T (&aNew)[COLS], T (&xNew)[COLS],
                                bool& allArrived) {
                    T const*          tile = reinterpret_cast<T const*>(tiles + toLoad.slot * SLOT_BYTES);
                    Vec<T, XV> const* xs   = reinterpret_cast<Vec<T, XV> const*>(
                        tiles + toLoad.slot * SLOT_BYTES + TILE_BYTES);
                    toLoad.advance();
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                    {
                        acc      = addRn(acc, pCur[j]);
                        pNext[j] = mulRn(aNext[j], xNext[j]);
                        aNew[j]  = tile[j * ROWS + r];
                        if(j % XV == 0u)
                        {
                            const Vec<T, XV> q = xs[j / XV];
#pragma unroll
                            for(uint32_t e = 0; e < XV; ++e)
                                xNew[j + e] = q.v[e];
                        }
                        if(j == COLS / 4u)
                            allArrived
                                = mbar_try_wait(&ctl->full[toPoll.slot], toPoll.phase) && allArrived;
                    }
                    toPoll.advance();
                    releaseSlot(); // tile t + 1: its values have been multiplied
                };
                T pA[COLS], pB[COLS], rA[COLS], rB[COLS], xA[COLS], xB[COLS];
                if(numFull > 0u)
                {
                    // prologue: tile 0 loaded and multiplied, tile 1 loaded
                    ok = mbar_wait(&ctl->full[0], 0u, &ctl->abort, WAIT_STAGE_FULL);
                    if(ok)
                    {
                        loadTile(0u, rA, xA);
                        toLoad.advance();
#pragma unroll
                        for(uint32_t j = 0; j < COLS; ++j)
                            pA[j] = mulRn(rA[j], xA[j]);
                        releaseSlot();
                        if(numFull > 1u)
                        {
                            ok = mbar_wait(&ctl->full[1], 0u, &ctl->abort, WAIT_STAGE_FULL);
                            if(ok)
                            {
                                loadTile(1u, rB, xB);
                                toLoad.advance();
                            }
                        }
                    }
                    // steady state, four tiles per trip (the register sets swap roles).  A trip
                    // starting at tile t loads tiles t + 2 .. t + 5 and polls t + 6 .. t + 9.
                    uint32_t t = 0;
                    toPoll     = toLoad;
                    for(uint32_t i = 0; i < 4u; ++i)
                        toPoll.advance();
                    bool arrivedAll = false;
                    for(; ok && t + 9 < numFull; t += 4)
                    {
                        if(!arrivedAll)
                        {
                            // first trip, or a poll came back early: wait for the four tiles
                            RingPos w = toLoad;
                            for(uint32_t i = 0; ok && i < 4u; ++i)
                            {
                                ok = mbar_wait(&ctl->full[w.slot], w.phase, &ctl->abort,
                                               WAIT_STAGE_FULL);
                                w.advance();
                            }
                            if(!ok)
                                break;
                        }
                        bool all = true;
                        step(pA, pB, rB, xB, rA, xA, all);
                        step(pB, pA, rA, xA, rB, xB, all);
                        step(pA, pB, rB, xB, rA, xA, all);
                        step(pB, pA, rA, xA, rB, xB, all);
                        arrivedAll = all;
                    }
                    // The last full tiles, one simple step each: add tile u; multiply tile u + 1
                    // if there is one; wait for and load tile u + 2 if there is one.  (t is
                    // even here; toLoad names tile t + 2.)
                    for(uint32_t u = t; ok && u < numFull; ++u)
                    {
                        const bool even = ((u & 1u) == 0u);
                        T const(&pCur)[COLS]  = even ? pA : pB;
                        T(&pNext)[COLS]       = even ? pB : pA;
                        T(&aNext)[COLS]       = even ? rB : rA;
                        T(&xNext)[COLS]       = even ? xB : xA;
                        T(&aNew)[COLS]        = even ? rA : rB;
                        T(&xNew)[COLS]        = even ? xA : xB;
                        const bool has1 = u + 1 < numFull, has2 = u + 2 < numFull;
#pragma unroll
                        for(uint32_t j = 0; j < COLS; ++j)
                        {
                            acc = addRn(acc, pCur[j]);
                            if(has1)
                                pNext[j] = mulRn(aNext[j], xNext[j]);
                        }
                        if(has1)
                            releaseSlot();
                        if(has2)
                        {
                            ok = mbar_wait(&ctl->full[toLoad.slot], toLoad.phase, &ctl->abort,
                                           WAIT_STAGE_FULL);
                            if(ok)
                            {
                                loadTile(toLoad.slot, aNew, xNew);
                                toLoad.advance();
                            }
                        }
                    }
                }
                if(ok && numFull < numKB)
                {
                    // the partial last tile (toLoad names its slot: it follows the full ones)
                    const uint32_t valid = k - numFull * COLS;
                    T              av[COLS], xv[COLS];
                    if(mbar_wait(&ctl->full[toLoad.slot], toLoad.phase, &ctl->abort,
                                 WAIT_STAGE_FULL))
                    {
                        loadTile(toLoad.slot, av, xv);
#pragma unroll
                        for(uint32_t j = 0; j < COLS; ++j)
                            if(j < valid)
                                acc = addRn(acc, mulRn(av[j], xv[j]));
                        releaseSlot();
                    }
                }
            }
            else
            {
                // 64-bit elements: one tile at a time (a second register set would not fit)
                T av[COLS], xv[COLS];
                for(uint32_t kb = 0; kb < numKB; ++kb)
                {
                    const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                    if(!mbar_wait(&ctl->full[s], ph, &ctl->abort, WAIT_STAGE_FULL))
                        break;
                    xValues(kb, xv);
                    T const* tile = reinterpret_cast<T const*>(tiles + s * SLOT_BYTES);
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        av[j] = tile[j * ROWS + r];
                    const uint32_t h0    = kb * COLS;
                    const uint32_t valid = (k - h0) < COLS ? (k - h0) : COLS;
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        if(j < valid)
                            acc = addRn(acc, mulRn(av[j], xv[j]));
                    mbar_arrive(&ctl->empty[s]);
                }
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

    // ---- fp32 with the multiplications taken off the adding warp ------------------------------
    // The floor of a bit-identical row sum is its chain of k dependent additions: 44 us for
    // k = 16384 measured on the bare chain, 58 us with one shared-memory load per addend
    // issued between the additions.  Here the work of a 32-row group is spread over five warps:
    //   * four multiplier warps take the tiles of the ring in turn; a thread reads its row's
    //     32 values of A and the tile's 32 values of x, multiplies (rounded, as the host
    //     routine does) and writes the 32 products of its row side by side into the slot's
    //     product area (rows 144 bytes apart, so that the 16-byte accesses of a warp spread
    //     over all banks), then arrives on the slot's `prod` barrier;
    //   * the chain warp waits for `prod`, reads its row's 32 products with eight 16-byte loads
    //     and adds them in column order -- the loads of tile t + 1 and the poll for a later
    //     tile issued between the additions of tile t -- and hands the slot back to the
    //     producer.
    // Block = ROWS / 32 chain warps, four times as many multiplier warps, one producer warp.
    // The chain warp's issue slots are what the launch time hangs on: a micro-benchmark of the
    // bare chain takes 44.5 us for k = 16384, 57.2 us with one 4-byte shared-memory load per
    // addend between the additions and 50.6 us with one 16-byte load per four addends -- hence
    // the row-wise product area -- and with one 32-row group per block the chain warp shares
    // its scheduler with the producer warp, which sleeps, not with a multiplier warp.
    // (The polls use mbarrier.try_wait on purpose: when a tile has not arrived it suspends the
    // warp for a while instead of returning at once, and the non-blocking test_wait in its
    // place made the single-warp form 20 % slower.)
    template <uint32_t ROWS, uint32_t STAGES>
    struct ChainGeometry
    {
        static constexpr uint32_t COLS       = 32;
        static constexpr uint32_t TILE_BYTES = ROWS * COLS * 4;
        static constexpr uint32_t PROD_STRIDE = COLS + 4; // floats between rows of products
        static constexpr uint32_t PROD_BYTES  = ROWS * PROD_STRIDE * 4;
        // the tile as TMA delivers it, the tile's values of x, the products row by row
        static constexpr uint32_t SLOT_BYTES = TILE_BYTES + 128 + PROD_BYTES;
        static constexpr uint32_t GROUPS     = ROWS / 32;
        static constexpr uint32_t MULT       = 4; // multiplier warps per 32-row group
        static constexpr uint32_t PRODUCERS  = 2; // producer warps, tiles in turn
        static constexpr uint32_t THREADS    = ((1 + MULT) * GROUPS + PRODUCERS) * 32;
        // A wait on a barrier's phase parity is only right while the waiter cannot be a whole
        // phase ahead of the barrier.  The warp that waits for tile t in a slot must therefore
        // be the one that handled the slot's previous occupant, tile t - STAGES: otherwise a
        // multiplier warp that has run ahead can find the slot's barrier still in the phase
        // of the previous occupant (its copy not landed yet), take that for completion of its
        // own phase and multiply stale data.
        static_assert(STAGES % MULT == 0 && STAGES % PRODUCERS == 0,
                      "ring slots must stay with one multiplier warp and one producer warp");
        struct Control
        {
            uint64_t   full[STAGES]; // TMA data has landed
            uint64_t   prod[STAGES]; // products are in place
            uint64_t   empty[STAGES]; // the chain warps have read them
            AbortState abort;
        };
        static constexpr uint32_t SMEM_BYTES = STAGES * SLOT_BYTES + 128 + sizeof(Control);
    };

    template <uint32_t ROWS, uint32_t STAGES>
    __global__ void __launch_bounds__(ChainGeometry<ROWS, STAGES>::THREADS, 1)
        gemvChainKernel(const __grid_constant__ CUtensorMap tmapA,
                        const __grid_constant__ CUtensorMap tmapX, uint32_t m, uint32_t k,
                        float const* yIn, float* yOut, float alpha, float beta, uint32_t* status)
    {
        using G       = ChainGeometry<ROWS, STAGES>;
        using Control = typename G::Control;
        constexpr uint32_t COLS = G::COLS, TILE_BYTES = G::TILE_BYTES, SLOT_BYTES = G::SLOT_BYTES;
        constexpr uint32_t GROUPS = G::GROUPS, MULT = G::MULT, PROD_STRIDE = G::PROD_STRIDE;
        constexpr uint32_t PROD_OFFSET = TILE_BYTES + 128;
        extern __shared__ uint8_t smemRaw[];
        const uint32_t            raw   = smem_addr(smemRaw);
        uint8_t*                  tiles = smemRaw + ((128u - (raw & 127u)) & 127u);
        Control* ctl = reinterpret_cast<Control*>(tiles + STAGES * SLOT_BYTES);

        const uint32_t warp  = threadIdx.x / 32u, lane = threadIdx.x % 32u;
        const uint32_t row0  = blockIdx.x * ROWS;
        const uint32_t numKB = (k + COLS - 1) / COLS;

        if(threadIdx.x == 0)
        {
            for(uint32_t s = 0; s < STAGES; ++s)
            {
                mbar_init(&ctl->full[s], 1);
                mbar_init(&ctl->prod[s], ROWS);
                mbar_init(&ctl->empty[s], ROWS);
            }
            ctl->abort.flag = 0;
            ctl->abort.code = 0;
            mbar_init_fence();
            tma_prefetch_descriptor(&tmapA);
            tma_prefetch_descriptor(&tmapX);
        }
        __syncthreads();
        grid_dependency_wait();
        grid_launch_dependents();

        struct RingPos
        {
            uint32_t slot, phase;
            __device__ void advance()
            {
                if(++slot == STAGES)
                {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        };

        // Roles.  Warp w issues through scheduler w % 4; with one 32-row group the chain warp
        // is warp 0 and the first producer warp 4, so that the chain shares its scheduler with
        // a warp that mostly sleeps: multipliers are warps 1, 2, 3 and 5, further producers 6...
        constexpr uint32_t NPROD = G::PRODUCERS;
        uint32_t           producer = ~0u; // index among the producer warps, or none
        if constexpr(GROUPS == 1u)
        {
            if(warp == 4u)
                producer = 0u;
            else if(warp >= 6u)
                producer = warp - 5u;
        }
        else if(warp >= (1u + MULT) * GROUPS)
            producer = warp - (1u + MULT) * GROUPS;
        if(producer != ~0u)
        {
            // ---- producers: one thread each, every NPROD-th tile, two TMA loads per tile ----
            // (one thread gets through a tile -- barrier test, expect_tx, two TMA instructions --
            // in ~230 cycles, more than the chain warp needs to add the tile up)
            if(elect_one())
            {
                RingPos pos{0u, 0u};
                for(uint32_t i = 0; i < producer; ++i)
                    pos.advance();
                uint32_t kb = producer;
                for(; kb < numKB; kb += NPROD)
                {
                    if(!mbar_wait(&ctl->empty[pos.slot], pos.phase ^ 1u, &ctl->abort,
                                  WAIT_STAGE_EMPTY))
                        break;
                    uint8_t* slot = tiles + pos.slot * SLOT_BYTES;
                    mbar_expect_tx(&ctl->full[pos.slot], PROD_OFFSET); // the tile and its x
                    tma_load_2d(slot, &tmapA, &ctl->full[pos.slot], int32_t(row0),
                                int32_t(kb * COLS));
                    tma_load_1d(slot + TILE_BYTES, &tmapX, &ctl->full[pos.slot],
                                int32_t(kb * COLS));
                    for(uint32_t i = 0; i < NPROD; ++i)
                        pos.advance();
                }
                if(kb < numKB)
                {
                    // leaving early: this thread's copies already issued (tiles kb - NPROD,
                    // kb - 2 NPROD, ... still in the ring) get a bounded time to land
                    const uint32_t issued  = (kb - producer) / NPROD;
                    const uint32_t inRing  = (STAGES + NPROD - 1u) / NPROD;
                    const uint32_t pending = issued < inRing ? issued : inRing;
                    for(uint32_t j = 0; j < pending; ++j)
                    {
                        const uint32_t  prev  = kb - NPROD * (1u + j);
                        const long long start = clock64();
                        while(!mbar_try_wait(&ctl->full[prev % STAGES], (prev / STAGES) & 1u)
                              && clock64() - start < 2000000ll)
                        {
                        }
                    }
                }
            }
        }
        else if(warp >= GROUPS)
        {
            // ---- multiplier warps: every MULT-th tile, rows of one 32-row group ----
            const uint32_t mw = GROUPS == 1u ? (warp < 4u ? warp - 1u : 3u) : warp - GROUPS;
            const uint32_t group = mw / MULT, turn = mw % MULT;
            const uint32_t r     = group * 32u + lane;
            RingPos        pos{0u, 0u};
            for(uint32_t i = 0; i < turn; ++i)
                pos.advance();
            for(uint32_t kb = turn; kb < numKB; kb += MULT)
            {
                if(!mbar_wait(&ctl->full[pos.slot], pos.phase, &ctl->abort, WAIT_STAGE_FULL))
                    break;
                float const* tile = reinterpret_cast<float const*>(tiles + pos.slot * SLOT_BYTES);
                Vec<float, 4> const* xs = reinterpret_cast<Vec<float, 4> const*>(
                    tiles + pos.slot * SLOT_BYTES + TILE_BYTES);
                Vec<float, 4>* out = reinterpret_cast<Vec<float, 4>*>(
                    tiles + pos.slot * SLOT_BYTES + PROD_OFFSET + r * PROD_STRIDE * 4u);
                float av[COLS], xv[COLS];
#pragma unroll
                for(uint32_t j = 0; j < COLS; j += 4u)
                {
                    const Vec<float, 4> q = xs[j / 4u]; // same address in every lane: broadcast
#pragma unroll
                    for(uint32_t e = 0; e < 4u; ++e)
                        xv[j + e] = q.v[e];
                }
#pragma unroll
                for(uint32_t j = 0; j < COLS; ++j)
                    av[j] = tile[j * ROWS + r];
#pragma unroll
                for(uint32_t j = 0; j < COLS; j += 4u)
                {
                    Vec<float, 4> q;
#pragma unroll
                    for(uint32_t e = 0; e < 4u; ++e)
                        q.v[e] = mulRn(av[j + e], xv[j + e]);
                    out[j / 4u] = q;
                }
                // releases the products to the chain warp; the TMA area of the slot has only
                // been read, and is not written again before the chain warp has handed the
                // slot back through `empty`
                mbar_arrive(&ctl->prod[pos.slot]);
                for(uint32_t i = 0; i < MULT; ++i)
                    pos.advance();
            }
        }
        else
        {
            // ---- chain warps: one row per thread, columns in ascending order ----
            const uint32_t r        = warp * 32u + lane;
            const uint32_t numFull  = k / COLS;
            float          acc      = 0.0f;
            RingPos        toLoad{0u, 0u}, toRelease{0u, 0u};
            bool           ok       = true;
            auto productsOf = [&](uint32_t s) {
                return reinterpret_cast<Vec<float, 4> const*>(tiles + s * SLOT_BYTES + PROD_OFFSET
                                                              + r * PROD_STRIDE * 4u);
            };
            auto loadProducts = [&](uint32_t s, float (&pv)[COLS]) {
                Vec<float, 4> const* row = productsOf(s);
#pragma unroll
                for(uint32_t j = 0; j < COLS; j += 4u)
                {
                    const Vec<float, 4> q = row[j / 4u];
#pragma unroll
                    for(uint32_t e = 0; e < 4u; ++e)
                        pv[j + e] = q.v[e];
                }
            };
            auto waitProd = [&](RingPos const& at) -> bool {
                return mbar_wait(&ctl->prod[at.slot], at.phase, &ctl->abort, WAIT_STAGE_FULL);
            };
            auto releaseSlot = [&]() {
                mbar_arrive(&ctl->empty[toRelease.slot]);
                toRelease.advance();
            };
            // one step: adds tile t (`cur`, in registers), loads tile t + 1 (whose arrival was
            // established before the trip) into `next`, polls for a tile four further on
            RingPos toPoll{0u, 0u};
            auto    step = [&](float const (&cur)[COLS], float (&next)[COLS], bool& allArrived) {
                Vec<float, 4> const* row = productsOf(toLoad.slot);
                toLoad.advance();
#pragma unroll
                for(uint32_t j = 0; j < COLS; ++j)
                {
                    acc = addRn(acc, cur[j]);
                    if(j % 4u == 0u)
                    {
                        const Vec<float, 4> q = row[j / 4u];
#pragma unroll
                        for(uint32_t e = 0; e < 4u; ++e)
                            next[j + e] = q.v[e];
                    }
                    if(j == COLS / 4u + 1u)
                        allArrived
                            = mbar_try_wait(&ctl->prod[toPoll.slot], toPoll.phase) && allArrived;
                }
                toPoll.advance();
                releaseSlot(); // tile t: its products were consumed by the additions above
            };
            float pA[COLS], pB[COLS];
            if(numFull > 0u)
            {
                ok = waitProd(toLoad);
                if(ok)
                {
                    loadProducts(toLoad.slot, pA);
                    toLoad.advance();
                }
                // steady state: a trip of four steps starting at tile t loads tiles
                // t + 1 .. t + 4 and polls t + 5 .. t + 8
                uint32_t t = 0;
                toPoll     = toLoad;
                for(uint32_t i = 0; i < 4u; ++i)
                    toPoll.advance();
                bool arrivedAll = false;
                for(; ok && t + 8u < numFull; t += 4u)
                {
                    if(!arrivedAll)
                    {
                        RingPos w = toLoad;
                        for(uint32_t i = 0; ok && i < 4u; ++i)
                        {
                            ok = waitProd(w);
                            w.advance();
                        }
                        if(!ok)
                            break;
                    }
                    bool all = true;
                    step(pA, pB, all);
                    step(pB, pA, all);
                    step(pA, pB, all);
                    step(pB, pA, all);
                    arrivedAll = all;
                }
                // the last full tiles, one simple step each (t is a multiple of 4: tile t is
                // in pA)
                for(uint32_t u = t; ok && u < numFull; ++u)
                {
                    const bool even        = ((u & 1u) == 0u);
                    float const(&cur)[COLS] = even ? pA : pB;
                    float(&next)[COLS]      = even ? pB : pA;
                    if(u + 1u < numFull)
                    {
                        ok = waitProd(toLoad);
                        if(!ok)
                            break;
                        loadProducts(toLoad.slot, next);
                        toLoad.advance();
                    }
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        acc = addRn(acc, cur[j]);
                    releaseSlot();
                }
            }
            if(ok && numFull < numKB)
            {
                // the partial last tile: columns beyond k hold 0 * 0 and must not enter the sum
                // (adding +0 could turn a -0 into +0)
                const uint32_t valid = k - numFull * COLS;
                float          pv[COLS];
                if(waitProd(toLoad))
                {
                    loadProducts(toLoad.slot, pv);
#pragma unroll
                    for(uint32_t j = 0; j < COLS; ++j)
                        if(j < valid)
                            acc = addRn(acc, pv[j]);
                    releaseSlot();
                }
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

    template <typename T, uint32_t ROWS, uint32_t STAGES>
    int launchStream(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha,
                     T beta, uint32_t lda, cudaStream_t stream)
    {
        using G = Geometry<T, ROWS, STAGES>;
        b200wmma::EncodeFn encode = b200wmma::tensorMapEncoder();
        if(!encode)
            return B200WMMA_ERR_CUDA;
        const CUtensorMapDataType dt = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT64;
        // A, column-major: m contiguous rows per column, k columns lda apart; a tile is ROWS
        // rows x COLS columns and lands in shared memory column after column
        CUtensorMap mapA, mapX;
        {
            cuuint64_t dims[2]    = {m, k};
            cuuint64_t strides[1] = {cuuint64_t(lda) * sizeof(T)};
            cuuint32_t box[2]     = {ROWS, G::COLS};
            cuuint32_t estr[2]    = {1, 1};
            if(encode(&mapA, dt, 2, const_cast<T*>(a), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return B200WMMA_ERR_CUDA;
        }
        {
            cuuint64_t dims[1]    = {k};
            cuuint64_t strides[1] = {0}; // a one-dimensional map has no strides; never read
            cuuint32_t box[1]     = {G::COLS};
            cuuint32_t estr[1]    = {1};
            if(encode(&mapX, dt, 1, const_cast<T*>(x), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return B200WMMA_ERR_CUDA;
        }
        auto        kernel = gemvStreamKernel<T, ROWS, STAGES>;
        static bool attrDone[64] = {};
        int         dev          = 0;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev < 0 || dev >= 64 || !attrDone[dev])
        {
            B200WMMA_CUDA_TRY(cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(G::SMEM_BYTES)));
            if(dev >= 0 && dev < 64)
                attrDone[dev] = true;
        }
        return b200wmma::cudaToStatus(b200wmma::launchOverlapped(
            kernel, dim3((m + ROWS - 1) / ROWS), dim3(G::THREADS), G::SMEM_BYTES, stream, mapA,
            mapX, m, k, yIn, yOut, alpha, beta, b200wmma::deviceStatusWord()));
    }

    template <uint32_t ROWS, uint32_t STAGES>
    int launchChain(uint32_t m, uint32_t k, float const* a, float const* x, float const* yIn,
                    float* yOut, float alpha, float beta, uint32_t lda, cudaStream_t stream)
    {
        using G = ChainGeometry<ROWS, STAGES>;
        b200wmma::EncodeFn encode = b200wmma::tensorMapEncoder();
        if(!encode)
            return B200WMMA_ERR_CUDA;
        CUtensorMap mapA, mapX;
        {
            cuuint64_t dims[2]    = {m, k};
            cuuint64_t strides[1] = {cuuint64_t(lda) * 4u};
            cuuint32_t box[2]     = {ROWS, G::COLS};
            cuuint32_t estr[2]    = {1, 1};
            if(encode(&mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(a), dims,
                      strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return B200WMMA_ERR_CUDA;
        }
        {
            cuuint64_t dims[1]    = {k};
            cuuint64_t strides[1] = {0}; // a one-dimensional map has no strides; never read
            cuuint32_t box[1]     = {G::COLS};
            cuuint32_t estr[1]    = {1};
            if(encode(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 1, const_cast<float*>(x), dims,
                      strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return B200WMMA_ERR_CUDA;
        }
        auto        kernel = gemvChainKernel<ROWS, STAGES>;
        static bool attrDone[64] = {};
        int         dev          = 0;
        B200WMMA_CUDA_TRY(cudaGetDevice(&dev));
        if(dev < 0 || dev >= 64 || !attrDone[dev])
        {
            B200WMMA_CUDA_TRY(cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(G::SMEM_BYTES)));
            if(dev >= 0 && dev < 64)
                attrDone[dev] = true;
        }
        return b200wmma::cudaToStatus(b200wmma::launchOverlapped(
            kernel, dim3((m + ROWS - 1) / ROWS), dim3(G::THREADS), G::SMEM_BYTES, stream, mapA,
            mapX, m, k, yIn, yOut, alpha, beta, b200wmma::deviceStatusWord()));
    }

    template <typename T>
    int run(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha, T beta,
            uint32_t lda, cudaStream_t stream)
    {
        // TMA needs 16-byte aligned bases and column stride
        const bool streamOK = (reinterpret_cast<uintptr_t>(a) % 16 == 0)
                              && (reinterpret_cast<uintptr_t>(x) % 16 == 0)
                              && ((size_t(lda) * sizeof(T)) % 16 == 0);
        if(!streamOK)
        {
            gemvPlainKernel<T><<<(m + 127) / 128, 128, 0, stream>>>(m, k, a, x, yIn, yOut, alpha,
                                                                  beta, lda);
            return b200wmma::cudaToStatus(cudaGetLastError());
        }
        // 64 rows per block fill a B200 from 148 x 2 x 64 = 18944 rows up; with fewer rows
        // than half of that, 32-row blocks put twice as many SMs to work (a row's ordered sum
        // takes the same time either way, so the launch takes as long as one block does).
        // B200WMMA_GEMV_ROWS=32|64 forces one form (tuning and comparison only).
        static const uint32_t rowsEnv = [] {
            const char* e = getenv("B200WMMA_GEMV_ROWS");
            return e ? uint32_t(atoi(e)) : 0u;
        }();
        const int sms = b200wmma::smCount();
        if(sms <= 0)
            return B200WMMA_ERR_CUDA;
        bool narrow = (m + 63u) / 64u < uint32_t(sms);
        if(rowsEnv == 32u || rowsEnv == 64u)
            narrow = rowsEnv == 32u;
        if constexpr(sizeof(T) == 4)
        {
            // fp32 with at most one 32-row block per SM (a row shard of a many-GPU run): the
            // launch takes as long as one row's ordered sum, so the multiplications go to
            // warps of their own (gemvChainKernel: 81 vs 93 us for 2048 and 4096 rows).  With
            // more rows than that the kernel is bandwidth-bound and the second pass through
            // shared memory costs more than it saves (8192 rows: 109 vs 95 us; 16384: 181 vs
            // 165).  B200WMMA_GEMV_FORM=single|chain forces one form (comparison).
            const char* form = getenv("B200WMMA_GEMV_FORM");
            const bool forced = form && form[0] == 'c';
            if(forced || (!(form && form[0] == 's') && (m + 31u) / 32u <= uint32_t(sms)))
            {
                if(!narrow)
                    return launchChain<64, 12>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
                // a ring of 20 slots fills the shared memory of an SM; with more blocks than
                // SMs two blocks share one, with 12 slots each
                if((m + 31u) / 32u <= uint32_t(sms))
                    return launchChain<32, 20>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
                return launchChain<32, 12>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
            }
        }
        if(narrow)
            return launchStream<T, 32, 24>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
        return launchStream<T, 64, 12>(m, k, a, x, yIn, yOut, alpha, beta, lda, stream);
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
