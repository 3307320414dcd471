// Fragment <-> memory movers shared by load/store_matrix_sync and their
// cooperative forms.
//
// Stands where rocWMMA has OpaqueLoad / OpaqueStore / CooperativeLoad /
// CooperativeStore (internal/opaque_load.hpp:78-158, internal/opaque_store.hpp,
// internal/coop_load.hpp:99-222).  Element (r, c) of the tile lives at
// data[r*ldm + c] for row_major and data[c*ldm + r] for col_major
// (internal/mapping_util_impl.hpp:142-150).  `data` may point to global or
// shared memory.  A unit whose elements are contiguous in memory moves as one
// 4/8/16-byte access when pointer and leading dimension allow it, otherwise
// element by element; the choice is uniform over the warp.
#ifndef ROCWMMA_B200_FRAG_IO_HPP
#define ROCWMMA_B200_FRAG_IO_HPP

#include "frag_geometry.hpp"

namespace rocwmma
{
    namespace detail
    {
        template <typename DataT, uint32_t N>
        struct alignas(sizeof(DataT) * N) Pack
        {
            DataT v[N];
        };

        template <typename Geom, typename DataLayoutT>
        struct UnitIO
        {
            static constexpr bool RowMajor   = stdx::is_same<DataLayoutT, row_major>::value;
            static constexpr bool Contiguous = (Geom::UnitAlongCols == RowMajor);
            static constexpr uint32_t US     = Geom::UnitSize;

            ROCWMMA_DEVICE static inline uint32_t offset(Coord2d const& c, uint32_t ldm)
            {
                return RowMajor ? c.data[0] * ldm + c.data[1] : c.data[1] * ldm + c.data[0];
            }
            // Stride between consecutive elements of a unit.
            ROCWMMA_DEVICE static inline uint32_t step(uint32_t ldm)
            {
                return Contiguous ? 1u : ldm;
            }

            template <typename DataT>
            ROCWMMA_DEVICE static inline bool canVectorize(DataT const* data, uint32_t ldm)
            {
                if constexpr(Contiguous && US > 1)
                {
                    constexpr uint32_t bytes = sizeof(DataT) * US;
                    return ((reinterpret_cast<uintptr_t>(data) | (uintptr_t(ldm) * sizeof(DataT)))
                            % bytes)
                           == 0;
                }
                return false;
            }

            // Position of unit u in the fragment's WORK-ITEM order, the order cooperative
            // transfers cut into per-warp slices.  For matrix_a and accumulator fragments it
            // is the unit order itself.  For a matrix_b fragment that has a transpose
            // (BlockN a multiple of 16) it is the index of the SAME data in the transposed
            // matrix_a fragment (applyTranspose, rocwmma_transforms.hpp), so that a slice
            // loaded into a B fragment is, after applyTranspose, exactly the slice a
            // cooperative store of the A fragment with the same warp index writes -- which
            // is how rocWMMA's macro-tile kernels stage B through shared memory
            // (samples/perf_hgemm.cpp:356-365).  In the reference the two fragment types
            // share one register layout and the property is automatic.
            ROCWMMA_DEVICE static constexpr uint32_t workIndex(uint32_t u)
            {
                if constexpr(Geom::IsB && (Geom::AtomsMajor % 2u == 0u))
                {
                    constexpr uint32_t UB = Geom::UnitsPerAtom, KT = Geom::AtomsMinor;
                    const uint32_t     atom = u / UB, jk = u % UB;
                    const uint32_t     nt = atom / KT, kt = atom % KT;
                    return ((nt / 2u) * KT + kt) * (2u * UB) + ((jk << 1) | (nt & 1u));
                }
                else
                    return u;
            }

            // Moves the units whose work-item index lies in [begin, begin + count) between
            // x[] and memory.
            template <bool Vectorized, typename DataT, uint32_t N>
            ROCWMMA_DEVICE static inline void
                load(DataT (&x)[N], DataT const* data, uint32_t ldm, uint32_t begin, uint32_t count)
            {
                const uint32_t lane = threadIdx.x & 31u;
                ROCWMMA_UNROLL
                for(uint32_t u = 0; u < Geom::Units; ++u)
                {
                    if(workIndex(u) >= begin && workIndex(u) < begin + count)
                    {
                        const uint32_t off = offset(Geom::unitCoord(u, lane), ldm);
                        if constexpr(Vectorized)
                        {
                            auto p = *reinterpret_cast<Pack<DataT, US> const*>(data + off);
                            ROCWMMA_UNROLL
                            for(uint32_t s = 0; s < US; ++s)
                                x[u * US + s] = p.v[s];
                        }
                        else
                        {
                            const uint32_t st = step(ldm);
                            ROCWMMA_UNROLL
                            for(uint32_t s = 0; s < US; ++s)
                                x[u * US + s] = data[off + s * st];
                        }
                    }
                }
            }

            template <bool Vectorized, typename DataT, uint32_t N>
            ROCWMMA_DEVICE static inline void store(DataT*   data,
                                                    DataT const (&x)[N],
                                                    uint32_t ldm,
                                                    uint32_t begin,
                                                    uint32_t count)
            {
                const uint32_t lane = threadIdx.x & 31u;
                ROCWMMA_UNROLL
                for(uint32_t u = 0; u < Geom::Units; ++u)
                {
                    if(workIndex(u) >= begin && workIndex(u) < begin + count)
                    {
                        const uint32_t off = offset(Geom::unitCoord(u, lane), ldm);
                        if constexpr(Vectorized)
                        {
                            Pack<DataT, US> p;
                            ROCWMMA_UNROLL
                            for(uint32_t s = 0; s < US; ++s)
                                p.v[s] = x[u * US + s];
                            *reinterpret_cast<Pack<DataT, US>*>(data + off) = p;
                        }
                        else
                        {
                            const uint32_t st = step(ldm);
                            ROCWMMA_UNROLL
                            for(uint32_t s = 0; s < US; ++s)
                                data[off + s * st] = x[u * US + s];
                        }
                    }
                }
            }

            template <typename DataT, uint32_t N>
            ROCWMMA_DEVICE static inline void loadRange(
                DataT (&x)[N], DataT const* data, uint32_t ldm, uint32_t begin, uint32_t count)
            {
                if(canVectorize(data, ldm))
                    load<Contiguous && (US > 1)>(x, data, ldm, begin, count);
                else
                    load<false>(x, data, ldm, begin, count);
            }
            template <typename DataT, uint32_t N>
            ROCWMMA_DEVICE static inline void storeRange(
                DataT* data, DataT const (&x)[N], uint32_t ldm, uint32_t begin, uint32_t count)
            {
                if(canVectorize(data, ldm))
                    store<Contiguous && (US > 1)>(data, x, ldm, begin, count);
                else
                    store<false>(data, x, ldm, begin, count);
            }
        };

        // Number of warps a cooperative transfer of `units` work items is split
        // over: the warp count, halved until it divides the work
        // (rocWMMA internal/coop_load.hpp:99-103).
        ROCWMMA_HOST_DEVICE constexpr inline uint32_t coopMaxWaves(uint32_t units,
                                                                   uint32_t waveCount)
        {
            uint32_t w = waveCount == 0u ? 1u : waveCount;
            while(w > 1u && (units % w) != 0u)
                w /= 2u;
            return w;
        }
    } // namespace detail
} // namespace rocwmma

#endif // ROCWMMA_B200_FRAG_IO_HPP
