// Cooperative fragment transfers: several warps of a thread block share the
// work of moving ONE tile, each moving a contiguous slice of the fragment's
// work items.  Same three live call forms as rocWMMA's rocwmma_coop.hpp:86-415
// (rocwmma_coop_impl.hpp:61-170):
//
//   load_matrix_coop_sync(frag, data, ldm, waveIndex, waveCount)
//   load_matrix_coop_sync(frag, data, ldm)            all warps, row-major warp order
//   load_matrix_coop_sync<WaveCount>(frag, data, ldm, waveIndex)
//
// and the same for store_matrix_coop_sync.  Rules kept from the reference:
// after a cooperative load a warp's fragment is only partially filled; a store
// with the same (waveIndex, waveCount) writes exactly what that load read, so a
// load/store pair over all warps moves the whole tile; when the warp count does
// not divide the work it is halved until it does, and warps beyond that count
// return without touching memory (internal/coop_load.hpp:99-127).
#ifndef ROCWMMA_B200_COOP_API_HPP
#define ROCWMMA_B200_COOP_API_HPP

#include "rocwmma.hpp"

namespace rocwmma
{
    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT*                                                   data,
                              uint32_t                                                       ldm,
                              uint32_t waveIndex,
                              uint32_t waveCount)
    {
        static_assert(!stdx::is_same<DataLayoutT, void>::value,
                      "Must provide layout information. Either statically assign data layout in "
                      "fragment declaration or use the run-time function overload.");
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geom;
        const uint32_t maxWaves = detail::coopMaxWaves(Geom::Units, waveCount);
        if(waveIndex >= maxWaves)
            return;
        const uint32_t per = Geom::Units / maxWaves;
        detail::UnitIO<Geom, DataLayoutT>::loadRange(frag.x, data, ldm, waveIndex * per, per);
    }

    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT*                                                   data,
                              uint32_t                                                       ldm)
    {
        // Default: all warps of the block take part, numbered row-major over (x, y)
        // (rocwmma_coop_impl.hpp:103-112).
        const uint32_t wavesX    = ::blockDim.x / Constants::AMDGCN_WAVE_SIZE;
        const uint32_t wavesY    = ::blockDim.y;
        const uint32_t waveIndex = (threadIdx.x / Constants::AMDGCN_WAVE_SIZE) * wavesY
                                   + threadIdx.y;
        load_matrix_coop_sync(frag, data, ldm, waveIndex, wavesX * wavesY);
    }

    template <uint32_t WaveCount,
              typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_coop_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                              const DataT*                                                   data,
                              uint32_t                                                       ldm,
                              uint32_t waveIndex)
    {
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geom;
        constexpr uint32_t maxWaves = detail::coopMaxWaves(Geom::Units, WaveCount);
        constexpr uint32_t per      = Geom::Units / maxWaves;
        if(waveIndex >= maxWaves)
            return;
        detail::UnitIO<Geom, DataLayoutT>::loadRange(frag.x, data, ldm, waveIndex * per, per);
    }

    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void store_matrix_coop_sync(
        DataT*                                                               data,
        fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
        uint32_t                                                             ldm,
        uint32_t                                                             waveIndex,
        uint32_t                                                             waveCount)
    {
        static_assert(!stdx::is_same<DataLayoutT, void>::value,
                      "Must provide data layout. Either statically assign data layout in "
                      "fragment declaration or use the run-time function overload.");
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geom;
        const uint32_t maxWaves = detail::coopMaxWaves(Geom::Units, waveCount);
        if(waveIndex >= maxWaves)
            return;
        const uint32_t per = Geom::Units / maxWaves;
        detail::UnitIO<Geom, DataLayoutT>::storeRange(data, frag.x, ldm, waveIndex * per, per);
    }

    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void store_matrix_coop_sync(
        DataT*                                                               data,
        fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
        uint32_t                                                             ldm)
    {
        const uint32_t wavesX    = ::blockDim.x / Constants::AMDGCN_WAVE_SIZE;
        const uint32_t wavesY    = ::blockDim.y;
        const uint32_t waveIndex = (threadIdx.x / Constants::AMDGCN_WAVE_SIZE) * wavesY
                                   + threadIdx.y;
        store_matrix_coop_sync(data, frag, ldm, waveIndex, wavesX * wavesY);
    }

    template <uint32_t WaveCount,
              typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void store_matrix_coop_sync(
        DataT*                                                               data,
        fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
        uint32_t                                                             ldm,
        uint32_t                                                             waveIndex)
    {
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geom;
        constexpr uint32_t maxWaves = detail::coopMaxWaves(Geom::Units, WaveCount);
        constexpr uint32_t per      = Geom::Units / maxWaves;
        if(waveIndex >= maxWaves)
            return;
        detail::UnitIO<Geom, DataLayoutT>::storeRange(data, frag.x, ldm, waveIndex * per, per);
    }
} // namespace rocwmma

#endif // ROCWMMA_B200_COOP_API_HPP
