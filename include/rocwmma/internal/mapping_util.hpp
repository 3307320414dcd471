// Warp <-> tile <-> matrix <-> memory coordinate helpers of the fragment API.
//
// Same contract as rocWMMA's MappingUtil (internal/mapping_util.hpp:131-210,
// internal/mapping_util_impl.hpp:46-278): the thread block is
// (warps_x * 32, warps_y); warp (x, y) of the grid owns tile row x and tile
// column y; a tile is BlockHeight x BlockWidth elements.
#ifndef ROCWMMA_B200_MAPPING_UTIL_HPP
#define ROCWMMA_B200_MAPPING_UTIL_HPP

#include "constants.hpp"
#include "coord.hpp"

namespace rocwmma
{
    struct row_major;
    struct col_major;

    namespace detail
    {
        template <typename Layout>
        struct DataSpace;

        template <>
        struct DataSpace<row_major>
        {
            ROCWMMA_HOST_DEVICE constexpr static uint32_t leadingDim(Coord2d const& size)
            {
                return size.data[1];
            }
            ROCWMMA_HOST_DEVICE constexpr static uint32_t fromMatrixCoord(Coord2d const& c,
                                                                          uint32_t       ld)
            {
                return c.data[0] * ld + c.data[1];
            }
        };
        template <>
        struct DataSpace<col_major>
        {
            ROCWMMA_HOST_DEVICE constexpr static uint32_t leadingDim(Coord2d const& size)
            {
                return size.data[0];
            }
            ROCWMMA_HOST_DEVICE constexpr static uint32_t fromMatrixCoord(Coord2d const& c,
                                                                          uint32_t       ld)
            {
                return c.data[1] * ld + c.data[0];
            }
        };
    } // namespace detail

    template <uint32_t BlockHeight, uint32_t BlockWidth, typename DataT, typename DataLayoutT>
    struct MappingUtil
    {
        using WaveCoordT    = Coord2d;
        using BlockCoordT   = Coord2d;
        using MatrixCoordT  = Coord2d;
        using WorkgroupDimT = Coord2d;
        using DataSpace     = detail::DataSpace<DataLayoutT>;

        ROCWMMA_DEVICE static inline uint32_t laneId()
        {
            return threadIdx.x & (Constants::AMDGCN_WAVE_SIZE - 1u);
        }
        // Warp position inside the thread block.
        ROCWMMA_DEVICE static inline WaveCoordT waveCoord()
        {
            return make_coord2d(threadIdx.x / Constants::AMDGCN_WAVE_SIZE, threadIdx.y);
        }
        // Warp position inside the grid == coordinate of the tile it owns.
        ROCWMMA_DEVICE static inline BlockCoordT blockCoord()
        {
            return make_coord2d((blockIdx.x * blockDim.x + threadIdx.x)
                                    / Constants::AMDGCN_WAVE_SIZE,
                                blockIdx.y * blockDim.y + threadIdx.y);
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoord()
        {
            return matrixCoord(blockCoord());
        }
        ROCWMMA_DEVICE static inline WorkgroupDimT workgroupDim()
        {
            return make_coord2d(blockDim.x / Constants::AMDGCN_WAVE_SIZE, blockDim.y);
        }
        ROCWMMA_DEVICE static inline DataT const* dataCoord(DataT const* baseAddr, uint32_t ldm)
        {
            return baseAddr + DataSpace::fromMatrixCoord(matrixCoord(), ldm);
        }
        ROCWMMA_DEVICE static inline DataT* dataCoord(DataT* baseAddr, uint32_t ldm)
        {
            return baseAddr + DataSpace::fromMatrixCoord(matrixCoord(), ldm);
        }
        ROCWMMA_DEVICE static inline BlockCoordT blockCoordM(uint32_t m)
        {
            auto c    = blockCoord();
            c.data[0] = m;
            return c;
        }
        ROCWMMA_DEVICE static inline BlockCoordT blockCoordN(uint32_t n)
        {
            auto c    = blockCoord();
            c.data[1] = n;
            return c;
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoordM(uint32_t m)
        {
            auto c    = matrixCoord();
            c.data[0] = m;
            return c;
        }
        ROCWMMA_DEVICE static inline MatrixCoordT matrixCoordN(uint32_t n)
        {
            auto c    = matrixCoord();
            c.data[1] = n;
            return c;
        }
        ROCWMMA_HOST_DEVICE static inline MatrixCoordT matrixCoord(BlockCoordT const& blockCoord)
        {
            return make_coord2d(blockCoord.data[0] * BlockHeight, blockCoord.data[1] * BlockWidth);
        }
        ROCWMMA_HOST_DEVICE static inline uint32_t dataOffset(MatrixCoordT const& matrixCoord,
                                                              uint32_t            ldm)
        {
            return DataSpace::fromMatrixCoord(matrixCoord, ldm);
        }
        ROCWMMA_HOST_DEVICE static inline DataT const*
            dataCoord(DataT const* baseAddr, MatrixCoordT const& matrixCoord, uint32_t ldm)
        {
            return baseAddr + DataSpace::fromMatrixCoord(matrixCoord, ldm);
        }
        ROCWMMA_HOST_DEVICE static inline DataT*
            dataCoord(DataT* baseAddr, MatrixCoordT const& matrixCoord, uint32_t ldm)
        {
            return baseAddr + DataSpace::fromMatrixCoord(matrixCoord, ldm);
        }
    };
} // namespace rocwmma

#endif // ROCWMMA_B200_MAPPING_UTIL_HPP
