// Which matrix element each lane of a warp keeps in which slot of a fragment.
//
// rocWMMA leaves the element order inside a fragment unspecified
// (rocwmma.hpp:126) and derives it from AMD MFMA/WMMA register layouts
// (internal/io_layout.hpp, internal/layout/*).  Here the order is the operand
// order of the warp-level mma.sync instruction for the data type, so that
// mma_sync can hand fragment storage to the tensor core unchanged:
//
//   * a fragment is cut into "atoms": 16 x KA tiles of A, KA x 8 tiles of B,
//     16 x 8 tiles of the accumulator, where KA is the K extent of one
//     mma.sync (4 for 64-bit, 8 for 32-bit, 16 for 16-bit, 32 for 8-bit types),
//     or of its half-depth form when BlockK is not a multiple of that extent
//     (4 for 32-bit, 8 for 16-bit, 16 for 8-bit types): rocWMMA's 32 x 32 blocks
//     go down to BlockK = 8 for 16-bit and 16 for 8-bit inputs
//     (test/gemm/gemm_predicates_base.hpp:137-209);
//   * inside an atom a lane (g = lane / 4, t = lane % 4) owns "units" of
//     consecutive elements: one 32-bit register worth of A or B elements along
//     K, or two neighbouring accumulator columns;
//   * the accumulator map depends only on BlockM x BlockN, never on the data
//     type or memory layout, so accumulator fragments of one shape can be
//     combined element by element (alpha * acc.x[i] + beta * c.x[i]), as
//     rocWMMA kernels do (samples/simple_hgemm.cpp:131-134).
//
// Sizes follow rocWMMA: A is BlockM x BlockK, B is BlockK x BlockN, the
// accumulator BlockM x BlockN (internal/io_shape.hpp:44-80), and a lane holds
// rows*cols/32 elements (internal/io_traits.hpp:60-66).
#ifndef ROCWMMA_B200_FRAG_GEOMETRY_HPP
#define ROCWMMA_B200_FRAG_GEOMETRY_HPP

#include "constants.hpp"
#include "coord.hpp"
#include "types.hpp"

namespace rocwmma
{
    struct row_major
    {
    };
    struct col_major
    {
    };
    struct matrix_a
    {
    };
    struct matrix_b
    {
    };
    struct accumulator
    {
    };

    namespace detail
    {
        template <typename DataT, uint32_t BlockK>
        ROCWMMA_HOST_DEVICE constexpr uint32_t kAtom()
        {
            return sizeof(DataT) == 8   ? 4u
                   : sizeof(DataT) == 4 ? ((BlockK % 8u == 0u) ? 8u : 4u)
                   : sizeof(DataT) == 2 ? ((BlockK % 16u == 0u) ? 16u : 8u)
                                        : ((BlockK % 32u == 0u) ? 32u : 16u);
        }

        // Elements of DataT in one 32-bit register (1 for 32- and 64-bit types).
        template <typename DataT>
        ROCWMMA_HOST_DEVICE constexpr uint32_t perReg()
        {
            return sizeof(DataT) >= 4 ? 1u : uint32_t(4u / sizeof(DataT));
        }

        template <typename MatrixT,
                  uint32_t BlockM,
                  uint32_t BlockN,
                  uint32_t BlockK,
                  typename DataT>
        struct FragGeom
        {
            static constexpr bool IsA   = stdx::is_same<MatrixT, matrix_a>::value;
            static constexpr bool IsB   = stdx::is_same<MatrixT, matrix_b>::value;
            static constexpr bool IsAcc = stdx::is_same<MatrixT, accumulator>::value;
            static_assert(IsA || IsB || IsAcc, "MatrixT must be matrix_a, matrix_b or accumulator");

            static constexpr uint32_t KA = kAtom<DataT, BlockK>();
            static constexpr uint32_t P  = perReg<DataT>();

            // Logical matrix held by the fragment.
            static constexpr uint32_t Height = IsB ? BlockK : BlockM;
            static constexpr uint32_t Width  = IsA ? BlockK : BlockN;
            // Leading ("block") and K dimensions as rocWMMA reports them.
            static constexpr uint32_t BlockDim = IsA ? BlockM : BlockN;
            static constexpr uint32_t KDim     = BlockK;

            // Elements in one unit, units in one atom, atoms along each axis.
            static constexpr uint32_t UnitSize     = IsAcc ? 2u : P;
            static constexpr uint32_t UnitsPerAtom = IsA ? KA / (2u * P) : IsB ? KA / (4u * P) : 2u;
            static constexpr uint32_t AtomsMajor   = IsB ? BlockN / 8u : BlockM / 16u;
            static constexpr uint32_t AtomsMinor   = IsAcc ? BlockN / 8u : BlockK / KA;
            static constexpr uint32_t Atoms        = AtomsMajor * AtomsMinor;
            static constexpr uint32_t Units        = Atoms * UnitsPerAtom;
            static constexpr uint32_t Size         = Units * UnitSize;

            // Units run along columns (A: K, accumulator: N) or along rows (B: K).
            static constexpr bool UnitAlongCols = !IsB;

            static_assert(IsB || BlockM % 16u == 0u, "BlockM must be a multiple of 16");
            static_assert(IsA || BlockN % 8u == 0u, "BlockN must be a multiple of 8");
            static_assert(IsAcc || BlockK % KA == 0u,
                          "BlockK must be a multiple of the K extent of the shallowest "
                          "tensor-core instruction (4 for f64, f32 and xf32, 8 for 16-bit, 16 for "
                          "8-bit types)");
            static_assert(Size * 32u == Height * Width, "fragment does not tile its matrix");

            // (row, col) of the first element of unit `u` for lane `lane`.
            ROCWMMA_DEVICE static inline Coord2d unitCoord(uint32_t u, uint32_t lane)
            {
                const uint32_t g    = lane >> 2;
                const uint32_t t    = lane & 3u;
                const uint32_t atom = u / UnitsPerAtom;
                const uint32_t j    = u % UnitsPerAtom;
                const uint32_t maj  = atom / AtomsMinor;
                const uint32_t min  = atom % AtomsMinor;
                if constexpr(IsA)
                {
                    return make_coord2d(maj * 16u + g + 8u * (j & 1u),
                                        min * KA + (j >> 1) * 4u * P + t * P);
                }
                else if constexpr(IsB)
                {
                    return make_coord2d(min * KA + j * 4u * P + t * P, maj * 8u + g);
                }
                else
                {
                    return make_coord2d(maj * 16u + g + 8u * j, min * 8u + 2u * t);
                }
            }
        };

        // Plain aggregate used for the packed / unpacked views of a fragment.
        template <typename T, uint32_t N>
        struct VecT
        {
            T data[N];

            ROCWMMA_HOST_DEVICE constexpr T&       operator[](uint32_t i) { return data[i]; }
            ROCWMMA_HOST_DEVICE constexpr T const& operator[](uint32_t i) const { return data[i]; }
            ROCWMMA_HOST_DEVICE constexpr static uint32_t size() { return N; }
        };

        template <typename DataT, uint32_t Bytes = sizeof(DataT)>
        struct PackedOf
        {
            using type = DataT;
        };
        template <typename DataT>
        struct PackedOf<DataT, 1>
        {
            using type = uint32_t;
        };
        template <typename DataT>
        struct PackedOf<DataT, 2>
        {
            using type = uint32_t;
        };
    } // namespace detail
} // namespace rocwmma

#endif // ROCWMMA_B200_FRAG_GEOMETRY_HPP
