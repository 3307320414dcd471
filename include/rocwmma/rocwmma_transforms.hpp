// Fragment transforms: the value-level helpers rocWMMA's macro-tile kernels use when they
// stage tiles through shared memory (rocwmma_transforms.hpp:37-66; used by
// samples/perf_hgemm.cpp:303-310, 350-364).
//
//   ApplyTranspose_t<FragT> / applyTranspose(frag)
//       matrix_a<BlockM, BlockN, BlockK, T, L>  <->  matrix_b<BlockN, BlockM, BlockK, T, L'>
//       with L' the other layout: the same data seen as its transpose.  In the reference the
//       two fragment types share a register layout and the call is a re-cast
//       (rocwmma_transforms_impl.hpp:58-172).  Here A and B fragments keep the operand order
//       of mma.sync, which differs between the two, so the call returns a copy whose
//       registers are permuted inside each lane; no data moves between lanes.
//   ApplyDataLayout_t<FragT, Layout> / applyDataLayout<Layout>(frag)
//       the same fragment tagged with another memory layout.  Register contents do not
//       depend on the layout tag here, so this is a re-cast (the WaveCount parameter of the
//       reference is accepted and ignored).
#ifndef ROCWMMA_B200_TRANSFORMS_API_HPP
#define ROCWMMA_B200_TRANSFORMS_API_HPP

#include "rocwmma.hpp"

namespace rocwmma
{
    namespace detail
    {
        template <typename LayoutT>
        struct OrthogonalLayout;
        template <>
        struct OrthogonalLayout<row_major>
        {
            using type = col_major;
        };
        template <>
        struct OrthogonalLayout<col_major>
        {
            using type = row_major;
        };
        template <>
        struct OrthogonalLayout<void>
        {
            using type = void;
        };

        template <typename FragT>
        struct ApplyTranspose;

        // A (BlockM x BlockK) -> B (BlockK x BlockM).  A's atom (mt, kt) holds rows
        // 16 mt + g (+8); as columns of the transpose these are B's atoms nt = 2 mt and
        // 2 mt + 1 of the same kt.  Unit j of A = (K half << 1) | row half.
        template <uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
                  typename DataLayoutT>
        struct ApplyTranspose<fragment<matrix_a, BlockM, BlockN, BlockK, DataT, DataLayoutT>>
        {
            using FragA = fragment<matrix_a, BlockM, BlockN, BlockK, DataT, DataLayoutT>;
            using Type  = fragment<matrix_b, BlockN, BlockM, BlockK, DataT,
                                  typename OrthogonalLayout<DataLayoutT>::type>;

            ROCWMMA_DEVICE static inline Type exec(FragA const& a)
            {
                using GA = typename FragA::Geom;
                using GB = typename Type::Geom;
                static_assert(GA::Size == GB::Size && GA::UnitSize == GB::UnitSize,
                              "transposed fragment must hold the same elements");
                constexpr uint32_t KT = GA::AtomsMinor, P = GA::UnitSize;
                constexpr uint32_t KH = GB::UnitsPerAtom; // K halves per atom (1 or 2)
                Type               b;
                ROCWMMA_UNROLL
                for(uint32_t mt = 0; mt < GA::AtomsMajor; ++mt)
                    ROCWMMA_UNROLL
                for(uint32_t kt = 0; kt < KT; ++kt)
                    ROCWMMA_UNROLL
                for(uint32_t jr = 0; jr < 2; ++jr)
                    ROCWMMA_UNROLL
                for(uint32_t jk = 0; jk < KH; ++jk)
                {
                    const uint32_t ua = (mt * KT + kt) * GA::UnitsPerAtom + ((jk << 1) | jr);
                    const uint32_t ub = ((2 * mt + jr) * KT + kt) * GB::UnitsPerAtom + jk;
                    ROCWMMA_UNROLL
                    for(uint32_t s = 0; s < P; ++s)
                        b.x[ub * P + s] = a.x[ua * P + s];
                }
                return b;
            }
        };

        // B (BlockK x BlockN) -> A (BlockN x BlockK): the inverse permutation.
        template <uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT,
                  typename DataLayoutT>
        struct ApplyTranspose<fragment<matrix_b, BlockM, BlockN, BlockK, DataT, DataLayoutT>>
        {
            using FragB = fragment<matrix_b, BlockM, BlockN, BlockK, DataT, DataLayoutT>;
            using Type  = fragment<matrix_a, BlockN, BlockM, BlockK, DataT,
                                  typename OrthogonalLayout<DataLayoutT>::type>;
            static_assert(BlockN % 16u == 0u,
                          "the transpose of a matrix_b fragment needs BlockN a multiple of 16");

            ROCWMMA_DEVICE static inline Type exec(FragB const& b)
            {
                using GA = typename Type::Geom;
                using GB = typename FragB::Geom;
                constexpr uint32_t KT = GA::AtomsMinor, P = GA::UnitSize;
                constexpr uint32_t KH = GB::UnitsPerAtom;
                Type               a;
                ROCWMMA_UNROLL
                for(uint32_t mt = 0; mt < GA::AtomsMajor; ++mt)
                    ROCWMMA_UNROLL
                for(uint32_t kt = 0; kt < KT; ++kt)
                    ROCWMMA_UNROLL
                for(uint32_t jr = 0; jr < 2; ++jr)
                    ROCWMMA_UNROLL
                for(uint32_t jk = 0; jk < KH; ++jk)
                {
                    const uint32_t ua = (mt * KT + kt) * GA::UnitsPerAtom + ((jk << 1) | jr);
                    const uint32_t ub = ((2 * mt + jr) * KT + kt) * GB::UnitsPerAtom + jk;
                    ROCWMMA_UNROLL
                    for(uint32_t s = 0; s < P; ++s)
                        a.x[ua * P + s] = b.x[ub * P + s];
                }
                return a;
            }
        };

        template <typename FragT, typename NewDataLayoutT>
        struct ApplyDataLayout;

        template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK,
                  typename DataT, typename DataLayoutT, typename NewDataLayoutT>
        struct ApplyDataLayout<fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>,
                               NewDataLayoutT>
        {
            using FragT = fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>;
            using Type  = fragment<MatrixT, BlockM, BlockN, BlockK, DataT, NewDataLayoutT>;

            ROCWMMA_DEVICE static inline Type const& exec(FragT const& frag)
            {
                return reinterpret_cast<Type const&>(frag);
            }
        };
    } // namespace detail

    template <typename FragT>
    using ApplyTranspose_t = typename detail::ApplyTranspose<stdx::decay_t<FragT>>::Type;

    template <typename FragT, typename NewDataLayoutT>
    using ApplyDataLayout_t =
        typename detail::ApplyDataLayout<stdx::decay_t<FragT>, NewDataLayoutT>::Type;

    template <typename FragT>
    ROCWMMA_DEVICE static inline decltype(auto) applyTranspose(FragT&& frag)
    {
        return detail::ApplyTranspose<stdx::decay_t<FragT>>::exec(frag);
    }

    template <typename DataLayoutT, uint32_t WaveCount = 1, typename FragT>
    ROCWMMA_DEVICE static inline decltype(auto) applyDataLayout(FragT&& frag)
    {
        return detail::ApplyDataLayout<stdx::decay_t<FragT>, DataLayoutT>::exec(frag);
    }

    // Fragment property accessors used by kernels (rocWMMA internal/accessors.hpp:33-91).
    template <typename FragT>
    struct GetIOShape
    {
        using F = stdx::decay_t<FragT>;
        static constexpr uint32_t BlockHeight = F::height();
        static constexpr uint32_t BlockWidth  = F::width();
        static constexpr uint32_t BlockDim    = F::blockDim();
        static constexpr uint32_t KDim        = F::kDim();
    };
    template <typename FragT>
    using GetIOShape_t = GetIOShape<FragT>;

    template <typename FragT>
    using GetDataType_t = typename stdx::decay_t<FragT>::element_type;

    // GetDataLayout_t<FragT>: the 1-D address map of the fragment's memory layout
    // (rocWMMA internal/accessors_impl.hpp:107-118): fromMatrixCoord((row, col), ld) is the
    // element offset row * ld + col for row_major, col * ld + row for col_major
    // (internal/mapping_util_impl.hpp:142-150).  Kernels use it to step through matrices in
    // units of fragments (samples/perf_hgemm.cpp:371-377, 558-571).
    namespace detail
    {
        template <typename FragT>
        struct GetDataLayout;
        template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK,
                  typename DataT, typename DataLayoutT>
        struct GetDataLayout<fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>>
        {
            static_assert(!stdx::is_same<DataLayoutT, void>::value,
                          "the fragment has no compile-time memory layout");
            using type = DataSpace<DataLayoutT>;
        };
    } // namespace detail
    template <typename FragT>
    using GetDataLayout_t = typename detail::GetDataLayout<stdx::decay_t<FragT>>::type;
} // namespace rocwmma

#endif // ROCWMMA_B200_TRANSFORMS_API_HPP
