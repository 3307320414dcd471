// rocWMMA fragment API for NVIDIA B200 (sm_100a): a from-scratch implementation
// of the public device interface declared by rocWMMA's rocwmma.hpp:74-317 --
// fragment, fill_fragment, load_matrix_sync, store_matrix_sync, mma_sync,
// synchronize_workgroup -- with the same template parameters, argument order,
// row/col-major meaning and data types, built on warp-level mma.sync tensor-core
// instructions instead of AMD MFMA/WMMA builtins.
//
// Contracts kept from the reference:
//   * every function is warp-wide: all 32 lanes call it together;
//   * threads of a block are laid out (warps_x * 32, warps_y); the lane is
//     threadIdx.x % 32;
//   * element (r, c) of a tile is data[r*ldm + c] (row_major) or
//     data[c*ldm + r] (col_major); data may be global or shared memory;
//   * frag.x[i], frag[i], frag.num_elements, frag::element_type, *frag exist;
//   * accumulator fragments of equal BlockM x BlockN share one element map
//     whatever their data type or layout tag.
// Supported element types: float16_t, bfloat16_t, float8_t (e4m3), bfloat8_t
// (e5m2), int8_t, float32_t (full fp32 products through a 3-term TF32 split),
// xfloat32_t (single TF32 product), float64_t.  BlockM is a multiple of 16,
// BlockN of 8, BlockK of the instruction's K extent (see
// internal/frag_geometry.hpp).
#ifndef ROCWMMA_B200_API_HPP
#define ROCWMMA_B200_API_HPP

#include "internal/config.hpp"
#include "internal/constants.hpp"
#include "internal/coord.hpp"
#include "internal/frag_geometry.hpp"
#include "internal/frag_io.hpp"
#include "internal/mapping_util.hpp"
#include "internal/mma_sync_ptx.hpp"
#include "internal/types.hpp"

namespace rocwmma
{
    // Run-time layout selector for accumulator fragments declared without a
    // layout tag (rocwmma.hpp:106-110).
    enum layout_t : uint32_t
    {
        mem_row_major,
        mem_col_major
    };

    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT = void>
    class fragment
    {
    public:
        using Geom = detail::FragGeom<MatrixT, BlockM, BlockN, BlockK, DataT>;

        struct Traits
        {
            using PackedElementT   = typename detail::PackedOf<DataT>::type;
            using UnpackedElementT = DataT;
            constexpr static uint32_t Size = Geom::Size;
            constexpr static uint32_t PackedSize
                = Size * uint32_t(sizeof(DataT)) / uint32_t(sizeof(PackedElementT));
            using AccessT  = detail::VecT<UnpackedElementT, Size>;
            using StorageT = detail::VecT<PackedElementT, PackedSize>;
            static_assert(Size * sizeof(DataT) == PackedSize * sizeof(PackedElementT),
                          "fragment elements must fill whole 32-bit registers");
        };

        fragment()                            = default;
        fragment(const fragment&)             = default;
        fragment& operator=(const fragment&)  = default;

        ROCWMMA_DEVICE inline DataT&       operator[](uint32_t index) { return x[index]; }
        ROCWMMA_DEVICE inline DataT const& operator[](uint32_t index) const { return x[index]; }
        ROCWMMA_DEVICE inline typename Traits::StorageT&       operator*() { return mStorage; }
        ROCWMMA_DEVICE inline typename Traits::StorageT const& operator*() const { return mStorage; }

        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t height() { return Geom::Height; }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t width() { return Geom::Width; }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t blockDim() { return Geom::BlockDim; }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t kDim() { return Geom::KDim; }
        ROCWMMA_HOST_DEVICE constexpr static inline uint32_t size() { return Geom::Size; }

        union
        {
            typename Traits::StorageT mStorage; // 32-bit registers as the tensor core reads them
            typename Traits::AccessT  mAccess; // one entry per element
            DataT                     x[Traits::Size]; // nvcuda::wmma-style element access
        };

        constexpr static uint32_t num_elements = Traits::Size;
        using element_type                     = DataT;
    };

    // ---- fill_fragment (rocwmma.hpp:211-219) ------------------------------------
    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        fill_fragment(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                      DataT                                                          value)
    {
        ROCWMMA_UNROLL
        for(uint32_t i = 0; i < frag.num_elements; ++i)
            frag.x[i] = value;
    }

    // ---- load_matrix_sync (rocwmma.hpp:229-253) ---------------------------------
    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        load_matrix_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>& frag,
                         const DataT*                                                   data,
                         uint32_t                                                       ldm)
    {
        static_assert(!stdx::is_same<DataLayoutT, void>::value,
                      "Must provide layout information. Either statically assign data layout in "
                      "fragment declaration or use the run-time function overload.");
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geom;
        detail::UnitIO<Geom, DataLayoutT>::loadRange(frag.x, data, ldm, 0u, Geom::Units);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT>
    ROCWMMA_DEVICE inline void
        load_matrix_sync(fragment<MatrixT, BlockM, BlockN, BlockK, DataT>& frag,
                         const DataT*                                      data,
                         uint32_t                                          ldm,
                         layout_t                                          layout)
    {
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT>::Geom;
        if(layout == layout_t::mem_row_major)
            detail::UnitIO<Geom, row_major>::loadRange(frag.x, data, ldm, 0u, Geom::Units);
        else
            detail::UnitIO<Geom, col_major>::loadRange(frag.x, data, ldm, 0u, Geom::Units);
    }

    // ---- store_matrix_sync (rocwmma.hpp:263-288) --------------------------------
    template <typename MatrixT,
              uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename DataT,
              typename DataLayoutT>
    ROCWMMA_DEVICE inline void
        store_matrix_sync(DataT*                                                               data,
                          fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT> const& frag,
                          uint32_t                                                             ldm)
    {
        static_assert(!stdx::is_same<DataLayoutT, void>::value,
                      "Must provide data layout. Either statically assign data layout in "
                      "fragment declaration or use the run-time function overload.");
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT, DataLayoutT>::Geom;
        detail::UnitIO<Geom, DataLayoutT>::storeRange(data, frag.x, ldm, 0u, Geom::Units);
    }

    template <typename MatrixT, uint32_t BlockM, uint32_t BlockN, uint32_t BlockK, typename DataT>
    ROCWMMA_DEVICE inline void
        store_matrix_sync(DataT*                                                  data,
                          fragment<MatrixT, BlockM, BlockN, BlockK, DataT> const& frag,
                          uint32_t                                                ldm,
                          layout_t                                                layout)
    {
        using Geom = typename fragment<MatrixT, BlockM, BlockN, BlockK, DataT>::Geom;
        if(layout == layout_t::mem_row_major)
            detail::UnitIO<Geom, row_major>::storeRange(data, frag.x, ldm, 0u, Geom::Units);
        else
            detail::UnitIO<Geom, col_major>::storeRange(data, frag.x, ldm, 0u, Geom::Units);
    }

    // ---- mma_sync (rocwmma.hpp:300-314): d = a * b + c ---------------------------
    // c and d may be the same object.  The layout tags of a, b, c, d do not
    // change the arithmetic.  Products are accumulated over K inside the call in
    // ComputeT-or-wider precision: fp32 for 16-bit accumulator types.
    namespace detail
    {
        ROCWMMA_DEVICE inline uint32_t f2u(float f)
        {
            return __float_as_uint(f);
        }
        // Two e4m3/e5m2 bytes -> two fp16 values (exact), as one 32-bit register.
        template <typename Fp8T>
        ROCWMMA_DEVICE inline uint32_t fp8x2_to_half2(uint32_t packed, uint32_t hiPair)
        {
            const __nv_fp8x2_storage_t two
                = __nv_fp8x2_storage_t(hiPair ? (packed >> 16) : (packed & 0xffffu));
            const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
                two, stdx::is_same<Fp8T, __nv_fp8_e4m3>::value ? __NV_E4M3 : __NV_E5M2);
            return uint32_t(h.x) | (uint32_t(h.y) << 16);
        }
    } // namespace detail

    template <uint32_t BlockM,
              uint32_t BlockN,
              uint32_t BlockK,
              typename InputTA,
              typename InputTB,
              typename ComputeT,
              typename LayoutA,
              typename LayoutB,
              typename LayoutC,
              typename LayoutD>
    ROCWMMA_DEVICE inline void
        mma_sync(fragment<accumulator, BlockM, BlockN, BlockK, ComputeT, LayoutD>&       d,
                 fragment<matrix_a, BlockM, BlockN, BlockK, InputTA, LayoutA> const&     a,
                 fragment<matrix_b, BlockM, BlockN, BlockK, InputTB, LayoutB> const&     b,
                 fragment<accumulator, BlockM, BlockN, BlockK, ComputeT, LayoutC> const& c)
    {
        static_assert(stdx::is_same<InputTA, InputTB>::value,
                      "A and B fragments must hold the same data type");
        using InT   = InputTA;
        using GeomA = detail::FragGeom<matrix_a, BlockM, BlockN, BlockK, InT>;
        using GeomB = detail::FragGeom<matrix_b, BlockM, BlockN, BlockK, InT>;

        constexpr uint32_t MT = BlockM / 16u;
        constexpr uint32_t NT = BlockN / 8u;
        constexpr uint32_t KT = GeomA::AtomsMinor;
        constexpr uint32_t RA = GeomA::UnitsPerAtom; // 32-bit (or 64-bit) registers per A atom
        constexpr uint32_t RB = GeomB::UnitsPerAtom;

        constexpr bool Is16   = stdx::is_same<InT, float16_t>::value
                              || stdx::is_same<InT, bfloat16_t>::value;
        constexpr bool IsFp8  = stdx::is_same<InT, float8_t>::value
                               || stdx::is_same<InT, bfloat8_t>::value;
        constexpr bool IsI8   = stdx::is_same<InT, int8_t>::value;
        constexpr bool IsF32  = stdx::is_same<InT, float32_t>::value;
        constexpr bool IsXF32 = stdx::is_same<InT, xfloat32_t>::value;
        constexpr bool IsF64  = stdx::is_same<InT, float64_t>::value;
        static_assert(Is16 || IsFp8 || IsI8 || IsF32 || IsXF32 || IsF64,
                      "unsupported input type for mma_sync");

        ROCWMMA_UNROLL
        for(uint32_t mt = 0; mt < MT; ++mt)
        {
            ROCWMMA_UNROLL
            for(uint32_t nt = 0; nt < NT; ++nt)
            {
                const uint32_t ci = (mt * NT + nt) * 4u;

                if constexpr(IsF64)
                {
                    static_assert(stdx::is_same<ComputeT, float64_t>::value,
                                  "float64_t inputs accumulate in float64_t");
                    double acc[4] = {c.x[ci], c.x[ci + 1], c.x[ci + 2], c.x[ci + 3]};
                    ROCWMMA_UNROLL
                    for(uint32_t kt = 0; kt < KT; ++kt)
                    {
                        const uint32_t ai    = (mt * KT + kt) * RA;
                        const uint32_t bi    = (nt * KT + kt) * RB;
                        const double   ar[2] = {a.x[ai], a.x[ai + 1]};
                        const double   br[1] = {b.x[bi]};
                        detail::mma_atom_f64(acc, ar, br, acc);
                    }
                    ROCWMMA_UNROLL
                    for(uint32_t e = 0; e < 4; ++e)
                        d.x[ci + e] = acc[e];
                }
                else if constexpr(IsI8)
                {
                    static_assert(stdx::is_same<ComputeT, int32_t>::value,
                                  "int8_t inputs accumulate in int32_t");
                    int32_t acc[4] = {c.x[ci], c.x[ci + 1], c.x[ci + 2], c.x[ci + 3]};
                    ROCWMMA_UNROLL
                    for(uint32_t kt = 0; kt < KT; ++kt)
                    {
                        const uint32_t ai = (mt * KT + kt) * RA;
                        const uint32_t bi = (nt * KT + kt) * RB;
                        if constexpr(GeomA::KA == 32u)
                        {
                            const uint32_t ar[4] = {a.mStorage[ai], a.mStorage[ai + 1],
                                                    a.mStorage[ai + 2], a.mStorage[ai + 3]};
                            const uint32_t br[2] = {b.mStorage[bi], b.mStorage[bi + 1]};
                            detail::mma_atom_s8_k32(acc, ar, br, acc);
                        }
                        else
                        {
                            const uint32_t ar[2] = {a.mStorage[ai], a.mStorage[ai + 1]};
                            const uint32_t br[1] = {b.mStorage[bi]};
                            detail::mma_atom_s8_k16(acc, ar, br, acc);
                        }
                    }
                    ROCWMMA_UNROLL
                    for(uint32_t e = 0; e < 4; ++e)
                        d.x[ci + e] = acc[e];
                }
                else if constexpr(Is16 && stdx::is_same<ComputeT, float16_t>::value
                                  && stdx::is_same<InT, float16_t>::value)
                {
                    // 16-bit accumulation requested: the tensor core accumulates in fp16.
                    uint32_t acc[2] = {c.mStorage[ci / 2u], c.mStorage[ci / 2u + 1u]};
                    ROCWMMA_UNROLL
                    for(uint32_t kt = 0; kt < KT; ++kt)
                    {
                        const uint32_t ai = (mt * KT + kt) * RA;
                        const uint32_t bi = (nt * KT + kt) * RB;
                        if constexpr(GeomA::KA == 16u)
                        {
                            const uint32_t ar[4] = {a.mStorage[ai], a.mStorage[ai + 1],
                                                    a.mStorage[ai + 2], a.mStorage[ai + 3]};
                            const uint32_t br[2] = {b.mStorage[bi], b.mStorage[bi + 1]};
                            detail::mma_atom_f16acc(acc, ar, br, acc);
                        }
                        else // K extent 8
                        {
                            const uint32_t ar[2] = {a.mStorage[ai], a.mStorage[ai + 1]};
                            const uint32_t br[1] = {b.mStorage[bi]};
                            detail::mma_atom_f16acc_k8(acc, ar, br, acc);
                        }
                    }
                    d.mStorage[ci / 2u]      = acc[0];
                    d.mStorage[ci / 2u + 1u] = acc[1];
                }
                else
                {
                    // fp32 accumulation (ComputeT float, or bfloat16_t carried through fp32
                    // as rocWMMA does for 16-bit compute types, internal/mfma_impl.hpp:101-156).
                    float acc[4] = {float(c.x[ci]), float(c.x[ci + 1]), float(c.x[ci + 2]),
                                    float(c.x[ci + 3])};
                    ROCWMMA_UNROLL
                    for(uint32_t kt = 0; kt < KT; ++kt)
                    {
                        const uint32_t ai = (mt * KT + kt) * RA;
                        const uint32_t bi = (nt * KT + kt) * RB;
                        if constexpr(Is16 && GeomA::KA == 16u)
                        {
                            const uint32_t ar[4] = {a.mStorage[ai], a.mStorage[ai + 1],
                                                    a.mStorage[ai + 2], a.mStorage[ai + 3]};
                            const uint32_t br[2] = {b.mStorage[bi], b.mStorage[bi + 1]};
                            detail::mma_atom(acc, ar, br, acc, InT{});
                        }
                        else if constexpr(Is16) // K extent 8
                        {
                            const uint32_t ar[2] = {a.mStorage[ai], a.mStorage[ai + 1]};
                            const uint32_t br[1] = {b.mStorage[bi]};
                            detail::mma_atom_k8(acc, ar, br, acc, InT{});
                        }
                        else if constexpr(IsFp8 && GeomA::KA == 32u)
                        {
                            const uint32_t ar[4] = {a.mStorage[ai], a.mStorage[ai + 1],
                                                    a.mStorage[ai + 2], a.mStorage[ai + 3]};
                            const uint32_t br[2] = {b.mStorage[bi], b.mStorage[bi + 1]};
                            detail::mma_atom(acc, ar, br, acc, InT{});
                        }
                        else if constexpr(IsFp8)
                        {
                            // K extent 16: each lane's four consecutive-K bytes of A and B are
                            // widened (exactly) to fp16 and fed to the fp16 instruction.  The
                            // instruction sees K in a permuted order, identically for A and B,
                            // which leaves every dot product unchanged.
                            const uint32_t ar[4]
                                = {detail::fp8x2_to_half2<InT>(a.mStorage[ai], 0),
                                   detail::fp8x2_to_half2<InT>(a.mStorage[ai + 1], 0),
                                   detail::fp8x2_to_half2<InT>(a.mStorage[ai], 1),
                                   detail::fp8x2_to_half2<InT>(a.mStorage[ai + 1], 1)};
                            const uint32_t br[2] = {detail::fp8x2_to_half2<InT>(b.mStorage[bi], 0),
                                                    detail::fp8x2_to_half2<InT>(b.mStorage[bi], 1)};
                            detail::mma_atom(acc, ar, br, acc, __half{});
                        }
                        else if constexpr(IsXF32 && GeomA::KA == 4u)
                        {
                            const uint32_t ar[2]
                                = {detail::f2u(a.x[ai].data), detail::f2u(a.x[ai + 1].data)};
                            const uint32_t br[1] = {detail::f2u(b.x[bi].data)};
                            detail::mma_atom_tf32_k4(acc, ar, br, acc);
                        }
                        else if constexpr(IsF32 && GeomA::KA == 4u)
                        {
                            uint32_t ah[2], al[2], bh[1], bl[1];
                            ROCWMMA_UNROLL
                            for(uint32_t r = 0; r < 2; ++r)
                            {
                                const float v = a.x[ai + r];
                                ah[r]         = detail::to_tf32(v);
                                al[r]         = detail::to_tf32(v - __uint_as_float(ah[r]));
                            }
                            {
                                const float v = b.x[bi];
                                bh[0]         = detail::to_tf32(v);
                                bl[0]         = detail::to_tf32(v - __uint_as_float(bh[0]));
                            }
                            detail::mma_atom_tf32_k4(acc, al, bh, acc);
                            detail::mma_atom_tf32_k4(acc, ah, bl, acc);
                            detail::mma_atom_tf32_k4(acc, ah, bh, acc);
                        }
                        else if constexpr(IsXF32)
                        {
                            const uint32_t ar[4]
                                = {detail::f2u(a.x[ai].data), detail::f2u(a.x[ai + 1].data),
                                   detail::f2u(a.x[ai + 2].data), detail::f2u(a.x[ai + 3].data)};
                            const uint32_t br[2]
                                = {detail::f2u(b.x[bi].data), detail::f2u(b.x[bi + 1].data)};
                            detail::mma_atom_tf32(acc, ar, br, acc);
                        }
                        else // IsF32: a = hi + lo with both parts TF32; drop only lo*lo
                        {
                            uint32_t ah[4], al[4], bh[2], bl[2];
                            ROCWMMA_UNROLL
                            for(uint32_t r = 0; r < 4; ++r)
                            {
                                const float v = a.x[ai + r];
                                ah[r]         = detail::to_tf32(v);
                                al[r]         = detail::to_tf32(v - __uint_as_float(ah[r]));
                            }
                            ROCWMMA_UNROLL
                            for(uint32_t r = 0; r < 2; ++r)
                            {
                                const float v = b.x[bi + r];
                                bh[r]         = detail::to_tf32(v);
                                bl[r]         = detail::to_tf32(v - __uint_as_float(bh[r]));
                            }
                            detail::mma_atom_tf32(acc, al, bh, acc);
                            detail::mma_atom_tf32(acc, ah, bl, acc);
                            detail::mma_atom_tf32(acc, ah, bh, acc);
                        }
                    }
                    ROCWMMA_UNROLL
                    for(uint32_t e = 0; e < 4; ++e)
                        d.x[ci + e] = ComputeT(acc[e]);
                }
            }
        }
    }

    // ---- synchronize_workgroup (rocwmma.hpp:317) ---------------------------------
    ROCWMMA_DEVICE inline void synchronize_workgroup()
    {
        __syncthreads();
    }

} // namespace rocwmma

#endif // ROCWMMA_B200_API_HPP
