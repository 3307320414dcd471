// Scalar types of the fragment API on sm_100a.
//
// rocWMMA names (internal/types.hpp:47-112) are kept; they alias the CUDA
// storage types.  float16_t and hfloat16_t are the same type here (nvcc device
// code has no _Float16).  float8_t / bfloat8_t are the OCP e4m3 / e5m2 formats
// (rocWMMA internal/types.hpp:100-101), not the "fnuz" flavours.
// xfloat32_t follows rocWMMA internal/rocwmma_xfloat32.hpp:110-203: fp32
// storage whose low 13 mantissa bits are cleared; the default conversion from
// float TRUNCATES, round_up() rounds to nearest even.
#ifndef ROCWMMA_B200_TYPES_HPP
#define ROCWMMA_B200_TYPES_HPP

#include "config.hpp"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace rocwmma
{
    using float16_t  = __half;
    using hfloat16_t = __half;
    using bfloat16_t = __nv_bfloat16;
    using float8_t   = __nv_fp8_e4m3;
    using bfloat8_t  = __nv_fp8_e5m2;
    using float32_t  = float;
    using float64_t  = double;
    using int8_t     = ::int8_t;
    using uint8_t    = ::uint8_t;
    using int16_t    = ::int16_t;
    using int32_t    = ::int32_t;
    using uint32_t   = ::uint32_t;
    using int64_t    = ::int64_t;
    using uint64_t   = ::uint64_t;
    using index_t    = ::int32_t;

    struct xfloat32_t
    {
        float data;

        xfloat32_t() = default;
        ROCWMMA_HOST_DEVICE xfloat32_t(float f)
        {
            union
            {
                float    f32;
                uint32_t u32;
            } v{f};
            v.u32 &= 0xffffe000u; // truncate to 10 explicit mantissa bits
            data = v.f32;
        }
        ROCWMMA_HOST_DEVICE static xfloat32_t round_up(float f)
        {
            union
            {
                float    f32;
                uint32_t u32;
            } v{f};
            if((~v.u32 & 0x7f800000u) != 0u) // finite: round to nearest even on bit 13
                v.u32 += 0x00000fffu + ((v.u32 >> 13) & 1u);
            else if((v.u32 & 0x007fffffu) != 0u) // NaN stays NaN
                v.u32 |= 0x00002000u;
            return xfloat32_t(v.f32);
        }
        ROCWMMA_HOST_DEVICE operator float() const
        {
            return data;
        }
        ROCWMMA_HOST_DEVICE xfloat32_t& operator+=(xfloat32_t const& o)
        {
            *this = xfloat32_t(data + o.data);
            return *this;
        }
    };

    // The arithmetic type mma_sync accumulates in for a given input type
    // (rocWMMA docs/api-reference/api-reference-guide.rst:80-153).
    template <typename T>
    struct compute_type
    {
        using type = float;
    };
    template <>
    struct compute_type<int8_t>
    {
        using type = int32_t;
    };
    template <>
    struct compute_type<double>
    {
        using type = double;
    };
} // namespace rocwmma

// Mixed float/half arithmetic.  rocWMMA kernels scale fragments with expressions
// such as `alpha * fragAcc.x[i] + beta * fragC.x[i]` where alpha/beta are float
// and fragC holds 16-bit elements (samples/simple_hgemm.cpp:131-134).  With the
// CUDA 16-bit classes that expression is ambiguous (both operands convert to
// the other's type), so exact-match overloads computing in the wider type are
// provided.
#define ROCWMMA_MIXED_OPS(WIDE, NARROW)                                                        \
    ROCWMMA_HOST_DEVICE inline WIDE operator*(WIDE a, NARROW const& b) { return a * WIDE(float(b)); } \
    ROCWMMA_HOST_DEVICE inline WIDE operator*(NARROW const& a, WIDE b) { return WIDE(float(a)) * b; } \
    ROCWMMA_HOST_DEVICE inline WIDE operator+(WIDE a, NARROW const& b) { return a + WIDE(float(b)); } \
    ROCWMMA_HOST_DEVICE inline WIDE operator+(NARROW const& a, WIDE b) { return WIDE(float(a)) + b; } \
    ROCWMMA_HOST_DEVICE inline WIDE operator-(WIDE a, NARROW const& b) { return a - WIDE(float(b)); } \
    ROCWMMA_HOST_DEVICE inline WIDE operator-(NARROW const& a, WIDE b) { return WIDE(float(a)) - b; } \
    ROCWMMA_HOST_DEVICE inline WIDE operator/(WIDE a, NARROW const& b) { return a / WIDE(float(b)); } \
    ROCWMMA_HOST_DEVICE inline WIDE operator/(NARROW const& a, WIDE b) { return WIDE(float(a)) / b; }

ROCWMMA_MIXED_OPS(float, __half)
ROCWMMA_MIXED_OPS(float, __nv_bfloat16)
ROCWMMA_MIXED_OPS(double, __half)
ROCWMMA_MIXED_OPS(double, __nv_bfloat16)
#undef ROCWMMA_MIXED_OPS

#endif // ROCWMMA_B200_TYPES_HPP
