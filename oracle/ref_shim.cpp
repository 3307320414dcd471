// Builds the reference's OWN host code for this path into oracle/_ref/libref.so.
//
// TEST INFRASTRUCTURE ONLY (checker and reported CPU baseline; never on the
// product path).  No reference source is copied into this repository: the
// Makefile slices the host-only part of the reference files, where they lie in
// the mounted rocWMMA tree, into a scratch header inside oracle/_ref/ (ignored
// by git), compiles this file against it and deletes the scratch header.
//
//   REF_IMPL_SLICE  = test/reference_impl.hpp, lines 1-179 (gemm_CPU,
//                     dlrm_fwd_CPU, dlrm_bwd_CPU) + the closing brace/#endif.
//                     Its three #includes are neutralised: two by defining
//                     their include guards, one by the stand-in under shim/.
//   REF_GEMV_SLICE  = samples/simple_sgemv.cpp, lines 46-67 (sgemv_cpu_h).
//
// The rest of those files needs HIP and an AMD GPU and cannot be built here.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <sys/types.h>
#include <type_traits>

#define ROCWMMA_TEST_HIP_DEVICE_HPP
#define ROCWMMA_REFERENCE_HPP
#define __host__

namespace rocwmma
{
    struct row_major
    {
    };
    struct col_major
    {
    };
    using float32_t = float;
} // namespace rocwmma

#include REF_IMPL_SLICE

using rocwmma::float32_t;
#include REF_GEMV_SLICE

namespace
{
    using rocwmma::col_major;
    using rocwmma::row_major;

    struct bf16_t
    {
        uint16_t bits;
        bf16_t() = default;
        explicit operator float() const
        {
            uint32_t u = uint32_t(bits) << 16;
            float    f;
            __builtin_memcpy(&f, &u, 4);
            return f;
        }
    };

    // 8-bit floating-point inputs: storage plus the format-defined (exact) decoding, which
    // in the reference comes from HIP's fp8 header.  e4m3: bias 7, no infinity, max 448;
    // e5m2: the upper byte of a binary16 number.
    struct e4m3_t
    {
        uint8_t bits;
        e4m3_t() = default;
        explicit operator float() const
        {
            const uint32_t e = (bits >> 3) & 0xF, m = bits & 7;
            float          r;
            if(e == 0xF && m == 7)
                r = __builtin_nanf("");
            else if(e == 0)
                r = std::ldexp(float(m), -9);
            else
                r = std::ldexp(1.0f + float(m) / 8.0f, int(e) - 7);
            return (bits & 0x80) ? -r : r;
        }
    };
    struct e5m2_t
    {
        uint8_t bits;
        e5m2_t() = default;
        explicit operator float() const
        {
            const uint16_t h = uint16_t(uint16_t(bits) << 8);
            _Float16       v;
            __builtin_memcpy(&v, &h, 2);
            return float(v);
        }
    };

    template <typename InT, typename OutT, typename CompT, typename LA, typename LB>
    void run(uint32_t m, uint32_t n, uint32_t k, void const* a, void const* b, void const* c,
             void* d, double alpha, double beta)
    {
        rocwmma::gemm_CPU<InT, OutT, CompT, LA, LB, row_major, row_major>(
            m, n, k, static_cast<InT const*>(a), static_cast<InT const*>(b),
            static_cast<OutT const*>(c), static_cast<OutT*>(d), CompT(alpha), CompT(beta));
    }

    template <typename InT, typename OutT, typename CompT>
    void run_layout(int la, int lb, uint32_t m, uint32_t n, uint32_t k, void const* a,
                    void const* b, void const* c, void* d, double alpha, double beta)
    {
        if(la == 0 && lb == 0)
            run<InT, OutT, CompT, row_major, row_major>(m, n, k, a, b, c, d, alpha, beta);
        else if(la == 0 && lb == 1)
            run<InT, OutT, CompT, row_major, col_major>(m, n, k, a, b, c, d, alpha, beta);
        else if(la == 1 && lb == 0)
            run<InT, OutT, CompT, col_major, row_major>(m, n, k, a, b, c, d, alpha, beta);
        else
            run<InT, OutT, CompT, col_major, col_major>(m, n, k, a, b, c, d, alpha, beta);
    }
} // namespace

extern "C" {

// gemm_CPU with natural leading dimensions, C and D row-major, for the type triple
// (input, output, compute).  dtype codes: 0 f16, 1 bf16 (inputs only), 2 e4m3 and 8 e5m2
// (inputs only), 3 i8, 4 f32, 5 xf32 (float storage), 6 f64, 7 i32.  comp_t < 0: the
// triple's usual compute type.
int ref_gemm_ex(int in_t, int out_t, int comp_t, uint32_t m, uint32_t n, uint32_t k,
                void const* a, void const* b, void const* c, void* d, double alpha, double beta,
                int layoutA, int layoutB)
{
    if(comp_t < 0)
        comp_t = in_t == 3 ? 7 : in_t == 6 ? 6 : 4;
#define REF_CASE(I, O, C, IT, OT, CT)                                                   \
    if(in_t == I && out_t == O && comp_t == C)                                          \
    {                                                                                   \
        run_layout<IT, OT, CT>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);     \
        return 0;                                                                       \
    }
    REF_CASE(0, 4, 4, _Float16, float, float)
    REF_CASE(0, 0, 4, _Float16, _Float16, float)
    REF_CASE(0, 0, 0, _Float16, _Float16, _Float16)
    REF_CASE(1, 4, 4, bf16_t, float, float)
    REF_CASE(2, 4, 4, e4m3_t, float, float)
    REF_CASE(8, 4, 4, e5m2_t, float, float)
    REF_CASE(3, 7, 7, int8_t, int32_t, int32_t)
    REF_CASE(3, 3, 7, int8_t, int8_t, int32_t)
    REF_CASE(4, 4, 4, float, float, float)
    REF_CASE(5, 4, 4, float, float, float)
    REF_CASE(6, 6, 6, double, double, double)
#undef REF_CASE
    return -1;
}

int ref_gemm(int in_t, int out_t, uint32_t m, uint32_t n, uint32_t k, void const* a,
             void const* b, void const* c, void* d, double alpha, double beta, int layoutA,
             int layoutB)
{
    return ref_gemm_ex(in_t, out_t, -1, m, n, k, a, b, c, d, alpha, beta, layoutA, layoutB);
}

int ref_dlrm_fwd(int dt, void const* input, void* output, uint32_t m, uint32_t k, uint32_t batch)
{
    if(dt == 0)
        rocwmma::dlrm_fwd_CPU(static_cast<_Float16 const*>(input), static_cast<_Float16*>(output),
                              m, k, batch);
    else if(dt == 4)
        rocwmma::dlrm_fwd_CPU(static_cast<float const*>(input), static_cast<float*>(output), m, k,
                              batch);
    else
        return -1;
    return 0;
}

int ref_dlrm_bwd(int dt, void const* input, void const* upstream, void* mlpGrad, void* grad,
                 uint32_t m, uint32_t k, uint32_t batch)
{
    if(dt == 0)
        rocwmma::dlrm_bwd_CPU(static_cast<_Float16 const*>(input),
                              static_cast<_Float16 const*>(upstream),
                              static_cast<_Float16*>(mlpGrad), static_cast<_Float16*>(grad), m, k,
                              batch);
    else if(dt == 4)
        rocwmma::dlrm_bwd_CPU(static_cast<float const*>(input),
                              static_cast<float const*>(upstream), static_cast<float*>(mlpGrad),
                              static_cast<float*>(grad), m, k, batch);
    else
        return -1;
    return 0;
}

// sgemv_cpu_h: y (in/out) = alpha*A*x + beta*y, A column-major with lda = m.
int ref_sgemv(uint32_t m, uint32_t k, float const* a, float const* x, float* y, float alpha,
              float beta)
{
    sgemv_cpu_h(m, 1, k, a, x, y, alpha, beta);
    return 0;
}
}
