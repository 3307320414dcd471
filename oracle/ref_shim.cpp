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

// gemm_CPU with natural leading dimensions, C and D row-major.  dtype codes:
// 0 f16, 1 bf16 (inputs only), 3 i8, 4 f32, 6 f64, 7 i32.
int ref_gemm(int in_t, int out_t, uint32_t m, uint32_t n, uint32_t k, void const* a,
             void const* b, void const* c, void* d, double alpha, double beta, int layoutA,
             int layoutB)
{
    if(in_t == 0 && out_t == 4)
        run_layout<_Float16, float, float>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);
    else if(in_t == 0 && out_t == 0)
        run_layout<_Float16, _Float16, float>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);
    else if(in_t == 1 && out_t == 4)
        run_layout<bf16_t, float, float>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);
    else if(in_t == 3 && out_t == 7)
        run_layout<int8_t, int32_t, int32_t>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);
    else if((in_t == 4 || in_t == 5) && out_t == 4)
        run_layout<float, float, float>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);
    else if(in_t == 6 && out_t == 6)
        run_layout<double, double, double>(layoutA, layoutB, m, n, k, a, b, c, d, alpha, beta);
    else
        return -1;
    return 0;
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
