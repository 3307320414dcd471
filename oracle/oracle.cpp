// CPU oracle for the matrix-multiply-accumulate hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, on the host, the arithmetic of
// rocWMMA's own CPU reference so that the CUDA kernels can be checked against
// it.  Nothing on the product path may call into it: only the test-suite, the
// smoke check and the CPU-baseline leg of the benchmark do.
//
// What is restated, and from where (paths inside the rocWMMA source tree):
//   * GEMM           test/reference_impl.hpp:36-81  (== samples/common.hpp:297-342)
//   * DLRM forward   test/reference_impl.hpp:83-119
//   * DLRM backward  test/reference_impl.hpp:121-179
//   * GEMV           samples/simple_sgemv.cpp:46-67
//   * error metric   samples/common.hpp:345-416
//
// Parity pins: the DLRM functions are checked against the reference's stored
// known-answer vectors (test/dlrm/data/*), and every function is checked
// bit-for-bit against the reference's own code compiled from its sources (see
// the Makefile in this directory).  Two conversions have no pin in the
// reference because they live in HIP headers that are not part of its tree
// (float -> e4m3 and float -> bf16 encoding): for those, parity is unpinned;
// this file defines round-to-nearest-even with saturation to the largest
// finite value, and the CUDA side uses the same rule.
//
// Build: g++ -O3 -std=c++17 -fopenmp -ffp-contract=off -shared -fPIC
// (-ffp-contract=off keeps "acc += a*b" as a rounded multiply followed by a
// rounded add, which is what the reference's un-fused host loop computes).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <omp.h>
#include <vector>

namespace
{
    // ---- dtype codes shared with the C ABI of the CUDA library -------------
    enum DType : int
    {
        DT_F16  = 0,
        DT_BF16 = 1,
        DT_E4M3 = 2,
        DT_I8   = 3,
        DT_F32  = 4,
        DT_XF32 = 5, // fp32 storage whose low 13 mantissa bits are zero
        DT_F64  = 6,
        DT_I32  = 7,
        DT_E5M2 = 8,
    };

    enum Layout : int
    {
        ROW_MAJOR = 0,
        COL_MAJOR = 1
    };

    // ---- scalar storage types ----------------------------------------------
    struct bf16_t
    {
        uint16_t bits;
    };
    struct e4m3_t
    {
        uint8_t bits;
    };
    struct e5m2_t
    {
        uint8_t bits;
    };

    inline float bits_to_float(uint32_t u)
    {
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
    inline uint32_t float_to_bits(float f)
    {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        return u;
    }

    inline float decode(bf16_t v)
    {
        return bits_to_float(uint32_t(v.bits) << 16);
    }

    // OCP e4m3 ("fn" flavour): bias 7, no infinity, S.1111.111 is NaN, max 448.
    inline float decode(e4m3_t v)
    {
        uint32_t s = v.bits >> 7, e = (v.bits >> 3) & 0xF, m = v.bits & 7;
        float    r;
        if(e == 0xF && m == 7)
            r = std::numeric_limits<float>::quiet_NaN();
        else if(e == 0)
            r = std::ldexp(float(m), -9); // subnormal: m/8 * 2^-6
        else
            r = std::ldexp(1.0f + float(m) / 8.0f, int(e) - 7);
        return s ? -r : r;
    }

    // OCP e5m2: bias 15, two mantissa bits, infinities and NaNs as in IEEE -- the upper
    // byte of a binary16 number.
    inline float decode(e5m2_t v)
    {
        uint32_t s = v.bits >> 7, e = (v.bits >> 2) & 0x1F, m = v.bits & 3;
        float    r;
        if(e == 0x1F)
            r = m ? std::numeric_limits<float>::quiet_NaN()
                  : std::numeric_limits<float>::infinity();
        else if(e == 0)
            r = std::ldexp(float(m), -16); // subnormal: m/4 * 2^-14
        else
            r = std::ldexp(1.0f + float(m) / 4.0f, int(e) - 15);
        return s ? -r : r;
    }

    inline bf16_t encode_bf16(float f)
    {
        uint32_t u = float_to_bits(f);
        if((u & 0x7fffffffu) > 0x7f800000u)
            return bf16_t{uint16_t((u >> 16) | 0x40)}; // quiet NaN
        u += 0x7fffu + ((u >> 16) & 1u); // round to nearest even
        return bf16_t{uint16_t(u >> 16)};
    }

    // float -> e4m3, round to nearest even, saturating to +-448.
    inline e4m3_t encode_e4m3(float f)
    {
        uint32_t u    = float_to_bits(f);
        uint8_t  sign = uint8_t((u >> 24) & 0x80);
        float    a    = std::fabs(f);
        if(std::isnan(f))
            return e4m3_t{uint8_t(sign | 0x7f)};
        if(a >= 448.0f)
            return e4m3_t{uint8_t(sign | 0x7e)};
        if(a < std::ldexp(1.0f, -10)) // below half of the smallest subnormal (2^-9)
            return e4m3_t{sign};
        int   ex;
        (void)std::frexp(a, &ex); // a = fr * 2^ex, fr in [0.5,1)
        int   e    = std::max(ex - 1, -6); // exponent of the leading bit, clamped to subnormal range
        float q    = std::ldexp(a, 3 - e); // value in units of the last kept bit
        float r    = std::nearbyint(q); // current rounding mode is round-to-nearest-even
        int   mant = int(r);
        if(mant == 16)
        {
            mant = 8;
            e += 1;
        }
        uint8_t bits;
        if(mant < 8) // subnormal (only reachable when e == -6)
            bits = uint8_t(mant);
        else
            bits = uint8_t(((e + 7) << 3) | (mant - 8));
        return e4m3_t{uint8_t(sign | bits)};
    }

    // float -> e5m2, round to nearest even, saturating to +-57344 (no infinities are
    // produced, like the e4m3 encoder).
    inline e5m2_t encode_e5m2(float f)
    {
        uint32_t u    = float_to_bits(f);
        uint8_t  sign = uint8_t((u >> 24) & 0x80);
        float    a    = std::fabs(f);
        if(std::isnan(f))
            return e5m2_t{uint8_t(sign | 0x7f)};
        if(a >= 57344.0f)
            return e5m2_t{uint8_t(sign | 0x7b)};
        if(a < std::ldexp(1.0f, -17)) // below half of the smallest subnormal (2^-16)
            return e5m2_t{sign};
        int ex;
        (void)std::frexp(a, &ex);
        int   e    = std::max(ex - 1, -14);
        float q    = std::ldexp(a, 2 - e);
        int   mant = int(std::nearbyint(q));
        if(mant == 8)
        {
            mant = 4;
            e += 1;
        }
        uint8_t bits;
        if(mant < 4)
            bits = uint8_t(mant);
        else
            bits = uint8_t(((e + 15) << 2) | (mant - 4));
        return e5m2_t{uint8_t(sign | bits)};
    }

    // bfloat16 as a COMPUTE type: every operation is carried out in float and rounded back
    // to bfloat16 (round to nearest even), which is how the host bfloat16 class used by the
    // reference (hip_bfloat16, outside the reference tree) behaves.
    struct bf16c_t
    {
        bf16_t v;
        bf16c_t() = default;
        bf16c_t(float f)
            : v(encode_bf16(f))
        {
        }
        operator float() const
        {
            return decode(v);
        }
        bf16c_t& operator+=(bf16c_t o)
        {
            *this = bf16c_t(float(*this) + float(o));
            return *this;
        }
    };
    inline bf16c_t operator*(bf16c_t a, bf16c_t b)
    {
        return bf16c_t(float(a) * float(b));
    }
    inline bf16c_t operator+(bf16c_t a, bf16c_t b)
    {
        return bf16c_t(float(a) + float(b));
    }

    template <typename T>
    struct Conv;
    template <>
    struct Conv<_Float16>
    {
        static float    up(_Float16 v) { return static_cast<float>(v); }
        static _Float16 down(float v) { return static_cast<_Float16>(v); }
    };
    template <>
    struct Conv<bf16_t>
    {
        static float  up(bf16_t v) { return decode(v); }
        static bf16_t down(float v) { return encode_bf16(v); }
    };
    template <>
    struct Conv<e4m3_t>
    {
        static float  up(e4m3_t v) { return decode(v); }
        static e4m3_t down(float v) { return encode_e4m3(v); }
    };
    template <>
    struct Conv<e5m2_t>
    {
        static float  up(e5m2_t v) { return decode(v); }
        static e5m2_t down(float v) { return encode_e5m2(v); }
    };
    template <>
    struct Conv<float>
    {
        static float up(float v) { return v; }
        static float down(float v) { return v; }
    };
    template <>
    struct Conv<double>
    {
        static double up(double v) { return v; }
        static double down(double v) { return v; }
    };
    template <>
    struct Conv<int8_t>
    {
        static int32_t up(int8_t v) { return int32_t(v); }
        static int8_t  down(int32_t v) { return int8_t(v); }
    };
    template <>
    struct Conv<int32_t>
    {
        static int32_t up(int32_t v) { return v; }
        static int32_t down(int32_t v) { return v; }
    };

    inline size_t idx(int layout, size_t row, size_t col, size_t ld)
    {
        return layout == ROW_MAJOR ? row * ld + col : col * ld + row;
    }

    // ------------------------------------------------------------------------
    // GEMM, literal form: for every (i,j) a ComputeT accumulator starts at 0 and
    // takes the products in ascending k order; the result is
    // OutputT(alpha*acc + beta*ComputeT(c)).  (test/reference_impl.hpp:66-80)
    // ------------------------------------------------------------------------
    template <typename InT, typename OutT, typename CompT>
    void gemm_literal(uint32_t m, uint32_t n, uint32_t k, InT const* a, InT const* b,
                      OutT const* c, OutT* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                      uint32_t ldd, CompT alpha, CompT beta, int la, int lb, int lc, int ldl)
    {
#pragma omp parallel for
        for(int64_t i = 0; i < int64_t(m); ++i)
        {
            for(uint32_t j = 0; j < n; ++j)
            {
                CompT acc = CompT(0);
                for(uint32_t h = 0; h < k; ++h)
                {
                    // Every operation is rounded to CompT on its own (named temporaries: a
                    // 16-bit CompT must not keep a wider intermediate).
                    const CompT p = CompT(Conv<InT>::up(a[idx(la, i, h, lda)]))
                                    * CompT(Conv<InT>::up(b[idx(lb, h, j, ldb)]));
                    acc += p;
                }
                const CompT cv = CompT(Conv<OutT>::up(c[idx(lc, i, j, ldc)]));
                const CompT t1 = alpha * acc;
                const CompT t2 = beta * cv;
                const CompT r  = t1 + t2;
                d[idx(ldl, i, j, ldd)] = Conv<OutT>::down(r);
            }
        }
    }

    // ------------------------------------------------------------------------
    // GEMM, blocked form.  Same arithmetic, same order per output element: each
    // (i,j) accumulator still receives its products one by one in ascending k,
    // so the result is bit-identical to the literal form.  The only change is
    // that a strip of j values advances together through k, which lets the
    // compiler use SIMD lanes across j (never across k).
    // ------------------------------------------------------------------------
    template <typename InT, typename OutT, typename CompT>
    void gemm_blocked(uint32_t m, uint32_t n, uint32_t k, InT const* a, InT const* b,
                      OutT const* c, OutT* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                      uint32_t ldd, CompT alpha, CompT beta, int la, int lb, int lc, int ldl)
    {
        // B as ComputeT, k-major rows so that a strip of j is contiguous.
        std::vector<CompT> bw(size_t(k) * n);
#pragma omp parallel for
        for(int64_t h = 0; h < int64_t(k); ++h)
            for(uint32_t j = 0; j < n; ++j)
                bw[size_t(h) * n + j] = CompT(Conv<InT>::up(b[idx(lb, h, j, ldb)]));

        constexpr uint32_t JB = 256;
#pragma omp parallel
        {
            std::vector<CompT> arow(k);
            CompT              acc[JB];
#pragma omp for schedule(dynamic, 1)
            for(int64_t i = 0; i < int64_t(m); ++i)
            {
                for(uint32_t h = 0; h < k; ++h)
                    arow[h] = CompT(Conv<InT>::up(a[idx(la, i, h, lda)]));
                for(uint32_t j0 = 0; j0 < n; j0 += JB)
                {
                    uint32_t jn = std::min(JB, n - j0);
                    for(uint32_t jj = 0; jj < jn; ++jj)
                        acc[jj] = CompT(0);
                    for(uint32_t h = 0; h < k; ++h)
                    {
                        CompT        av = arow[h];
                        CompT const* br = &bw[size_t(h) * n + j0];
                        for(uint32_t jj = 0; jj < jn; ++jj)
                        {
                            const CompT p = av * br[jj];
                            acc[jj] += p;
                        }
                    }
                    for(uint32_t jj = 0; jj < jn; ++jj)
                    {
                        uint32_t j  = j0 + jj;
                        const CompT cv = CompT(Conv<OutT>::up(c[idx(lc, i, j, ldc)]));
                        const CompT t1 = alpha * acc[jj];
                        const CompT t2 = beta * cv;
                        const CompT r  = t1 + t2;
                        d[idx(ldl, i, j, ldd)] = Conv<OutT>::down(r);
                    }
                }
            }
        }
    }

    template <typename InT, typename OutT, typename CompT>
    int gemm_run(int literal, uint32_t m, uint32_t n, uint32_t k, void const* a, void const* b,
                 void const* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                 double alpha, double beta, int la, int lb, int lc, int ldl)
    {
        auto fn = literal ? gemm_literal<InT, OutT, CompT> : gemm_blocked<InT, OutT, CompT>;
        fn(m, n, k, static_cast<InT const*>(a), static_cast<InT const*>(b),
           static_cast<OutT const*>(c), static_cast<OutT*>(d), lda, ldb, ldc, ldd, CompT(alpha),
           CompT(beta), la, lb, lc, ldl);
        return 0;
    }

    // ------------------------------------------------------------------------
    // DLRM dot interaction, forward (test/reference_impl.hpp:83-119).
    // input  [batch][m][k], output [batch][k + m(m-1)/2]:
    //   first k values = row 0 of the sample, then the strict lower triangle of
    //   X X^T in row-major (i, j<i) order; float accumulator, ascending k.
    // ------------------------------------------------------------------------
    template <typename T>
    void dlrm_fwd(T const* input, T* output, uint32_t m, uint32_t k, uint32_t batch)
    {
        size_t inStride  = size_t(m) * k;
        size_t outStride = size_t(m) * (m - 1) / 2 + k;
#pragma omp parallel for
        for(int64_t b = 0; b < int64_t(batch); ++b)
        {
            T const* x = input + b * inStride;
            T*       o = output + b * outStride;
            for(uint32_t i = 0; i < k; ++i)
                *o++ = x[i];
            for(uint32_t i = 0; i < m; ++i)
                for(uint32_t j = 0; j < i; ++j)
                {
                    float acc = 0.0f;
                    for(uint32_t h = 0; h < k; ++h)
                        acc += Conv<T>::up(x[i * k + h]) * Conv<T>::up(x[j * k + h]);
                    *o++ = Conv<T>::down(acc);
                }
        }
    }

    // ------------------------------------------------------------------------
    // DLRM dot interaction, backward (test/reference_impl.hpp:121-179).
    // upstream [batch][k + m(m-1)/2]; mlpGrad[b] = first k values; the rest is
    // unpacked into a symmetric m x m matrix G with zero diagonal, held in the
    // storage type T; grad[b] = G . X with a float accumulator over ascending h.
    // ------------------------------------------------------------------------
    template <typename T>
    void dlrm_bwd(T const* input, T const* upstream, T* mlpGrad, T* grad, uint32_t m, uint32_t k,
                  uint32_t batch)
    {
        size_t inStride = size_t(m) * k;
        size_t upStride = size_t(m) * (m - 1) / 2 + k;
#pragma omp parallel
        {
            std::vector<T> g(size_t(m) * m);
#pragma omp for
            for(int64_t b = 0; b < int64_t(batch); ++b)
            {
                T const* x  = input + b * inStride;
                T const* up = upstream + b * upStride;
                for(uint32_t j = 0; j < k; ++j)
                    mlpGrad[b * k + j] = up[j];
                T const* t = up + k;
                for(uint32_t i = 0; i < m; ++i)
                    for(uint32_t j = 0; j <= i; ++j)
                    {
                        if(i == j)
                            g[i * m + j] = Conv<T>::down(0.0f);
                        else
                        {
                            g[i * m + j] = *t;
                            g[j * m + i] = *t;
                            ++t;
                        }
                    }
                for(uint32_t i = 0; i < m; ++i)
                    for(uint32_t j = 0; j < k; ++j)
                    {
                        float acc = 0.0f;
                        for(uint32_t h = 0; h < m; ++h)
                            acc += Conv<T>::up(g[i * m + h]) * Conv<T>::up(x[h * k + j]);
                        grad[b * inStride + i * k + j] = Conv<T>::down(acc);
                    }
            }
        }
    }

    // GEMV (samples/simple_sgemv.cpp:46-67): A is column-major with lda = m,
    // y[i] = alpha * sum_h A[h*lda+i]*x[h] + beta*y[i], ascending h.
    template <typename T>
    void gemv(uint32_t m, uint32_t k, T const* a, T const* x, T const* yin, T* yout, T alpha,
              T beta, uint32_t lda)
    {
        // Row strips advance together through h; per-row order is unchanged.
        constexpr uint32_t IB = 512;
#pragma omp parallel for
        for(int64_t i0 = 0; i0 < int64_t(m); i0 += IB)
        {
            T        acc[IB];
            uint32_t in = std::min<uint32_t>(IB, m - uint32_t(i0));
            for(uint32_t ii = 0; ii < in; ++ii)
                acc[ii] = T(0);
            for(uint32_t h = 0; h < k; ++h)
            {
                T const* col = a + size_t(h) * lda + i0;
                T        xv  = x[h];
                for(uint32_t ii = 0; ii < in; ++ii)
                    acc[ii] += col[ii] * xv;
            }
            for(uint32_t ii = 0; ii < in; ++ii)
                yout[i0 + ii] = alpha * acc[ii] + beta * yin[i0 + ii];
        }
    }

    // Error metric of samples/common.hpp:345-416: max over elements of
    // |a-b| / (|a|+|b|+1) evaluated in double; returns -1 when an infinity and
    // -2 when a NaN shows up.
    template <typename T>
    double max_rel_err(T const* a, T const* b, size_t n)
    {
        double worst = 0.0;
        int    bad   = 0;
#pragma omp parallel for reduction(max : worst) reduction(max : bad)
        for(int64_t i = 0; i < int64_t(n); ++i)
        {
            double va  = double(Conv<T>::up(a[i]));
            double vb  = double(Conv<T>::up(b[i]));
            double num = std::fabs(va - vb);
            double den = std::fabs(va) + std::fabs(vb) + 1.0;
            if(std::isinf(num) || std::isinf(den))
                bad = std::max(bad, 1);
            else
            {
                double r = num / den;
                if(std::isnan(r))
                    bad = std::max(bad, 2);
                else
                    worst = std::max(worst, r);
            }
        }
        if(bad == 2)
            return -2.0;
        if(bad == 1)
            return -1.0;
        return worst;
    }
} // namespace

extern "C" {

// D = alpha*A*B + beta*C on the host for the type triple (input, output, compute) --
// rocWMMA's Ti / To / Tc (docs/api-reference/api-reference-guide.rst:80-153).  comp_t < 0
// selects the triple's usual compute type (float for floating-point inputs up to 32 bits,
// int32 for int8, double for double).  Returns 0, or -1 for a triple the reference's type
// table does not have.  `literal` != 0 selects the plain triple loop (slow; used to check
// the blocked form).
int oracle_gemm_ex(int in_t, int out_t, int comp_t, int literal, uint32_t m, uint32_t n,
                   uint32_t k, void const* a, void const* b, void const* c, void* d, uint32_t lda,
                   uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta,
                   int layoutA, int layoutB, int layoutC, int layoutD)
{
    if(comp_t < 0)
        comp_t = in_t == DT_I8 ? DT_I32 : in_t == DT_F64 ? DT_F64 : DT_F32;
#define ORACLE_CASE(I, O, C, IT, OT, CT)                                                    \
    if(in_t == I && out_t == O && comp_t == C)                                              \
        return gemm_run<IT, OT, CT>(literal, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha, \
                                    beta, layoutA, layoutB, layoutC, layoutD);
    ORACLE_CASE(DT_F16, DT_F32, DT_F32, _Float16, float, float)
    ORACLE_CASE(DT_F16, DT_F16, DT_F32, _Float16, _Float16, float)
    ORACLE_CASE(DT_F16, DT_F16, DT_F16, _Float16, _Float16, _Float16)
    ORACLE_CASE(DT_BF16, DT_F32, DT_F32, bf16_t, float, float)
    ORACLE_CASE(DT_BF16, DT_BF16, DT_F32, bf16_t, bf16_t, float)
    ORACLE_CASE(DT_BF16, DT_BF16, DT_BF16, bf16_t, bf16_t, bf16c_t)
    ORACLE_CASE(DT_E4M3, DT_F32, DT_F32, e4m3_t, float, float)
    ORACLE_CASE(DT_E4M3, DT_BF16, DT_F32, e4m3_t, bf16_t, float)
    ORACLE_CASE(DT_E5M2, DT_F32, DT_F32, e5m2_t, float, float)
    ORACLE_CASE(DT_E5M2, DT_BF16, DT_F32, e5m2_t, bf16_t, float)
    ORACLE_CASE(DT_I8, DT_I32, DT_I32, int8_t, int32_t, int32_t)
    ORACLE_CASE(DT_I8, DT_I8, DT_I32, int8_t, int8_t, int32_t)
    ORACLE_CASE(DT_F32, DT_F32, DT_F32, float, float, float)
    ORACLE_CASE(DT_XF32, DT_F32, DT_F32, float, float, float)
    ORACLE_CASE(DT_F64, DT_F64, DT_F64, double, double, double)
#undef ORACLE_CASE
    return -1;
}

int oracle_gemm(int in_t, int out_t, int literal, uint32_t m, uint32_t n, uint32_t k,
                void const* a, void const* b, void const* c, void* d, uint32_t lda, uint32_t ldb,
                uint32_t ldc, uint32_t ldd, double alpha, double beta, int layoutA, int layoutB,
                int layoutC, int layoutD)
{
    return oracle_gemm_ex(in_t, out_t, -1, literal, m, n, k, a, b, c, d, lda, ldb, ldc, ldd, alpha,
                          beta, layoutA, layoutB, layoutC, layoutD);
}

int oracle_dlrm_fwd(int dt, void const* input, void* output, uint32_t m, uint32_t k,
                    uint32_t batch)
{
    if(dt == DT_F16)
        dlrm_fwd(static_cast<_Float16 const*>(input), static_cast<_Float16*>(output), m, k, batch);
    else if(dt == DT_F32)
        dlrm_fwd(static_cast<float const*>(input), static_cast<float*>(output), m, k, batch);
    else
        return -1;
    return 0;
}

int oracle_dlrm_bwd(int dt, void const* input, void const* upstream, void* mlpGrad, void* grad,
                    uint32_t m, uint32_t k, uint32_t batch)
{
    if(dt == DT_F16)
        dlrm_bwd(static_cast<_Float16 const*>(input), static_cast<_Float16 const*>(upstream),
                 static_cast<_Float16*>(mlpGrad), static_cast<_Float16*>(grad), m, k, batch);
    else if(dt == DT_F32)
        dlrm_bwd(static_cast<float const*>(input), static_cast<float const*>(upstream),
                 static_cast<float*>(mlpGrad), static_cast<float*>(grad), m, k, batch);
    else
        return -1;
    return 0;
}

int oracle_gemv(int dt, uint32_t m, uint32_t k, void const* a, void const* x, void const* yin,
                void* yout, double alpha, double beta, uint32_t lda)
{
    if(dt == DT_F32)
        gemv(m, k, static_cast<float const*>(a), static_cast<float const*>(x),
             static_cast<float const*>(yin), static_cast<float*>(yout), float(alpha), float(beta),
             lda);
    else if(dt == DT_F64)
        gemv(m, k, static_cast<double const*>(a), static_cast<double const*>(x),
             static_cast<double const*>(yin), static_cast<double*>(yout), alpha, beta, lda);
    else
        return -1;
    return 0;
}

double oracle_max_rel_err(int dt, void const* a, void const* b, uint64_t n)
{
    switch(dt)
    {
    case DT_F16:
        return max_rel_err(static_cast<_Float16 const*>(a), static_cast<_Float16 const*>(b), n);
    case DT_BF16:
        return max_rel_err(static_cast<bf16_t const*>(a), static_cast<bf16_t const*>(b), n);
    case DT_E4M3:
        return max_rel_err(static_cast<e4m3_t const*>(a), static_cast<e4m3_t const*>(b), n);
    case DT_F32:
    case DT_XF32:
        return max_rel_err(static_cast<float const*>(a), static_cast<float const*>(b), n);
    case DT_F64:
        return max_rel_err(static_cast<double const*>(a), static_cast<double const*>(b), n);
    case DT_I32:
        return max_rel_err(static_cast<int32_t const*>(a), static_cast<int32_t const*>(b), n);
    case DT_I8:
        return max_rel_err(static_cast<int8_t const*>(a), static_cast<int8_t const*>(b), n);
    }
    return -3.0;
}

// Element-wise encoders/decoders, exposed so that the input generators and the
// tests use exactly the routines the GEMM above uses.
void oracle_encode_e4m3(float const* src, uint8_t* dst, uint64_t n)
{
#pragma omp parallel for
    for(int64_t i = 0; i < int64_t(n); ++i)
        dst[i] = encode_e4m3(src[i]).bits;
}
void oracle_decode_e4m3(uint8_t const* src, float* dst, uint64_t n)
{
#pragma omp parallel for
    for(int64_t i = 0; i < int64_t(n); ++i)
        dst[i] = decode(e4m3_t{src[i]});
}
void oracle_encode_e5m2(float const* src, uint8_t* dst, uint64_t n)
{
#pragma omp parallel for
    for(int64_t i = 0; i < int64_t(n); ++i)
        dst[i] = encode_e5m2(src[i]).bits;
}
void oracle_decode_e5m2(uint8_t const* src, float* dst, uint64_t n)
{
#pragma omp parallel for
    for(int64_t i = 0; i < int64_t(n); ++i)
        dst[i] = decode(e5m2_t{src[i]});
}
void oracle_encode_bf16(float const* src, uint16_t* dst, uint64_t n)
{
#pragma omp parallel for
    for(int64_t i = 0; i < int64_t(n); ++i)
        dst[i] = encode_bf16(src[i]).bits;
}
void oracle_decode_bf16(uint16_t const* src, float* dst, uint64_t n)
{
#pragma omp parallel for
    for(int64_t i = 0; i < int64_t(n); ++i)
        dst[i] = decode(bf16_t{src[i]});
}

int oracle_num_threads()
{
    return omp_get_max_threads();
}

// Sets the number of OpenMP threads later parallel regions of this process use (this
// library's and the reference build's: they share one OpenMP runtime).  A launcher may have
// exported OMP_NUM_THREADS=1 for every worker it starts; the timed CPU baseline must not
// inherit that.
void oracle_set_num_threads(int n)
{
    if(n >= 1)
        omp_set_num_threads(n);
}
} // extern "C"
