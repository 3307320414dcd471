// C++ test-and-bench driver over the C ABI (include/rocwmma_b200.h + libb200wmma.so), in the
// shape of the reference's host programs: allocate, fill, two warm-up launches, N timed
// launches between events, throughput, validation against the CPU reference
// (samples/perf_hgemm.cpp:716-944 `gemm_test`, samples/simple_sgemv.cpp:157-270,
// samples/simple_dlrm.cpp:443-680), and the result table of the reference's GEMM test
// programs (test/gemm/gemm_kernel_base_impl.hpp:441-523: printHeader / printKernel).
//
//   bench_harness gemm [--in T] [--out T] [--m M] [--n N] [--k K] [--alpha A] [--beta B]
//                      [--layout-a row|col] [--layout-b row|col] [--simple] [--block 16|32]
//                      [--block-k K] [--check-rows R] [--warmup W] [--iters I]
//   bench_harness gemv [--type f32|f64] [--m M] [--k K] [--alpha A] [--beta B]
//   bench_harness dlrm [--bwd] [--m M] [--k K] [--batch B] [--check-samples S]
//
// T: f16 bf16 f8 bf8 i8 i32 f32 xf32 f64 (the reference's spellings, dataTypeToString).
// Validation uses the CPU oracle (liboracle.so), which is why this program lives with the
// tests.  Exit code 0 = PASSED, 1 = FAILED, 2+ = could not run.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_runtime.h>
#include <map>
#include <rocwmma_b200.h>
#include <string>
#include <vector>

extern "C" {
int    oracle_gemm_ex(int, int, int, int, uint32_t, uint32_t, uint32_t, void const*, void const*,
                      void const*, void*, uint32_t, uint32_t, uint32_t, uint32_t, double, double,
                      int, int, int, int);
int    oracle_dlrm_fwd(int, void const*, void*, uint32_t, uint32_t, uint32_t);
int    oracle_dlrm_bwd(int, void const*, void const*, void*, void*, uint32_t, uint32_t, uint32_t);
int    oracle_gemv(int, uint32_t, uint32_t, void const*, void const*, void const*, void*, double,
                   double, uint32_t);
double oracle_max_rel_err(int, void const*, void const*, uint64_t);
void   oracle_encode_bf16(float const*, uint16_t*, uint64_t);
void   oracle_encode_e4m3(float const*, uint8_t*, uint64_t);
void   oracle_encode_e5m2(float const*, uint8_t*, uint64_t);
}

#define CHECK_CUDA(expr)                                                                   \
    do                                                                                     \
    {                                                                                      \
        cudaError_t e = (expr);                                                            \
        if(e != cudaSuccess)                                                               \
        {                                                                                  \
            std::fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e), __LINE__); \
            std::exit(2);                                                                  \
        }                                                                                  \
    } while(0)

namespace
{
    struct TypeInfo
    {
        int         code;
        size_t      bytes;
        char const* name;
    };
    TypeInfo typeByName(std::string const& s)
    {
        static const std::map<std::string, TypeInfo> table = {
            {"f16", {B200WMMA_F16, 2, "f16"}},   {"bf16", {B200WMMA_BF16, 2, "bf16"}},
            {"f8", {B200WMMA_E4M3, 1, "f8"}},    {"bf8", {B200WMMA_E5M2, 1, "bf8"}},
            {"i8", {B200WMMA_I8, 1, "i8"}},      {"i32", {B200WMMA_I32, 4, "i32"}},
            {"f32", {B200WMMA_F32, 4, "f32"}},   {"xf32", {B200WMMA_XF32, 4, "xf32"}},
            {"f64", {B200WMMA_F64, 8, "f64"}}};
        auto it = table.find(s);
        if(it == table.end())
        {
            std::fprintf(stderr, "unknown type %s\n", s.c_str());
            std::exit(2);
        }
        return it->second;
    }

    // splitmix64: one value per index, so any element can be regenerated
    inline uint64_t mix(uint64_t z)
    {
        z += 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    inline float uniform(uint64_t seed, uint64_t i) // [-1, 1]
    {
        return float(double(mix(seed * 0x100000001B3ull + i) >> 11) / double(1ull << 53) * 2.0 - 1.0);
    }
    inline float normal(uint64_t seed, uint64_t i) // Box-Muller on two uniforms
    {
        const double u1 = (double(mix(seed * 7919ull + 2 * i) >> 11) + 1.0) / double(1ull << 53);
        const double u2 = double(mix(seed * 7919ull + 2 * i + 1) >> 11) / double(1ull << 53);
        return float(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
    }

    // `count` elements of type t: uniform [-1, 1] (ints: the full int8 range / small int32),
    // or N(0,1) when `gauss`; 8-bit floats are scaled so that the largest magnitude maps to
    // the format's maximum
    std::vector<uint8_t> fill(TypeInfo t, size_t count, uint64_t seed, bool gauss = false)
    {
        std::vector<uint8_t> out(count * t.bytes);
        std::vector<float>   f;
        auto value = [&](size_t i) { return gauss ? normal(seed, i) : uniform(seed, i); };
        switch(t.code)
        {
        case B200WMMA_I8:
            for(size_t i = 0; i < count; ++i)
                reinterpret_cast<int8_t*>(out.data())[i] = int8_t(int(mix(seed + i) % 256) - 128);
            break;
        case B200WMMA_I32:
            for(size_t i = 0; i < count; ++i)
                reinterpret_cast<int32_t*>(out.data())[i] = int32_t(mix(seed + i) % 201) - 100;
            break;
        case B200WMMA_F32:
            for(size_t i = 0; i < count; ++i)
                reinterpret_cast<float*>(out.data())[i] = value(i);
            break;
        case B200WMMA_XF32: // low 13 mantissa bits cleared (the reference's truncation)
            for(size_t i = 0; i < count; ++i)
            {
                float    v = value(i);
                uint32_t u;
                std::memcpy(&u, &v, 4);
                u &= 0xFFFFE000u;
                std::memcpy(out.data() + 4 * i, &u, 4);
            }
            break;
        case B200WMMA_F64:
            for(size_t i = 0; i < count; ++i)
                reinterpret_cast<double*>(out.data())[i] = double(value(i));
            break;
        default:
            f.resize(count);
            for(size_t i = 0; i < count; ++i)
                f[i] = value(i);
            if(t.code == B200WMMA_E4M3 || t.code == B200WMMA_E5M2)
            {
                float top = 0.f;
                for(float v : f)
                    top = std::max(top, std::fabs(v));
                const float scale = (t.code == B200WMMA_E4M3 ? 448.f : 57344.f) / top;
                for(float& v : f)
                    v *= scale;
                if(t.code == B200WMMA_E4M3)
                    oracle_encode_e4m3(f.data(), out.data(), count);
                else
                    oracle_encode_e5m2(f.data(), out.data(), count);
            }
            else if(t.code == B200WMMA_BF16)
                oracle_encode_bf16(f.data(), reinterpret_cast<uint16_t*>(out.data()), count);
            else // f16
                for(size_t i = 0; i < count; ++i)
                    reinterpret_cast<_Float16*>(out.data())[i] = _Float16(f[i]);
        }
        return out;
    }

    struct Args
    {
        std::map<std::string, std::string> kv;
        bool has(std::string const& k) const { return kv.count(k) != 0; }
        std::string str(std::string const& k, std::string const& d) const
        {
            auto it = kv.find(k);
            return it == kv.end() ? d : it->second;
        }
        double num(std::string const& k, double d) const
        {
            auto it = kv.find(k);
            return it == kv.end() ? d : atof(it->second.c_str());
        }
    };
    Args parse(int argc, char** argv, int first)
    {
        Args a;
        for(int i = first; i < argc; ++i)
        {
            std::string k = argv[i];
            if(k.rfind("--", 0) != 0)
            {
                std::fprintf(stderr, "unexpected argument %s\n", argv[i]);
                std::exit(2);
            }
            k = k.substr(2);
            if(i + 1 < argc && std::strncmp(argv[i + 1], "--", 2) != 0)
                a.kv[k] = argv[++i];
            else
                a.kv[k] = "1";
        }
        return a;
    }

    void* toDevice(std::vector<uint8_t> const& h)
    {
        void* d = nullptr;
        CHECK_CUDA(cudaMalloc(&d, std::max<size_t>(h.size(), 16)));
        CHECK_CUDA(cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice));
        return d;
    }

    // warm-ups, then `iters` launches between two events: milliseconds per launch
    template <typename F>
    double timeLaunches(F&& launch, int warmups, int iters)
    {
        for(int i = 0; i < warmups; ++i)
            if(int rc = launch())
            {
                std::fprintf(stderr, "launch failed: %s\n", b200wmma_status_string(rc));
                std::exit(3);
            }
        cudaEvent_t start, stop;
        CHECK_CUDA(cudaEventCreate(&start));
        CHECK_CUDA(cudaEventCreate(&stop));
        CHECK_CUDA(cudaEventRecord(start));
        for(int i = 0; i < iters; ++i)
            launch();
        CHECK_CUDA(cudaEventRecord(stop));
        CHECK_CUDA(cudaEventSynchronize(stop));
        float ms = 0;
        CHECK_CUDA(cudaEventElapsedTime(&ms, start, stop));
        if(int rc = b200wmma_check_device(nullptr, nullptr))
        {
            std::fprintf(stderr, "device check failed: %s\n", b200wmma_status_string(rc));
            std::exit(4);
        }
        return double(ms) / iters;
    }

    double tolerance(int inType, int outType)
    {
        double tol = 2e-3;
        switch(inType)
        {
        case B200WMMA_I8: tol = 0.0; break;
        case B200WMMA_E4M3:
        case B200WMMA_E5M2: tol = 1e-2; break;
        case B200WMMA_F32:
        case B200WMMA_XF32: tol = 1e-4; break;
        case B200WMMA_F64: tol = 1e-12; break;
        }
        // a bf16 result has 8 significant bits: two correct results may be one step apart
        if(outType == B200WMMA_BF16)
            tol = std::max(tol, 4e-3);
        return tol;
    }

    int runGemm(Args const& a)
    {
        const TypeInfo ti = typeByName(a.str("in", "f16"));
        const TypeInfo to = typeByName(a.str("out", ti.code == B200WMMA_I8     ? "i32"
                                                    : ti.code == B200WMMA_F64  ? "f64"
                                                    : ti.bytes == 2            ? ti.name
                                                                               : "f32"));
        const uint32_t m = uint32_t(a.num("m", 1024)), n = uint32_t(a.num("n", 1024)),
                       k = uint32_t(a.num("k", 1024));
        const bool   simple = a.has("simple");
        const int    block  = int(a.num("block", 16)), blockK = int(a.num("block-k", 0));
        const int    la     = a.str("layout-a", "row") == "row" ? B200WMMA_ROW_MAJOR : B200WMMA_COL_MAJOR;
        const int    lb     = a.str("layout-b", "col") == "row" ? B200WMMA_ROW_MAJOR : B200WMMA_COL_MAJOR;
        const bool   fp8    = ti.code == B200WMMA_E4M3 || ti.code == B200WMMA_E5M2;
        // 8-bit float inputs reach the format's maximum; the default alpha brings the results
        // back to O(100), where the reference's metric is a relative one
        const double alphaDefault = ti.code == B200WMMA_E4M3 ? 1.0 / 4096 : ti.code == B200WMMA_E5M2 ? 1.0 / 67108864 : 2.0;
        const double alpha = a.num("alpha", ti.code == B200WMMA_I8 ? 2 : alphaDefault);
        const double beta  = a.num("beta", ti.code == B200WMMA_I8 ? 1 : 2.0);
        const int    warm = int(a.num("warmup", 2)), iters = int(a.num("iters", 5));
        const uint32_t lda = la == B200WMMA_ROW_MAJOR ? k : m, ldb = lb == B200WMMA_ROW_MAJOR ? n : k;

        auto hA = fill(ti, size_t(m) * k, 1, fp8), hB = fill(ti, size_t(k) * n, 2, fp8);
        auto hC = fill(to, size_t(m) * n, 3);
        std::vector<uint8_t> hD(size_t(m) * n * to.bytes);
        void *dA = toDevice(hA), *dB = toDevice(hB), *dC = toDevice(hC), *dD = nullptr;
        CHECK_CUDA(cudaMalloc(&dD, hD.size()));
        CHECK_CUDA(cudaMemset(dD, 0xff, hD.size())); // NaN pattern: unwritten outputs show up

        auto launch = [&]() {
            if(simple)
                return b200wmma_gemm_simple_ex(ti.code, to.code, -1, m, n, k, dA, dB, dC, dD, lda,
                                               ldb, n, n, alpha, beta, la, lb, B200WMMA_ROW_MAJOR,
                                               block, blockK, nullptr);
            return b200wmma_gemm(ti.code, to.code, m, n, k, dA, dB, dC, dD, lda, ldb, n, n, alpha,
                                 beta, la, lb, nullptr);
        };
        const double ms     = timeLaunches(launch, warm, iters);
        const double gflops = 2.0 * m * n * k / 1e9;
        const double tflops = gflops / ms; // GFLOP / ms = TFLOP/s
        CHECK_CUDA(cudaMemcpy(hD.data(), dD, hD.size(), cudaMemcpyDeviceToHost));

        // CPU validation of the first `check-rows` rows (all rows by default)
        const uint32_t rows = uint32_t(std::min<double>(m, a.num("check-rows", m)));
        std::vector<uint8_t> ref(size_t(rows) * n * to.bytes);
        std::vector<uint8_t> aRows;
        void const*          aPtr = hA.data();
        uint32_t             ldaRef = lda;
        if(la == B200WMMA_COL_MAJOR && rows < m)
        {
            // first `rows` rows of a column-major A: k columns of `rows` values
            aRows.resize(size_t(rows) * k * ti.bytes);
            for(uint32_t h = 0; h < k; ++h)
                std::memcpy(aRows.data() + size_t(h) * rows * ti.bytes,
                            hA.data() + size_t(h) * m * ti.bytes, size_t(rows) * ti.bytes);
            aPtr   = aRows.data();
            ldaRef = rows;
        }
        if(oracle_gemm_ex(ti.code, to.code, -1, 0, rows, n, k, aPtr, hB.data(), hC.data(),
                          ref.data(), ldaRef, ldb, n, n, alpha, beta, la, lb, 0, 0)
           != 0)
        {
            std::fprintf(stderr, "the CPU reference has no such type pair\n");
            return 2;
        }
        const double err  = oracle_max_rel_err(to.code, hD.data(), ref.data(), uint64_t(rows) * n);
        const bool   pass = err >= 0.0 && err <= tolerance(ti.code, to.code);

        // peak for the efficiency column: nominal dense tensor throughput of a B200
        const double peak = ti.bytes == 1 ? 4500.0 : ti.bytes == 2 ? 2250.0 : ti.bytes == 4 ? 1125.0 : 40.0;
        const char*  comp = ti.code == B200WMMA_I8 ? "i32" : ti.code == B200WMMA_F64 ? "f64" : "f32";
        std::printf("TBlkX, TBlkY, BlkM, BlkN, BlkK, MatM, MatN, MatK, alpha, lda, ldb, beta, ldc, ldd, "
                    "LytA_LytB_LytC_LytD, Ti_To_Tc, elapsedMs, Problem Size(GFlops), TFlops/s, "
                    "Efficiency(%%), Result\n");
        if(simple)
            std::printf("128, 4, %d, %d, %d, ", block, block, blockK ? blockK : 16);
        else if(ti.code == B200WMMA_F64)
            std::printf("256, 1, 128, 128, 16, ");
        else
            std::printf("192, 1, 256, 256, %d, ", int(128 / ti.bytes));
        std::printf("%u, %u, %u, %g, %u, %u, %g, %u, %u, %s_%s_row_row, %s_%s_%s, %f, %f, %f, %f, %s\n",
                    m, n, k, alpha, lda, ldb, beta, n, n, la == B200WMMA_ROW_MAJOR ? "row" : "col",
                    lb == B200WMMA_ROW_MAJOR ? "row" : "col", ti.name, to.name, comp, ms, gflops,
                    tflops, 100.0 * tflops / peak, pass ? "PASSED" : "FAILED");
        std::printf("{\"kernel\": \"gemm\", \"ms\": %f, \"tflops\": %f, \"max_rel_err\": %g, "
                    "\"rows_checked\": %u, \"tolerance\": %g}\n",
                    ms, tflops, err, rows, tolerance(ti.code, to.code));
        cudaFree(dA), cudaFree(dB), cudaFree(dC), cudaFree(dD);
        return pass ? 0 : 1;
    }

    int runGemv(Args const& a)
    {
        const TypeInfo t = typeByName(a.str("type", "f32"));
        const uint32_t m = uint32_t(a.num("m", 4096)), k = uint32_t(a.num("k", 4096));
        const double   alpha = a.num("alpha", 2.1), beta = a.num("beta", 2.1);
        const int      warm = int(a.num("warmup", 2)), iters = int(a.num("iters", 5));
        auto hA = fill(t, size_t(m) * k, 11), hX = fill(t, k, 12), hY = fill(t, m, 13);
        std::vector<uint8_t> hOut(size_t(m) * t.bytes), ref(size_t(m) * t.bytes);
        void *dA = toDevice(hA), *dX = toDevice(hX), *dY = toDevice(hY), *dOut = nullptr;
        CHECK_CUDA(cudaMalloc(&dOut, hOut.size()));
        auto launch = [&]() {
            return b200wmma_gemv(t.code, m, k, dA, dX, dY, dOut, alpha, beta, m, nullptr);
        };
        const double ms = timeLaunches(launch, warm, iters);
        CHECK_CUDA(cudaMemcpy(hOut.data(), dOut, hOut.size(), cudaMemcpyDeviceToHost));
        oracle_gemv(t.code, m, k, hA.data(), hX.data(), hY.data(), ref.data(), alpha, beta, m);
        const bool   same  = std::memcmp(hOut.data(), ref.data(), hOut.size()) == 0;
        const double bytes = (double(m) * k + k + 2.0 * m) * t.bytes;
        std::printf("MatM, MatK, alpha, beta, lda, Ti, elapsedMs, GB/s, Result\n");
        std::printf("%u, %u, %g, %g, %u, %s, %f, %f, %s\n", m, k, alpha, beta, m, t.name, ms,
                    bytes / ms / 1e6, same ? "PASSED" : "FAILED");
        std::printf("{\"kernel\": \"gemv\", \"ms\": %f, \"gbs\": %f, \"bit_identical\": %s}\n", ms,
                    bytes / ms / 1e6, same ? "true" : "false");
        cudaFree(dA), cudaFree(dX), cudaFree(dY), cudaFree(dOut);
        return same ? 0 : 1;
    }

    int runDlrm(Args const& a)
    {
        const TypeInfo t   = typeByName("f16");
        const uint32_t m = uint32_t(a.num("m", 27)), k = uint32_t(a.num("k", 128)),
                       batch = uint32_t(a.num("batch", 1024));
        const bool     bwd   = a.has("bwd");
        const int      warm = int(a.num("warmup", 2)), iters = int(a.num("iters", 5));
        const uint32_t outLen = k + m * (m - 1) / 2;
        auto hX = fill(t, size_t(batch) * m * k, 21, true);
        auto hUp = fill(t, size_t(batch) * outLen, 22, true);
        void *dX = toDevice(hX), *dUp = toDevice(hUp), *dOut = nullptr, *dGrad = nullptr,
             *dMlp = nullptr;
        CHECK_CUDA(cudaMalloc(&dOut, size_t(batch) * outLen * 2));
        CHECK_CUDA(cudaMalloc(&dGrad, size_t(batch) * m * k * 2));
        CHECK_CUDA(cudaMalloc(&dMlp, size_t(batch) * k * 2));
        auto launch = [&]() {
            return bwd ? b200wmma_dlrm_bwd(B200WMMA_F16, dX, dUp, dGrad, dMlp, m, k, batch, nullptr)
                       : b200wmma_dlrm_fwd(B200WMMA_F16, dX, dOut, m, k, batch, nullptr);
        };
        const double   ms = timeLaunches(launch, warm, iters);
        const uint32_t s  = uint32_t(std::min<double>(batch, a.num("check-samples", batch)));
        double         err = 0.0;
        bool           exact = true;
        if(!bwd)
        {
            std::vector<uint8_t> got(size_t(s) * outLen * 2), ref(got.size());
            CHECK_CUDA(cudaMemcpy(got.data(), dOut, got.size(), cudaMemcpyDeviceToHost));
            oracle_dlrm_fwd(B200WMMA_F16, hX.data(), ref.data(), m, k, s);
            err = oracle_max_rel_err(B200WMMA_F16, got.data(), ref.data(), uint64_t(s) * outLen);
        }
        else
        {
            std::vector<uint8_t> grad(size_t(s) * m * k * 2), mlp(size_t(s) * k * 2),
                refGrad(grad.size()), refMlp(mlp.size());
            CHECK_CUDA(cudaMemcpy(grad.data(), dGrad, grad.size(), cudaMemcpyDeviceToHost));
            CHECK_CUDA(cudaMemcpy(mlp.data(), dMlp, mlp.size(), cudaMemcpyDeviceToHost));
            oracle_dlrm_bwd(B200WMMA_F16, hX.data(), hUp.data(), refMlp.data(), refGrad.data(), m, k,
                            s);
            err   = oracle_max_rel_err(B200WMMA_F16, grad.data(), refGrad.data(),
                                     uint64_t(s) * m * k);
            exact = std::memcmp(mlp.data(), refMlp.data(), mlp.size()) == 0;
        }
        const bool   pass  = exact && err >= 0.0 && err <= 2e-3;
        const double bytes = bwd ? double(batch) * (2.0 * m * k + outLen + k) * 2
                                 : double(batch) * (double(m) * k + outLen) * 2;
        std::printf("pass, m, k, batch, Ti, elapsedMs, GB/s, maxRelErr, Result\n");
        std::printf("%s, %u, %u, %u, f16, %f, %f, %g, %s\n", bwd ? "bwd" : "fwd", m, k, batch, ms,
                    bytes / ms / 1e6, err, pass ? "PASSED" : "FAILED");
        std::printf("{\"kernel\": \"dlrm_%s\", \"ms\": %f, \"gbs\": %f, \"max_rel_err\": %g, "
                    "\"samples_checked\": %u}\n",
                    bwd ? "bwd" : "fwd", ms, bytes / ms / 1e6, err, s);
        cudaFree(dX), cudaFree(dUp), cudaFree(dOut), cudaFree(dGrad), cudaFree(dMlp);
        return pass ? 0 : 1;
    }
} // namespace

int main(int argc, char** argv)
{
    if(argc < 2)
    {
        std::fprintf(stderr, "usage: bench_harness gemm|gemv|dlrm [--option value ...]\n");
        return 2;
    }
    const std::string what = argv[1];
    const Args        args = parse(argc, argv, 2);
    int               rc   = 2;
    if(what == "gemm")
        rc = runGemm(args);
    else if(what == "gemv")
        rc = runGemv(args);
    else if(what == "dlrm")
        rc = runDlrm(args);
    else
        std::fprintf(stderr, "unknown kernel family %s\n", what.c_str());
    b200wmma_shutdown();
    return rc;
}
