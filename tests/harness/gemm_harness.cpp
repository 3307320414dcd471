// C++ host driver over the C ABI, in the shape of the reference's sample drivers
// (samples/perf_hgemm.cpp:716-944 `gemm_test`: allocate, fill, launch with events around
// it, report TFLOP/s, validate against the CPU reference).  It shows what a C++ user of
// rocWMMA's samples links against here: include/rocwmma_b200.h + libb200wmma.so, plain
// CUDA runtime calls for memory.  Validation uses the CPU oracle (liboracle.so), which is
// why this program lives with the tests and not in the product.
//
//   gemm_harness <m> <n> <k> [alpha] [beta]     fp16 A row-major, fp16 B col-major, fp16 C/D
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <rocwmma_b200.h>
#include <vector>

extern "C" int    oracle_gemm(int, int, int, uint32_t, uint32_t, uint32_t, void const*, void const*,
                              void const*, void*, uint32_t, uint32_t, uint32_t, uint32_t, double,
                              double, int, int, int, int);
extern "C" double oracle_max_rel_err(int, void const*, void const*, uint64_t);

#define CHECK_CUDA(expr)                                                                   \
    do                                                                                     \
    {                                                                                      \
        cudaError_t e = (expr);                                                            \
        if(e != cudaSuccess)                                                               \
        {                                                                                  \
            std::fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e), __LINE__); \
            return 2;                                                                      \
        }                                                                                  \
    } while(0)

static void fill(std::vector<__half>& v, uint64_t seed)
{
    uint64_t s = seed * 0x9E3779B97F4A7C15ull + 1;
    for(auto& x : v)
    {
        s ^= s << 13, s ^= s >> 7, s ^= s << 17; // xorshift64
        x = __float2half(float(int64_t(s % 2001) - 1000) / 1000.0f);
    }
}

int main(int argc, char** argv)
{
    const uint32_t m = argc > 1 ? atoi(argv[1]) : 1024, n = argc > 2 ? atoi(argv[2]) : 1024,
                   k = argc > 3 ? atoi(argv[3]) : 1024;
    const double alpha = argc > 4 ? atof(argv[4]) : 2.0, beta = argc > 5 ? atof(argv[5]) : 2.0;

    std::vector<__half> a(size_t(m) * k), b(size_t(k) * n), c(size_t(m) * n), d(size_t(m) * n),
        ref(size_t(m) * n);
    fill(a, 1), fill(b, 2), fill(c, 3);

    __half *dA, *dB, *dC, *dD;
    CHECK_CUDA(cudaMalloc(&dA, a.size() * 2));
    CHECK_CUDA(cudaMalloc(&dB, b.size() * 2));
    CHECK_CUDA(cudaMalloc(&dC, c.size() * 2));
    CHECK_CUDA(cudaMalloc(&dD, d.size() * 2));
    CHECK_CUDA(cudaMemcpy(dA, a.data(), a.size() * 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, b.data(), b.size() * 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dC, c.data(), c.size() * 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemset(dD, 0xff, d.size() * 2)); // NaN pattern: unwritten outputs show up

    auto launch = [&]() {
        return b200wmma_gemm(B200WMMA_F16, B200WMMA_F16, m, n, k, dA, dB, dC, dD, k, k, n, n, alpha,
                             beta, B200WMMA_ROW_MAJOR, B200WMMA_COL_MAJOR, nullptr);
    };
    const int warmups = 2, recorded = 5; // as the reference sample does
    for(int i = 0; i < warmups; ++i)
        if(int rc = launch())
        {
            std::fprintf(stderr, "launch failed: %s\n", b200wmma_status_string(rc));
            return 3;
        }
    cudaEvent_t start, stop;
    CHECK_CUDA(cudaEventCreate(&start));
    CHECK_CUDA(cudaEventCreate(&stop));
    CHECK_CUDA(cudaEventRecord(start));
    for(int i = 0; i < recorded; ++i)
        launch();
    CHECK_CUDA(cudaEventRecord(stop));
    CHECK_CUDA(cudaEventSynchronize(stop));
    float ms = 0;
    CHECK_CUDA(cudaEventElapsedTime(&ms, start, stop));
    if(int rc = b200wmma_check_device(nullptr, nullptr))
    {
        std::fprintf(stderr, "device check failed: %s\n", b200wmma_status_string(rc));
        return 4;
    }
    const double tflops = 2.0 * m * n * k * recorded / (ms * 1e-3) / 1e12;
    CHECK_CUDA(cudaMemcpy(d.data(), dD, d.size() * 2, cudaMemcpyDeviceToHost));

    // CPU validation, dtype codes: 0 = f16; layouts: 0 row, 1 col
    oracle_gemm(0, 0, 0, m, n, k, a.data(), b.data(), c.data(), ref.data(), k, k, n, n, alpha, beta,
                0, 1, 0, 0);
    const double err = oracle_max_rel_err(0, d.data(), ref.data(), uint64_t(m) * n);
    std::printf("BlkM, BlkN, BlkK, M, N, K, alpha, beta, elapsedMs, TFlops, maxRelErr\n");
    std::printf("256, 256, 64, %u, %u, %u, %g, %g, %f, %f, %g\n", m, n, k, alpha, beta,
                ms / recorded, tflops, err);
    const bool pass = err >= 0.0 && err <= 2e-3;
    std::printf("%s\n", pass ? "PASSED" : "FAILED");
    cudaFree(dA), cudaFree(dB), cudaFree(dC), cudaFree(dD);
    b200wmma_shutdown();
    return pass ? 0 : 1;
}
