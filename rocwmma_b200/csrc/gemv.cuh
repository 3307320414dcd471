// Internal interface of the GEMV kernels (gemv.cu).
#ifndef ROCWMMA_B200_CSRC_GEMV_CUH
#define ROCWMMA_B200_CSRC_GEMV_CUH
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace b200wmma
{
    // Chooses how many K slices the partial-sum kernel uses and how many columns
    // each covers; the scratch array needs kSplit * m elements.
    void gemvPlan(uint32_t m, uint32_t k, size_t elemBytes, int sms, uint32_t* kSplit,
                  uint32_t* kChunk);

    // Runs both GEMV kernels on `stream` with caller-provided scratch `partial`.
    template <typename T>
    int gemvRun(uint32_t m, uint32_t k, T const* a, T const* x, T const* yIn, T* yOut, T alpha,
                T beta, uint32_t lda, T* partial, uint32_t kSplit, uint32_t kChunk,
                cudaStream_t stream);
} // namespace b200wmma
#endif
