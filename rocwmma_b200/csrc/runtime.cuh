// Per-device caches owned by runtime.cu.
#ifndef ROCWMMA_B200_CSRC_RUNTIME_CUH
#define ROCWMMA_B200_CSRC_RUNTIME_CUH
#include <cstddef>

namespace b200wmma
{
    // A device buffer of at least `bytes`, kept per device and grown on demand
    // (contents are not preserved across growth).  nullptr on failure.
    void* deviceScratch(size_t bytes);
    // Staging buffers for the host-buffer GEMM entry point; slot 0..3 = A, B, C, D.
    void* stagingBuffer(int slot, size_t bytes);
} // namespace b200wmma
#endif
