// Per-device caches owned by runtime.cu.
#ifndef ROCWMMA_B200_CSRC_RUNTIME_CUH
#define ROCWMMA_B200_CSRC_RUNTIME_CUH
#include <cstddef>
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

namespace b200wmma
{
    // cuTensorMapEncodeTiled, looked up once through the runtime (no link-time dependency on
    // the driver library).  nullptr when the driver does not offer it.
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    EncodeFn tensorMapEncoder();

    // A device buffer of at least `bytes`, kept per device and grown on demand
    // (contents are not preserved across growth).  nullptr on failure.
    void* deviceScratch(size_t bytes);
    // Workspace of the GEMM's split tiles: at least `bytes` of device memory (grown on demand)
    // and, through *counters, 256 zero-initialised 32-bit arrival counters that the kernels
    // leave at zero.  One per device: GEMM launches that split tiles must not overlap on one
    // device (different streams).  nullptr on failure.
    void* splitWorkspace(size_t bytes, uint32_t** counters);
    // Staging buffers for the host-buffer GEMM entry point; slot 0..3 = A, B, C, D.
    void* stagingBuffer(int slot, size_t bytes);

    // A 4-byte device counter for one kernel launch on `stream` (work distribution).  Every
    // stream of a device owns one counter (up to 64 streams; a 65th makes the call wait for
    // the device and start over), which the launches of that stream share: they run one
    // after the other.  A counter is zero when it is handed out and the kernel that uses it
    // must leave it at zero (the counters are zeroed once, synchronously, when they are
    // allocated: the first call on a device must not be made while a stream is being
    // captured).  nullptr on failure.
    unsigned int* launchCounter(cudaStream_t stream);
    // Puts every counter of the current device back to zero (after a kernel gave up).
    void resetLaunchCounters();

    // Lock held by the host-buffer GEMM entry point for the whole call: its staging buffers,
    // copy streams and events exist once per device.  nullptr without a device.
    std::mutex* hostCallMutex();

    // Copy streams and events for the host-buffer GEMM entry point (created on first use,
    // one set per device, destroyed by b200wmma_shutdown).
    constexpr int HOST_PIPE_MAX_CHUNKS = 16;
    struct HostPipe
    {
        cudaStream_t h2d = nullptr, d2h = nullptr;
        cudaEvent_t  start = nullptr, bReady = nullptr;
        cudaEvent_t  in[HOST_PIPE_MAX_CHUNKS]  = {};
        cudaEvent_t  out[HOST_PIPE_MAX_CHUNKS] = {};
        bool         ok = false;
    };
    HostPipe* hostPipe();
} // namespace b200wmma
#endif
