// Shared host-side helpers for the launchers of this library.
#ifndef ROCWMMA_B200_CSRC_COMMON_CUH
#define ROCWMMA_B200_CSRC_COMMON_CUH

#include "rocwmma_b200.h"
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>

namespace b200wmma
{
    inline int cudaToStatus(cudaError_t e)
    {
        return e == cudaSuccess ? B200WMMA_OK : B200WMMA_ERR_CUDA;
    }

#define B200WMMA_CUDA_TRY(expr)               \
    do                                        \
    {                                         \
        cudaError_t e__ = (expr);             \
        if(e__ != cudaSuccess)                \
        {                                     \
            (void)cudaGetLastError();         \
            return B200WMMA_ERR_CUDA;         \
        }                                     \
    } while(0)

    inline size_t dtypeSize(int dt)
    {
        switch(dt)
        {
        case B200WMMA_F16:
        case B200WMMA_BF16:
            return 2;
        case B200WMMA_E4M3:
        case B200WMMA_E5M2:
        case B200WMMA_I8:
            return 1;
        case B200WMMA_F32:
        case B200WMMA_XF32:
        case B200WMMA_I32:
            return 4;
        case B200WMMA_F64:
            return 8;
        }
        return 0;
    }

    // Kernels of this library whose prologue touches no global data are launched with
    // programmatic stream serialization: they may be scheduled while the previous kernel of
    // the stream drains, set up shared memory, and block in griddepcontrol.wait until that
    // kernel has completed.  B200WMMA_LAUNCH_OVERLAP=0 launches them fully serialised.
    inline bool launchOverlapEnabled()
    {
        static const bool on = [] {
            const char* e = getenv("B200WMMA_LAUNCH_OVERLAP");
            return !(e && e[0] == '0');
        }();
        return on;
    }

    template <typename... Params, typename... Args>
    inline cudaError_t launchOverlapped(void (*kernel)(Params...), dim3 grid, dim3 block,
                                        size_t smemBytes, cudaStream_t stream, Args&&... args)
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim            = grid;
        cfg.blockDim           = block;
        cfg.dynamicSmemBytes   = smemBytes;
        cfg.stream             = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs    = attr;
        cfg.numAttrs = launchOverlapEnabled() ? 1 : 0;
        return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
    }

    // Device-side error word shared by all kernels that contain bounded waits.
    // Returns the device address of a zero-initialised uint32_t[4] for the
    // current device (allocated once per device), or nullptr on failure.
    uint32_t* deviceStatusWord();

    // Number of SMs of the current device (cached).
    int smCount();
} // namespace b200wmma

#endif
