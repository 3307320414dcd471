// Shared host-side helpers for the launchers of this library.
#ifndef ROCWMMA_B200_CSRC_COMMON_CUH
#define ROCWMMA_B200_CSRC_COMMON_CUH

#include "rocwmma_b200.h"
#include <cstdint>
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

    // Device-side error word shared by all kernels that contain bounded waits.
    // Returns the device address of a zero-initialised uint32_t[4] for the
    // current device (allocated once per device), or nullptr on failure.
    uint32_t* deviceStatusWord();

    // Number of SMs of the current device (cached).
    int smCount();
} // namespace b200wmma

#endif
