// Build configuration for the sm_100a implementation of the rocWMMA device API.
// Replaces the arch detection of rocWMMA's internal/config.hpp:48-224 (AMD gfx
// targets, wave64/wave32) with a single target: NVIDIA Blackwell B200, 32-lane
// warps.
#ifndef ROCWMMA_B200_CONFIG_HPP
#define ROCWMMA_B200_CONFIG_HPP

#include <cstdint>
#include <cuda_runtime.h>

#define ROCWMMA_DEVICE __device__
#define ROCWMMA_HOST __host__
#define ROCWMMA_HOST_DEVICE __host__ __device__
#define ROCWMMA_KERNEL __global__

#define ROCWMMA_ARCH_SM100A 1
#define ROCWMMA_WAVE32_MODE 1

#define ROCWMMA_VERSION_MAJOR 1
#define ROCWMMA_VERSION_MINOR 7
#define ROCWMMA_VERSION_PATCH 0

#define ROCWMMA_UNROLL _Pragma("unroll")

#endif // ROCWMMA_B200_CONFIG_HPP
