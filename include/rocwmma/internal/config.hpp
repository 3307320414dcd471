// Build configuration for the sm_100a implementation of the rocWMMA device API.
// Replaces the arch detection of rocWMMA's internal/config.hpp:48-224 (AMD gfx
// targets, wave64/wave32) with a single target: NVIDIA Blackwell B200, 32-lane
// warps.
#ifndef ROCWMMA_B200_CONFIG_HPP
#define ROCWMMA_B200_CONFIG_HPP

// Under run-time compilation (NVRTC defines __CUDACC_RTC__) no host headers exist: the
// fixed-width integers and the type traits come from libcu++ instead, which ships with the
// toolkit and works in both modes.  rocWMMA makes the same promise for hipRTC
// (docs/conceptual/programmers-guide.rst:28-34).
#if defined(__CUDACC_RTC__)
#include <cuda/std/cstdint>
#include <cuda/std/type_traits>
using cuda::std::int16_t;
using cuda::std::int32_t;
using cuda::std::int64_t;
using cuda::std::int8_t;
using cuda::std::uint16_t;
using cuda::std::uint32_t;
using cuda::std::uint64_t;
using cuda::std::uint8_t;
using cuda::std::uintptr_t;
namespace rocwmma
{
    namespace stdx = ::cuda::std;
}
#else
#include <cstdint>
#include <cuda_runtime.h>
namespace rocwmma
{
    namespace stdx = ::std;
}
#endif

#define ROCWMMA_DEVICE __device__
#define ROCWMMA_HOST __host__
#define ROCWMMA_HOST_DEVICE __host__ __device__
#define ROCWMMA_KERNEL __global__

#define ROCWMMA_ARCH_SM100A 1
// 1 while the host side of a translation unit is compiled, 0 in the device pass: kernels
// written for rocWMMA wrap their bodies in `if constexpr(!ROCWMMA_ARCH_HOST)`
// (rocWMMA internal/config.hpp:73-111, samples/perf_hgemm.cpp:532).
#if defined(__CUDA_ARCH__)
#define ROCWMMA_ARCH_HOST 0
#else
#define ROCWMMA_ARCH_HOST 1
#endif
#define ROCWMMA_WAVE32_MODE 1

#define ROCWMMA_VERSION_MAJOR 1
#define ROCWMMA_VERSION_MINOR 7
#define ROCWMMA_VERSION_PATCH 0

#define ROCWMMA_UNROLL _Pragma("unroll")

#endif // ROCWMMA_B200_CONFIG_HPP
