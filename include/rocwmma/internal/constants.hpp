// Hardware constants.  Kernels written for rocWMMA read the lane count of the
// scheduling unit as rocwmma::Constants::AMDGCN_WAVE_SIZE
// (rocWMMA internal/constants.hpp:85-96, used e.g. by samples/simple_hgemm.cpp:106);
// the name is kept and is 32 on this target.
#ifndef ROCWMMA_B200_CONSTANTS_HPP
#define ROCWMMA_B200_CONSTANTS_HPP

#include "config.hpp"

namespace rocwmma
{
    struct Constants
    {
        static constexpr uint32_t AMDGCN_WAVE_SIZE_32 = 32u;
        static constexpr uint32_t AMDGCN_WAVE_SIZE_64 = 64u;
        static constexpr uint32_t AMDGCN_WAVE_SIZE    = AMDGCN_WAVE_SIZE_32;
        static constexpr uint32_t WARP_SIZE           = AMDGCN_WAVE_SIZE;

        static constexpr uint32_t AMDGCN_REGISTER_ELEMENT_SIZE_BYTES = 4u;
        static constexpr uint32_t AMDGCN_REGISTER_SIZE_BYTES
            = AMDGCN_REGISTER_ELEMENT_SIZE_BYTES * AMDGCN_WAVE_SIZE;

        // Shared memory available to one thread block on B200 (opt-in maximum).
        static constexpr uint32_t AMDGCN_LDS_MAX_SIZE_BYTES = 232448u;
        static constexpr uint32_t AMDGCN_CACHE_LINE_SIZE_BYTES = 128u;
    };
} // namespace rocwmma

#endif // ROCWMMA_B200_CONSTANTS_HPP
