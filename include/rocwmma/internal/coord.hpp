// Two-component coordinates (row, col) used by the mapping helpers of the API.
// Mirrors the user-visible part of rocWMMA's Coord2d / make_coord2d / get<I>
// (internal/types.hpp, internal/vector.hpp:448) without the HIP vector
// machinery behind them.
#ifndef ROCWMMA_B200_COORD_HPP
#define ROCWMMA_B200_COORD_HPP

#include "config.hpp"

namespace rocwmma
{
    struct Coord2d
    {
        uint32_t data[2];

        ROCWMMA_HOST_DEVICE constexpr uint32_t&       operator[](uint32_t i) { return data[i]; }
        ROCWMMA_HOST_DEVICE constexpr uint32_t const& operator[](uint32_t i) const { return data[i]; }

        ROCWMMA_HOST_DEVICE constexpr Coord2d operator+(Coord2d const& o) const
        {
            return Coord2d{{data[0] + o.data[0], data[1] + o.data[1]}};
        }
        ROCWMMA_HOST_DEVICE constexpr Coord2d operator-(Coord2d const& o) const
        {
            return Coord2d{{data[0] - o.data[0], data[1] - o.data[1]}};
        }
        ROCWMMA_HOST_DEVICE constexpr Coord2d operator*(Coord2d const& o) const
        {
            return Coord2d{{data[0] * o.data[0], data[1] * o.data[1]}};
        }
        ROCWMMA_HOST_DEVICE constexpr Coord2d operator*(uint32_t s) const
        {
            return Coord2d{{data[0] * s, data[1] * s}};
        }
        ROCWMMA_HOST_DEVICE constexpr Coord2d& operator+=(Coord2d const& o)
        {
            data[0] += o.data[0];
            data[1] += o.data[1];
            return *this;
        }
        ROCWMMA_HOST_DEVICE constexpr bool operator==(Coord2d const& o) const
        {
            return data[0] == o.data[0] && data[1] == o.data[1];
        }
    };

    ROCWMMA_HOST_DEVICE constexpr inline Coord2d make_coord2d(uint32_t x, uint32_t y)
    {
        return Coord2d{{x, y}};
    }

    template <uint32_t I>
    ROCWMMA_HOST_DEVICE constexpr inline uint32_t& get(Coord2d& c)
    {
        static_assert(I < 2, "Coord2d has two components");
        return c.data[I];
    }
    template <uint32_t I>
    ROCWMMA_HOST_DEVICE constexpr inline uint32_t get(Coord2d const& c)
    {
        static_assert(I < 2, "Coord2d has two components");
        return c.data[I];
    }

    ROCWMMA_HOST_DEVICE constexpr inline Coord2d swap(Coord2d const& c)
    {
        return Coord2d{{c.data[1], c.data[0]}};
    }

    // Log2<N>::value for a power of two N, as a compile-time constant (rocWMMA
    // internal/utils.hpp:151-168; kernels use it to turn divisions by tile sizes into
    // shifts, samples/simple_dlrm.cpp:206).
    template <uint32_t N>
    struct Log2
    {
        static_assert(N != 0u && (N & (N - 1u)) == 0u, "Log2 needs a power of two");
        static constexpr uint32_t value = 1u + Log2<(N >> 1)>::value;
    };
    template <>
    struct Log2<1u>
    {
        static constexpr uint32_t value = 0u;
    };

    template <typename IntT1, typename IntT2>
    ROCWMMA_HOST_DEVICE constexpr inline auto ceilDiv(IntT1 numerator, IntT2 divisor)
    {
        return (numerator + divisor - 1) / divisor;
    }
} // namespace rocwmma

#endif // ROCWMMA_B200_COORD_HPP
