// Warp-level tensor-core instructions (mma.sync) behind rocwmma::mma_sync.
//
// Takes the place of rocWMMA's MFMA/WMMA builtin wrappers
// (internal/mfma_impl.hpp:159-697, internal/wmma_impl.hpp:114-420).  Every
// function multiplies one 16 x KAtom tile of A by one KAtom x 8 tile of B and
// adds into a 16 x 8 accumulator tile held as four values per lane.  Operand
// registers are passed in the order the PTX ISA defines for each shape, which
// is also the order in which fragments keep their elements, so mma_sync needs
// no data movement between lanes.
#ifndef ROCWMMA_B200_MMA_SYNC_PTX_HPP
#define ROCWMMA_B200_MMA_SYNC_PTX_HPP

#include "types.hpp"

namespace rocwmma
{
    namespace detail
    {
        // ---- f16 x f16 -> f32, m16n8k16 ---------------------------------------
        ROCWMMA_DEVICE inline void mma_atom(float (&d)[4], uint32_t const (&a)[4],
                                            uint32_t const (&b)[2], float const (&c)[4], __half)
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
        }
        // ---- bf16 x bf16 -> f32, m16n8k16 --------------------------------------
        ROCWMMA_DEVICE inline void mma_atom(float (&d)[4], uint32_t const (&a)[4],
                                            uint32_t const (&b)[2], float const (&c)[4],
                                            __nv_bfloat16)
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
        }
        // ---- e4m3 x e4m3 -> f32, m16n8k32 --------------------------------------
        ROCWMMA_DEVICE inline void mma_atom(float (&d)[4], uint32_t const (&a)[4],
                                            uint32_t const (&b)[2], float const (&c)[4],
                                            __nv_fp8_e4m3)
        {
            asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
        }
        // ---- e5m2 x e5m2 -> f32, m16n8k32 --------------------------------------
        ROCWMMA_DEVICE inline void mma_atom(float (&d)[4], uint32_t const (&a)[4],
                                            uint32_t const (&b)[2], float const (&c)[4],
                                            __nv_fp8_e5m2)
        {
            asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e5m2.e5m2.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
        }
        // ---- tf32 x tf32 -> f32, m16n8k8 (operands are fp32 bit patterns; the
        //      tensor core reads the upper 19 bits) --------------------------------
        ROCWMMA_DEVICE inline void mma_atom_tf32(float (&d)[4], uint32_t const (&a)[4],
                                                 uint32_t const (&b)[2], float const (&c)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
        }
        // ---- s8 x s8 -> s32, m16n8k32 and m16n8k16 -------------------------------
        ROCWMMA_DEVICE inline void mma_atom_s8_k32(int32_t (&d)[4], uint32_t const (&a)[4],
                                                   uint32_t const (&b)[2], int32_t const (&c)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
                         "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
        }
        ROCWMMA_DEVICE inline void mma_atom_s8_k16(int32_t (&d)[4], uint32_t const (&a)[2],
                                                   uint32_t const (&b)[1], int32_t const (&c)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]), "r"(c[0]), "r"(c[1]), "r"(c[2]),
                           "r"(c[3]));
        }
        // ---- f64 x f64 -> f64, m16n8k4 -------------------------------------------
        ROCWMMA_DEVICE inline void mma_atom_f64(double (&d)[4], double const (&a)[2],
                                                double const (&b)[1], double const (&c)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                         : "=d"(d[0]), "=d"(d[1]), "=d"(d[2]), "=d"(d[3])
                         : "d"(a[0]), "d"(a[1]), "d"(b[0]), "d"(c[0]), "d"(c[1]), "d"(c[2]),
                           "d"(c[3]));
        }
        // ---- f16 x f16 -> f16, m16n8k16 (16-bit accumulation) ---------------------
        ROCWMMA_DEVICE inline void mma_atom_f16acc(uint32_t (&d)[2], uint32_t const (&a)[4],
                                                   uint32_t const (&b)[2], uint32_t const (&c)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 "
                         "{%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%9};"
                         : "=r"(d[0]), "=r"(d[1])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]),
                           "r"(c[0]), "r"(c[1]));
        }

        // ---- half-depth forms, for fragments whose BlockK is below the K extent above ----
        // f16 / bf16, m16n8k8: two A registers (rows g and g + 8), one B register
        ROCWMMA_DEVICE inline void mma_atom_k8(float (&d)[4], uint32_t const (&a)[2],
                                               uint32_t const (&b)[1], float const (&c)[4], __half)
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]), "f"(c[0]), "f"(c[1]), "f"(c[2]),
                           "f"(c[3]));
        }
        ROCWMMA_DEVICE inline void mma_atom_k8(float (&d)[4], uint32_t const (&a)[2],
                                               uint32_t const (&b)[1], float const (&c)[4],
                                               __nv_bfloat16)
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]), "f"(c[0]), "f"(c[1]), "f"(c[2]),
                           "f"(c[3]));
        }
        ROCWMMA_DEVICE inline void mma_atom_f16acc_k8(uint32_t (&d)[2], uint32_t const (&a)[2],
                                                      uint32_t const (&b)[1],
                                                      uint32_t const (&c)[2])
        {
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f16.f16.f16.f16 "
                         "{%0,%1}, {%2,%3}, {%4}, {%5,%6};"
                         : "=r"(d[0]), "=r"(d[1])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]), "r"(c[0]), "r"(c[1]));
        }
        // tf32, m16n8k4: two A registers, one B register
        ROCWMMA_DEVICE inline void mma_atom_tf32_k4(float (&d)[4], uint32_t const (&a)[2],
                                                    uint32_t const (&b)[1], float const (&c)[4])
        {
            asm volatile("mma.sync.aligned.m16n8k4.row.col.f32.tf32.tf32.f32 "
                         "{%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                         : "r"(a[0]), "r"(a[1]), "r"(b[0]), "f"(c[0]), "f"(c[1]), "f"(c[2]),
                           "f"(c[3]));
        }

        // fp32 -> tf32 with round-to-nearest (ties away), as a bit pattern.
        ROCWMMA_DEVICE inline uint32_t to_tf32(float f)
        {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
            return r;
        }
    } // namespace detail
} // namespace rocwmma

#endif // ROCWMMA_B200_MMA_SYNC_PTX_HPP
