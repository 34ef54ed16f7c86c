// Truncating quantisation of the distance operands
// (src/CudaLib/copy_and_transform_kernel.h:27-28: static_cast<T>(value * factor), i.e. toward zero).
#pragma once
#include <cstdint>

namespace pinkb {

// Truncating conversion of v * 255 (v * 65535); float-to-integer cvt clamps to
// the destination range, so one instruction both converts and saturates.
__device__ __forceinline__ uint32_t quant_u8(float v)
{
    uint32_t q;
    asm("cvt.rzi.u8.f32 %0, %1;" : "=r"(q) : "f"(__fmul_rn(v, 255.0f)));
    return q;
}

__device__ __forceinline__ uint32_t quant_u16(float v)
{
    uint32_t q;
    asm("cvt.rzi.u16.f32 %0, %1;" : "=r"(q) : "f"(__fmul_rn(v, 65535.0f)));
    return q;
}

} // namespace pinkb
