// 16-bit float storage of activations and weights: bf16 (8 exponent bits, 7 mantissa bits) or fp16 (5 exponent
// bits, 10 mantissa bits -- the mantissa of tf32, so an fp16 tensor holds what the tf32 path would have rounded
// an fp32 one to, in half the bytes, as long as magnitudes stay inside [2^-14, 65504]).  Both travel as raw 16-bit
// words; `f16` picks the format.  Conversions round to nearest even; an fp16 conversion of a larger magnitude
// gives infinity, which the kernels that produce values report through the status word (ST_RANGE_F16).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace one {

static constexpr float F16_MAX = 65504.f;

__device__ __forceinline__ uint32_t h16_pack2(float a, float b, bool f16)
{
    if (f16) {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ float2 h16_unpack2(uint32_t w, bool f16)
{
    if (f16) return __half22float2(*reinterpret_cast<const __half2 *>(&w));
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w));
}
__device__ __forceinline__ uint16_t h16_pack1(float a, bool f16)
{
    if (f16) return __half_as_ushort(__float2half_rn(a));
    return __bfloat16_as_ushort(__float2bfloat16_rn(a));
}
__device__ __forceinline__ float h16_unpack1(uint16_t w, bool f16)
{
    if (f16) return __half2float(__ushort_as_half(w));
    return __bfloat162float(__ushort_as_bfloat16(w));
}

}  // namespace one
