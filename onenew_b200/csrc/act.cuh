// act.cuh -- the fused activation shared by the contraction epilogue and the depthwise kernel.
#pragma once
#include <cuda_runtime.h>

namespace one {

// ACT_TYPE_E of the reference ABI: 0 none, 1 relu, 2 relu6 (never handled by the reference:
// identity), 3 silu (table), 4 clip, 5 hard-silu, 6 leaky relu.  Mirrors do_act,
// device/x86/Conv/conv.c:1216-1304, with the multiplies and adds kept separate as the
// reference's -std=c11 build does (no FMA contraction).
// The table lookup of do_act's SiLU (device/x86/Conv/conv.c:1216-1304) and of Gelu
// (device/x86/Gelu/gelu.c:22-38; same grid, another table), branch free so that the lookups of
// neighbouring elements overlap.  `lut` may point to global or to shared memory.
__device__ __forceinline__ float silu_table(float v, const float *__restrict__ lut)
{
    const float c = fminf(fmaxf(v, -8.0f), 7.998046875f);              // keeps the index inside the table
    const float t = lut[(int)__fmul_rn(__fadd_rn(c, 8.0f), 512.0f)];
    return v < -8.0f ? 0.f : (v >= 8.0f ? v : t);
}

__device__ __forceinline__ float apply_act(float v, int act, float p0, float p1, const float *__restrict__ lut)
{
    switch (act) {
    case 1: return v > 0.f ? v : 0.f;
    case 3:
        if (v < -8.0f) return 0.f;
        if (v >= 8.0f) return v;
        if (v >= -8.0f && v < 8.0f) return __ldg(lut + (int)__fmul_rn(__fadd_rn(v, 8.0f), 512.0f));
        return v;
    case 4: {
        float t = v > p0 ? v : p0;
        return t < p1 ? t : p1;
    }
    case 5: {
        float t = __fadd_rn(__fmul_rn(p0, v), p1);
        t = t > 0.f ? t : 0.f;
        return __fmul_rn(v, t < 1.f ? t : 1.f);
    }
    case 6: return v > 0.f ? v : __fmul_rn(p0, v);
    default: return v;
    }
}

}  // namespace one
