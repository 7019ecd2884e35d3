// Arithmetic shared by every kernel that evaluates batch norm + 2x2 average pool between SC layers, so that
// the fused and the separate forms give bit-identical values: the same expressions, compiled once.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace geo {

// Where a kernel reads the convolution's value from: fp32 x, or the int32 bit counts it was made from
// (x = counts * scale with scale = 1 / bit_length, a power of two, so the product is exact).
struct XSource {
    const void *p;
    float scale;
    int counts;
};

// Four consecutive values starting at element 4 * i.
__device__ __forceinline__ float4 load_x4(const XSource &xs, size_t i) {
    if (xs.counts) {
        const int4 v = __ldg((const int4 *)xs.p + i);
        return make_float4((float)v.x * xs.scale, (float)v.y * xs.scale, (float)v.z * xs.scale, (float)v.w * xs.scale);
    }
    return __ldg((const float4 *)xs.p + i);
}

// Two consecutive values starting at element 2 * i.
__device__ __forceinline__ float2 load_x2(const XSource &xs, size_t i) {
    if (xs.counts) {
        const int2 v = __ldg((const int2 *)xs.p + i);
        return make_float2((float)v.x * xs.scale, (float)v.y * xs.scale);
    }
    return __ldg((const float2 *)xs.p + i);
}

// Mean over a 2x2 window of (x * w + b): sum the window, then divide by its size (the association of avg_pool2d).
__device__ __forceinline__ float pooled_value(float x00, float x01, float x10, float x11, float w, float b) {
    return ((x00 * w + b) + (x01 * w + b) + (x10 * w + b) + (x11 * w + b)) / 4.0f;
}

// clamp(rint(v * levels), -(levels - 1), levels - 1) / levels; NaN stays NaN (utils_functional.py:33-39)
__device__ __forceinline__ float quantize_value(float v, float levels, float inv) {
    const float q = fminf(fmaxf(rintf(v * levels), 1.0f - levels), levels - 1.0f) * inv;
    return v != v ? v : q;
}

}  // namespace geo
