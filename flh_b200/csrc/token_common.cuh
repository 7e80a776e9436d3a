// Pieces shared by the per-token quantiser kernels: row reductions and the scale / zero-point rule.
#pragma once
#include "common.cuh"

namespace flh {

__device__ __forceinline__ float min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, s));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
    return v;
}

// Quantisation parameters of one token row from its minimum a (<= 0) and maximum b (>= 0) BEFORE the
// 1/c normalisation of the transform (c = sqrt(K), folded into the scale):
//   scale = f16((clip b - clip a) / 15 / c), never zero;  d = c * scale;  rd = 1 / d (correctly rounded);
//   zero  = rint(-clip a * rd).
// `clamp` tells whether any code of the row can leave 0..15 before clamping: without clipping every
// element lies in [a, b], the product with rd and rint are monotonic, so the codes lie in
// [rint(a rd) + zero, rint(b rd) + zero].
struct TokenRowParams {
    __half scale;
    float rd, zero;
    bool clamp;
};
__device__ __forceinline__ TokenRowParams token_row_params(float a, float b, float clip, float c) {
    float zmin = __fmul_rn(a, clip), zmax = __fmul_rn(b, clip);
    if (zmin == 0.0f && zmax == 0.0f) { zmin = -1.0f; zmax = 1.0f; }
    float scale32 = __fdiv_rn(__fsub_rn(zmax, zmin), 15.0f);
    scale32 = __fdiv_rn(scale32, c);
    __half sh = __float2half_rn(scale32);
    if ((__half_as_ushort(sh) & 0x7fffu) == 0) sh = __ushort_as_half(0x0001u);
    const float d = __fmul_rn(c, __half2float(sh));
    TokenRowParams r;
    r.scale = sh;
    r.rd = __frcp_rn(d);
    r.zero = rintf(__fmul_rn(-zmin, r.rd));
    const bool in_range = clip == 1.0f && rintf(__fmul_rn(b, r.rd)) + r.zero <= 15.0f &&
                          rintf(__fmul_rn(a, r.rd)) + r.zero >= 0.0f;
    r.clamp = !in_range;
    return r;
}

}  // namespace flh
