// SiLU(gate) * up of the MLP (flh/quantized_model/modeling_llama.py:522-526: act_fn(gate_proj(x)) * up_proj(x)), defined
// so that the CPU restatement gives the same bits: every step is one IEEE binary32 operation in a fixed order.
//   e      = exp32(-g)                    g, u: the two 16-bit inputs widened to binary32
//   s      = round16(g / (1 + e))         (torch rounds silu's result to the 16-bit type too)
//   result = round16(s * u)               (the product of two 16-bit values is exact in binary32)
//   exp32(t), t clamped to [-87, 88]:  n = rint(t * log2(e));  r = t - n ln2 (two fma, ln2 split in two);
//   y = 1 + r + r^2 P(r) with the degree-5 polynomial of the Cephes expf (Horner, fma);  exp32 = y * 2^n.
#pragma once
#include "common.cuh"

namespace flh {

__device__ __forceinline__ float exp32(float t) {
    t = fminf(fmaxf(t, -87.0f), 88.0f);
    const float n = rintf(__fmul_rn(t, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693359375f, t);
    r = __fmaf_rn(n, 2.12194440e-4f, r);
    const float z = __fmul_rn(r, r);
    float y = 1.9875691500e-4f;
    y = __fmaf_rn(y, r, 1.3981999507e-3f);
    y = __fmaf_rn(y, r, 8.3334519073e-3f);
    y = __fmaf_rn(y, r, 4.1665795894e-2f);
    y = __fmaf_rn(y, r, 1.6666665459e-1f);
    y = __fmaf_rn(y, r, 5.0000001201e-1f);
    y = __fmaf_rn(y, z, r);
    y = __fadd_rn(y, 1.0f);
    return __fmul_rn(y, __int_as_float(((int)n + 127) << 23));
}

// two neighbouring elements at once: g2, u2 hold two 16-bit values each (low half = the lower index)
template <bool BF16>
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t g2, uint32_t u2) {
    float g0, g1, u0, u1;
    if (BF16) {
        g0 = __uint_as_float(g2 << 16); g1 = __uint_as_float(g2 & 0xffff0000u);
        u0 = __uint_as_float(u2 << 16); u1 = __uint_as_float(u2 & 0xffff0000u);
    } else {
        const float2 gf = __half22float2(*reinterpret_cast<const __half2 *>(&g2));
        const float2 uf = __half22float2(*reinterpret_cast<const __half2 *>(&u2));
        g0 = gf.x; g1 = gf.y; u0 = uf.x; u1 = uf.y;
    }
    const float s0 = __fdiv_rn(g0, __fadd_rn(1.0f, exp32(-g0)));
    const float s1 = __fdiv_rn(g1, __fadd_rn(1.0f, exp32(-g1)));
    if (BF16) {
        const float a0 = __bfloat162float(__float2bfloat16_rn(s0)), a1 = __bfloat162float(__float2bfloat16_rn(s1));
        const __nv_bfloat162 o = __floats2bfloat162_rn(__fmul_rn(a0, u0), __fmul_rn(a1, u1));
        return *reinterpret_cast<const uint32_t *>(&o);
    }
    const float a0 = __half2float(__float2half_rn(s0)), a1 = __half2float(__float2half_rn(s1));
    const __half2 o = __floats2half2_rn(__fmul_rn(a0, u0), __fmul_rn(a1, u1));
    return *reinterpret_cast<const uint32_t *>(&o);
}

template <bool BF16>
__device__ __forceinline__ uint4 silu_mul_8(const uint4 g, const uint4 u) {
    return make_uint4(silu_mul_pair<BF16>(g.x, u.x), silu_mul_pair<BF16>(g.y, u.y), silu_mul_pair<BF16>(g.z, u.z),
                      silu_mul_pair<BF16>(g.w, u.w));
}

}  // namespace flh
