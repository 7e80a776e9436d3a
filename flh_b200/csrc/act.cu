// Element-wise pieces of the decoder wiring that sit either side of the quantised linears
// (flh/quantized_model/modeling_llama.py:389-470, 522-526):
//   * silu_mul_kernel     SiLU(gate) * up from the merged gate/up GEMM output into a 16-bit matrix (the form the fused
//                         quantiser entry falls back to for widths its tensor-core kernel does not take);
//   * rope_kv_kernel      rotary embedding of q and k (half-split convention) straight from the merged QKV GEMM output:
//                         q goes to a [B, heads, S, D] tensor for the attention call, k and v are written into the KV cache
//                         at the step's position — one pass instead of split / rope / transpose / two cache copies.
#include "act_common.cuh"

namespace flh {
namespace {

template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint8_t *__restrict__ gu, long M, long F, long ld_bytes, uint8_t *__restrict__ out) {
    const long cpr = F / 8;                                        // 16-byte chunks per output row
    const long total = M * cpr;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long m = i / cpr, c = i - m * cpr;
        const uint8_t *row = gu + m * ld_bytes;
        const uint4 g = ldg_nc_v4(row + c * 16), u = ldg_nc_v4(row + F * 2 + c * 16);
        *reinterpret_cast<uint4 *>(out + (m * F + c * 8) * 2) = silu_mul_8<BF16>(g, u);
    }
}

struct RopeParams {
    const __half *qkv;         // [B * S, (nh + 2 nkv) * D]
    const float *cos, *sin;    // [S, D / 2] for the S positions of this step
    __half *q_out;             // [B, nh, S, D]
    __half *k_cache, *v_cache; // [B, nkv, T, D]
    int B, S, nh, nkv, D, T, cur;
};

// one thread per (token, head, pair of rotation partners x 4): 8 bytes of the first half and 8 of the second
__global__ void __launch_bounds__(256) rope_kv_kernel(const RopeParams p) {
    const int half = p.D / 2, vec = half / 4;                       // 4-element vectors per half head
    const int heads = p.nh + 2 * p.nkv;
    const long total = (long)p.B * p.S * heads * vec;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec);
        long r = i / vec;
        const int h = (int)(r % heads);
        r /= heads;
        const int s = (int)(r % p.S), b = (int)(r / p.S);
        const __half *src = p.qkv + ((long)(b * p.S + s) * heads + h) * p.D + v * 4;
        const uint2 lo = *reinterpret_cast<const uint2 *>(src), hi = *reinterpret_cast<const uint2 *>(src + half);
        uint2 olo = lo, ohi = hi;
        if (h < p.nh + p.nkv) {                                    // q and k rotate; v passes through
            const float4 c = *reinterpret_cast<const float4 *>(p.cos + (long)s * half + v * 4);
            const float4 sn = *reinterpret_cast<const float4 *>(p.sin + (long)s * half + v * 4);
            const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
            const __half *a = reinterpret_cast<const __half *>(&lo), *bb = reinterpret_cast<const __half *>(&hi);
            __half o1[4], o2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x1 = __half2float(a[e]), x2 = __half2float(bb[e]);
                // x1 cos - x2 sin and x2 cos + x1 sin, every product and sum rounded on its own (as separate tensor operations do)
                o1[e] = __float2half_rn(__fsub_rn(__fmul_rn(x1, cc[e]), __fmul_rn(x2, ss[e])));
                o2[e] = __float2half_rn(__fadd_rn(__fmul_rn(x2, cc[e]), __fmul_rn(x1, ss[e])));
            }
            olo = *reinterpret_cast<const uint2 *>(o1);
            ohi = *reinterpret_cast<const uint2 *>(o2);
        }
        __half *dst;
        if (h < p.nh) dst = p.q_out + (((long)b * p.nh + h) * p.S + s) * p.D;
        else if (h < p.nh + p.nkv) dst = p.k_cache + (((long)b * p.nkv + (h - p.nh)) * p.T + p.cur + s) * p.D;
        else dst = p.v_cache + (((long)b * p.nkv + (h - p.nh - p.nkv)) * p.T + p.cur + s) * p.D;
        *reinterpret_cast<uint2 *>(dst + v * 4) = olo;
        *reinterpret_cast<uint2 *>(dst + half + v * 4) = ohi;
    }
}

}  // namespace

int launch_silu_mul(const void *gu, int in_dtype, long M, long F, long ld, void *out, cudaStream_t stream) {
    const long total = M * (F / 8);
    if (total == 0) return 0;
    long grid = (total + 255) / 256;
    if (grid > 16L * kNumSMs) grid = 16L * kNumSMs;
    if (in_dtype == FLH_B200_BF16)
        silu_mul_kernel<true><<<(unsigned)grid, 256, 0, stream>>>(static_cast<const uint8_t *>(gu), M, F, ld * 2, static_cast<uint8_t *>(out));
    else
        silu_mul_kernel<false><<<(unsigned)grid, 256, 0, stream>>>(static_cast<const uint8_t *>(gu), M, F, ld * 2, static_cast<uint8_t *>(out));
    return cuda_status(cudaGetLastError(), "silu_mul launch");
}

int launch_rope_kv(const void *qkv, const float *cos, const float *sin, void *q_out, void *k_cache, void *v_cache,
                   int B, int S, int nh, int nkv, int D, int T, int cur, cudaStream_t stream) {
    RopeParams p;
    p.qkv = static_cast<const __half *>(qkv);
    p.cos = cos; p.sin = sin;
    p.q_out = static_cast<__half *>(q_out);
    p.k_cache = static_cast<__half *>(k_cache);
    p.v_cache = static_cast<__half *>(v_cache);
    p.B = B; p.S = S; p.nh = nh; p.nkv = nkv; p.D = D; p.T = T; p.cur = cur;
    const long total = (long)B * S * (nh + 2 * nkv) * (D / 8);
    if (total == 0) return 0;
    long grid = (total + 255) / 256;
    if (grid > 16L * kNumSMs) grid = 16L * kNumSMs;
    rope_kv_kernel<<<(unsigned)grid, 256, 0, stream>>>(p);
    return cuda_status(cudaGetLastError(), "rope_kv launch");
}

}  // namespace flh
