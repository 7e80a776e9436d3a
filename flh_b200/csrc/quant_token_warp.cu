// Per-token quantiser for K = 4096 with one WARP per token row, and K = 8192 with two (full-width binary32
// Hadamard in matmul_hadU's order + asymmetric int4 + nibble packing): the hidden states of Llama-7B / 70B.
// Described for K = 4096; with two warps a lane still owns 128 values, the second pass runs bits 7-12 over
// 2-wide columns (64-bit shared loads), the warps of a row meet at named barriers, and a lane stores one
// byte (two codes) per m.
//
// Every lane owns 128 values in registers, as 64 packed binary32 pairs:
//   pass 1  the row is staged in shared memory by coalesced 16-byte cp.async (the NEXT row of the
//           persistent warp is prefetched into L2 at once and copied while the second half of this
//           row is computed); a lane picks up 128 consecutive inputs and runs butterfly bits 0-6;
//   pass 2  one transpose through padded shared memory, 128-bit accesses on both sides: a lane then
//           owns elements m * 128 + 4 lane + i (m < 32, i < 4) and runs bits 7-11 over m, the two
//           halves of a packed pair being neighbouring elements;
//   quant   warp min/max by shuffles, scale and zero-point computed redundantly by every lane, four
//           neighbouring codes packed into 16 bits with shift-adds and stored directly.
// No block-level barrier, no byte staging of the codes.  Each butterfly is the IEEE sum or difference of
// its two inputs in ascending bit order, so the result is bit-identical to the 64-thread kernel and to the
// CPU restatement.
#include "token_common.cuh"

namespace flh {
namespace {

constexpr int kRowK = 4096;                             // values per warp of a row
static_assert(kRowK * 2 <= 32 * 132 * 4, "the staged row must fit the transpose buffer");
constexpr int kChunkWords = 132;                        // 128 values of a lane + 4 words of padding
constexpr int kXposeBytes = 32 * kChunkWords * 4;
constexpr int kWarpBytes = kXposeBytes;                 // 16,896 bytes per warp: the staged row aliases the transpose buffer
constexpr int kWarpsPerCta = 4;
constexpr int kCtasPerSm = 3;                           // 12 warps per SM: 168 registers, 66 KB per CTA

struct WarpParams {
    const uint8_t *x;      // rows of 4096 16-bit values
    long ld_bytes;
    long M;
    float clip;
    float eps;             // RMS-norm epsilon (NORM kernels)
    uint8_t *q;
    __half *scale;
    __half *zero;
};

// butterflies over the pair index k (0..63): partner k ^ h for h = H0, 2 H0, ... < 64
template <int H0>
__device__ __forceinline__ void bfly_pairs(uint64_t (&p)[64]) {
#pragma unroll
    for (int h = H0; h < 64; h <<= 1) {
#pragma unroll
        for (int k = 0; k < 64; ++k) {
            if ((k & h) == 0) {
                const uint64_t a = p[k], b = p[k + h];
                p[k] = add2(a, b);
                p[k + h] = sub2(a, b);
            }
        }
    }
}

// issue the sixteen 16-byte copies of this lane for one row of W warps (t = lane index inside the row, 0 .. 32 W - 1);
// chunk c of 128-byte line L lands at chunk c ^ ((L >> 1) & 7) of that line, which makes the reads of pass 1 conflict-free
template <int W>
__device__ __forceinline__ void stage_row(const WarpParams &p, long row, uint32_t stage, int t) {
    const uint8_t *src = p.x + row * p.ld_bytes + t * 16;
    // copy i covers chunks i * 32 W + t: line = i * 4 W + (t >> 3), (line >> 1) & 7 = (i * 2 W + (t >> 4)) & 7
    const int c0 = (t & 7) ^ (t >> 4);
    const uint32_t base = stage + ((t >> 3) << 7);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t dst = base + i * 512 * W + ((c0 ^ ((2 * W * i) & 7)) << 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + i * 512 * W));
    }
    asm volatile("cp.async.commit_group;" ::);
}

// HAD: apply the transform.  NORM: first RMS-normalise the row (weight 1) exactly as a separate kernel writing the
// input's 16-bit type would: s = sum of squares (each lane adds its 128 values in order with fma, lanes are joined
// by xor-shuffles 16, 8, 4, 2, 1, the two warps of a row last), c = 1 / sqrt(s / K + eps) correctly rounded,
// y = round16(x * c) — the quantiser then sees y.
template <bool BF16, int W, bool HAD, bool NORM>
__global__ void __launch_bounds__(kWarpsPerCta * 32, kCtasPerSm) quant_token_warp_kernel(const WarpParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ float red[kWarpsPerCta][2];
    __shared__ float red_sq[kWarpsPerCta];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = warp / W;                               // row slot of this warp inside the CTA
    const int t = (warp % W) * 32 + lane;                   // lane index inside the row: 0 .. 32 W - 1
    uint8_t *my = smem_raw + grp * (W * kWarpBytes);        // the row's buffer: 32 W chunks of 132 words
    const uint32_t stage = smem_u32(my);
    const uint32_t xp = stage;                              // transpose buffer (aliases the staged row)
    auto row_sync = [&]() {                                 // the warps of this row
        if (W == 1) __syncwarp();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(32 * W) : "memory");
    };

    const long nwarps = (long)gridDim.x * (kWarpsPerCta / W);    // rows in flight
    long row = (long)blockIdx.x * (kWarpsPerCta / W) + grp;
    if (row < p.M) stage_row<W>(p, row, stage, t);

    for (; row < p.M; row += nwarps) {
        uint64_t v[64];

        // ---------------- pass 1: 128 consecutive inputs, bits 0-6 --------------------------------
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        row_sync();
        {
            const uint8_t *mine = my + t * 256;
            const int tx = t & 7;
            // one 32-bit word = two neighbouring inputs -> one packed pair: with the transform (a + b, a - b), i.e. bit 0
            auto consume = [&](uint32_t word, int idx) {
                float lo, hi;
                if (BF16) {
                    const float a = __uint_as_float(word << 16);
                    const float b = __uint_as_float(word & 0xffff0000u);
                    lo = HAD ? __fadd_rn(a, b) : a;
                    hi = HAD ? __fsub_rn(a, b) : b;
                } else if (HAD) {
                    // bit 0 straight from the binary16 pair: a + b and fma(b, -1, a) with b widened inside the
                    // instruction are the same IEEE binary32 sum and difference as after two conversions
                    uint16_t ha, hb;
                    asm("mov.b32 {%0, %1}, %2;" : "=h"(ha), "=h"(hb) : "r"(word));
                    const float a = __half2float(__ushort_as_half(ha));
                    const uint16_t neg1 = 0xBC00u;
                    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(lo) : "h"(hb), "f"(a));
                    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(hi) : "h"(hb), "h"(neg1), "f"(a));
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&word));
                    lo = f.x; hi = f.y;
                }
                v[idx] = pack2(lo, hi);
            };
            if (NORM) {
                uint4 raw[16];
                float ssq = 0.0f;
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    raw[cc] = *reinterpret_cast<const uint4 *>(mine + (cc >> 3) * 128 + (((cc & 7) ^ tx) << 4));
                    const uint32_t w[4] = {raw[cc].x, raw[cc].y, raw[cc].z, raw[cc].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float a, b;
                        if (BF16) { a = __uint_as_float(w[k] << 16); b = __uint_as_float(w[k] & 0xffff0000u); }
                        else { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k])); a = f.x; b = f.y; }
                        ssq = __fmaf_rn(a, a, ssq);
                        ssq = __fmaf_rn(b, b, ssq);
                    }
                }
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) ssq = __fadd_rn(ssq, __shfl_xor_sync(0xffffffffu, ssq, sft));
                if (W > 1) {
                    if (lane == 0) red_sq[warp] = ssq;
                    row_sync();
                    ssq = __fadd_rn(red_sq[grp * W], red_sq[grp * W + 1]);
                }
                const float c = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(ssq, 1.0f / (float)(kRowK * W)), p.eps)));
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    const uint32_t w[4] = {raw[cc].x, raw[cc].y, raw[cc].z, raw[cc].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t word;
                        if (BF16) {
                            const __nv_bfloat162 y = __floats2bfloat162_rn(__fmul_rn(__uint_as_float(w[k] << 16), c),
                                                                           __fmul_rn(__uint_as_float(w[k] & 0xffff0000u), c));
                            word = *reinterpret_cast<const uint32_t *>(&y);
                        } else {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
                            const __half2 y = __floats2half2_rn(__fmul_rn(f.x, c), __fmul_rn(f.y, c));
                            word = *reinterpret_cast<const uint32_t *>(&y);
                        }
                        consume(word, cc * 4 + k);
                    }
                }
            } else {
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    const uint4 w4 = *reinterpret_cast<const uint4 *>(mine + (cc >> 3) * 128 + (((cc & 7) ^ tx) << 4));
                    consume(w4.x, cc * 4 + 0); consume(w4.y, cc * 4 + 1); consume(w4.z, cc * 4 + 2); consume(w4.w, cc * 4 + 3);
                }
            }
        }
        row_sync();                                     // the staged row is in registers everywhere
        const bool more = row + nwarps < p.M;
        if (more) {                                     // next row: towards L2 now, into shared memory below
            const uint8_t *nx = p.x + (row + nwarps) * p.ld_bytes + t * 128;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nx));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + 4096 * W));
        }
        if (!HAD) {
            if (more) stage_row<W>(p, row + nwarps, stage, t);       // no transpose: the buffer is free at once
        } else {
            bfly_pairs<1>(v);                               // bits 1-6

            // ---------------- transpose: lane's chunk out, 4-wide (W = 2: 2-wide) columns in ---------------
            {
                const uint32_t out = xp + t * (kChunkWords * 4);
#pragma unroll
                for (int k = 0; k < 64; k += 2)
                    asm volatile("st.shared.v2.u64 [%0], {%1, %2};" ::"r"(out + 8 * k), "l"(v[k]), "l"(v[k + 1]) : "memory");
            }
            row_sync();
            if (W == 1) {
                // pair index k = 2 m + h: elements m * 128 + 4 lane + 2 h + {0, 1}
                const uint32_t in = xp + t * 16;
#pragma unroll
                for (int m = 0; m < 32; ++m)
                    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v[2 * m]), "=l"(v[2 * m + 1]) : "r"(in + m * (kChunkWords * 4)) : "memory");
            } else {
                // pair index k = m (0..63): elements m * 128 + 2 t + {0, 1}
                const uint32_t in = xp + t * 8;
#pragma unroll
                for (int m = 0; m < 64; ++m)
                    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v[m]) : "r"(in + m * (kChunkWords * 4)) : "memory");
            }
            row_sync();                                     // the buffer is free again: stage the next row into it
            if (more) stage_row<W>(p, row + nwarps, stage, t);
            if (W == 1) bfly_pairs<2>(v);                   // bits 7-11 (over m, two pairs per m)
            else bfly_pairs<1>(v);                          // bits 7-12 (over m, one pair per m)
        }

        // ---------------- row min / max, parameters ------------------------------------------------
        float vmin = 0.0f, vmax = 0.0f;
#pragma unroll
        for (int k = 0; k < 64; ++k) {
            float a, b;
            unpack2(v[k], a, b);
            vmin = min3(vmin, a, b);
            vmax = max3(vmax, a, b);
        }
        vmin = warp_min(vmin);
        vmax = warp_max(vmax);
        if (W > 1) {                                    // join the warps of the row
            if (lane == 0) { red[warp][0] = vmin; red[warp][1] = vmax; }
            row_sync();
#pragma unroll
            for (int o = 0; o < W; ++o) { vmin = fminf(vmin, red[grp * W + o][0]); vmax = fmaxf(vmax, red[grp * W + o][1]); }
            // (the next write of red comes after three more row barriers)
        }
        const TokenRowParams rp = token_row_params(vmin, vmax, p.clip, !HAD ? 1.0f : W == 1 ? 64.0f : 90.50966799187809f);   // sqrt(4096 W) with the transform
        if (t == 0) { p.scale[row] = rp.scale; p.zero[row] = __float2half_rn(rp.zero); }

        // ---------------- codes --------------------------------------------------------------------
        // v * rd, (clamped only when the row needs it), + 1.5 * 2^23 leaves rint(v rd) = code - zero in
        // the low mantissa bits.  With b_i the four bit patterns of one m, the low 16 bits of
        // b0 + 16 b1 + 256 b2 + 4096 b3 + 0x1111 zero are the four packed codes: the constant upper
        // part of the patterns is a multiple of 2^16, and the sum of the true codes fits 16 bits.
        const uint64_t rd2 = pack2(rp.rd, rp.rd);
#pragma unroll
        for (int k = 0; k < 64; ++k) v[k] = mul2(v[k], rd2);
        if (rp.clamp) {
            const float lo = -rp.zero, hi = 15.0f - rp.zero;
#pragma unroll
            for (int k = 0; k < 64; ++k) {
                float a, b;
                unpack2(v[k], a, b);
                v[k] = pack2(fmaxf(fminf(a, hi), lo), fmaxf(fminf(b, hi), lo));
            }
        }
        const uint64_t magic2 = pack2(12582912.0f, 12582912.0f);
        if (!HAD) {
            // the lane holds 128 consecutive elements: eight codes per 32-bit word by Horner in 16; the constant upper
            // part J of the eight bit patterns contributes J * 0x11111111, which is taken off again (all mod 2^32)
            const uint32_t fix = 0x11111111u * (uint32_t)(int)rp.zero - 0x4B400000u * 0x11111111u;
            uint4 *qrow = reinterpret_cast<uint4 *>(p.q + row * (long)(kRowK * W / 2) + t * 64);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t w = 0;
#pragma unroll
                    for (int i = 3; i >= 0; --i) {
                        float r0, r1;
                        unpack2(add2(v[g * 16 + j * 4 + i], magic2), r0, r1);
                        w = (w * 16u + __float_as_uint(r1)) * 16u + __float_as_uint(r0);
                    }
                    o[j] = w + fix;
                }
                qrow[g] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        } else if (W == 1) {
            const uint32_t zsum = 0x1111u * (uint32_t)(int)rp.zero;
            uint16_t *qrow = reinterpret_cast<uint16_t *>(p.q + row * (long)(kRowK / 2)) + t;
#pragma unroll
            for (int m = 0; m < 32; ++m) {
                float r0, r1, r2, r3;
                unpack2(add2(v[2 * m], magic2), r0, r1);
                unpack2(add2(v[2 * m + 1], magic2), r2, r3);
                // Horner in 16: ((b3 16 + b2) 16 + b1) 16 + b0 + 0x1111 zero
                uint32_t w = __float_as_uint(r3) * 16u + __float_as_uint(r2);
                w = w * 16u + __float_as_uint(r1);
                w = w * 16u + __float_as_uint(r0);
                w += zsum;
                qrow[m * 32] = (uint16_t)w;
            }
        } else {
            // two neighbouring codes per m: the low byte of b0 + 16 b1 + 0x11 zero
            const uint32_t zsum = 0x11u * (uint32_t)(int)rp.zero;
            uint8_t *qrow = p.q + row * (long)(kRowK * W / 2) + t;
#pragma unroll
            for (int m = 0; m < 64; ++m) {
                float r0, r1;
                unpack2(add2(v[m], magic2), r0, r1);
                qrow[m * 64] = (uint8_t)(__float_as_uint(r1) * 16u + __float_as_uint(r0) + zsum);
            }
        }
    }
}

}  // namespace

// K = 4096 or 8192 (no factor stage), with or without the transform, optionally RMS-normalised first (norm_eps >= 0).
// Returns -1000 when the shape is not one this kernel takes (the caller then uses the general kernel).
int launch_quant_token_warp(const void *x, int in_dtype, long M, long K, long ld, int hadamard, float norm_eps, float clip,
                            uint8_t *q, void *scale, void *zero, cudaStream_t stream) {
    if (K != kRowK && K != 2 * kRowK) return -1000;
    const int W = (int)(K / kRowK);
    WarpParams p;
    p.x = static_cast<const uint8_t *>(x);
    p.ld_bytes = ld * 2;
    p.M = M;
    p.clip = clip;
    p.eps = norm_eps;
    p.q = q;
    p.scale = static_cast<__half *>(scale);
    p.zero = static_cast<__half *>(zero);
    const size_t smem = (size_t)kWarpsPerCta * kWarpBytes;
    const bool bf = in_dtype == FLH_B200_BF16, had = hadamard != 0, norm = norm_eps >= 0.0f;
    using Kern = void (*)(const WarpParams);
    // [bf16][W - 1][HAD][NORM]
    static const Kern table[2][2][2][2] = {
        {{{quant_token_warp_kernel<false, 1, false, false>, quant_token_warp_kernel<false, 1, false, true>},
          {quant_token_warp_kernel<false, 1, true, false>, quant_token_warp_kernel<false, 1, true, true>}},
         {{quant_token_warp_kernel<false, 2, false, false>, quant_token_warp_kernel<false, 2, false, true>},
          {quant_token_warp_kernel<false, 2, true, false>, quant_token_warp_kernel<false, 2, true, true>}}},
        {{{quant_token_warp_kernel<true, 1, false, false>, quant_token_warp_kernel<true, 1, false, true>},
          {quant_token_warp_kernel<true, 1, true, false>, quant_token_warp_kernel<true, 1, true, true>}},
         {{quant_token_warp_kernel<true, 2, false, false>, quant_token_warp_kernel<true, 2, false, true>},
          {quant_token_warp_kernel<true, 2, true, false>, quant_token_warp_kernel<true, 2, true, true>}}}};
    const Kern kern = table[bf][W - 1][had][norm];
    static bool attr_done[16][64] = {};
    const int which = (int)bf * 8 + (W - 1) * 4 + (int)had * 2 + (int)norm;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
    if (dev < 0 || !attr_done[which][dev]) {         // the attribute is per device
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "quant_token_warp smem attribute");
        if (dev >= 0) attr_done[which][dev] = true;
    }
    const int rows_per_cta = kWarpsPerCta / W;
    long grid = (M + rows_per_cta - 1) / rows_per_cta;
    if (grid > (long)kCtasPerSm * kNumSMs) grid = (long)kCtasPerSm * kNumSMs;
    kern<<<(unsigned)grid, kWarpsPerCta * 32, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "quant_token_warp launch");
}

}  // namespace flh
