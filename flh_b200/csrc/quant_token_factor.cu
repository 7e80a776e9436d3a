// Per-token quantiser for K = kfac * 64 (Llama-7B's down_proj input, K = 11008 = 172 * 64): binary32
// butterflies on the 64-long chunks, then the kfac x kfac +-1 factor of matmul_hadU on the 5th-generation
// tensor cores, then the asymmetric int4 quantiser, two token rows per step of a persistent CTA.
//
//   y[r][k * 64 + j] = sum_k' S[k][k'] * z[r][k' * 64 + j]            z = chunk-wise FHT of the row
// is the GEMM  D[m = (r, j)][n = k] = A[m][k'] * B[n][k']  with A = z (M-major: j is contiguous) and B = S.
// z is binary32; it is split EXACTLY into three bfloat16 planes (8 + 8 + 8 significand bits), every product with
// +-1 is exact and tcgen05.mma (kind::f16, bf16 operands) accumulates in binary32 in TMEM, so the result
// differs from the sequential sum of the CPU restatement only in the order and rounding of binary32 additions
// (the bit-exact order is the CUDA-core kernel, hadamard = 2).
//
// One step (two rows, M = 128), all 384 threads in the same role:
//   butterflies of pair i from registers loaded one step ahead  ->  wait for MMA(i-1)  ->  write the three
//   A planes (128-byte-swizzled, M-major) -> one thread issues 3 * kp/16 MMAs into TMEM buffer i & 1 ->
//   epilogue of pair i-1 from the other TMEM buffer (tcgen05.ld, row min/max, codes, pack, store)
// so the tensor core works on pair i while the CUDA cores finish pair i-1 and prepare pair i+1.
// The wait on the MMA barrier is bounded; a timeout sets a status word (flh_b200_gemm_status) and ends the CTA.
#include "tc_common.cuh"
#include "token_common.cuh"

namespace flh {
namespace {

constexpr int kThreadsF = 384;
__device__ int g_status_tf[4];

struct FactorParams {
    const uint8_t *x;               // rows of K 16-bit values
    long ld_bytes;
    long M;
    int bf16;
    int F, Fp;                      // factor order and its padding to a multiple of 16
    int K;                          // F * 64
    const __nv_bfloat16 *sign_mat;  // Fp x Fp, +-1, zero padding
    float clip, c;
    uint8_t *q;
    __half *scale, *zero;
};

// bytes of shared memory: three A planes, B, code staging for two rows, reductions + barrier + slack
__host__ __device__ inline int a_plane_bytes(int Fp) { return Fp / 8 * 2 * 1024; }
__host__ __device__ inline int b_bytes(int Fp) { return ((Fp + 63) / 64) * (Fp / 8) * 1024; }
__host__ __device__ inline int factor_smem_bytes(int Fp, int K) { return 3 * a_plane_bytes(Fp) + b_bytes(Fp) + 2 * K + 1024 + 1024; }

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void bfly6(float (&x)[64]) {
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const float a = x[2 * k], b = x[2 * k + 1];
        x[2 * k] = __fadd_rn(a, b);
        x[2 * k + 1] = __fsub_rn(a, b);
    }
    uint64_t p[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) p[k] = pack2(x[2 * k], x[2 * k + 1]);
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            if ((k & h) == 0) {
                const uint64_t a = p[k], b = p[k + h];
                p[k] = add2(a, b);
                p[k + h] = sub2(a, b);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 32; ++k) unpack2(p[k], x[2 * k], x[2 * k + 1]);
}

__global__ void __launch_bounds__(kThreadsF, 1) quant_token_factor_kernel(const FactorParams p) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_dyn + (base - raw);
    const int Fp = p.Fp, F = p.F, K = p.K;
    const int plane = a_plane_bytes(Fp);
    const uint32_t a_base = base, b_base = base + 3 * plane;
    uint8_t *cb = sm + 3 * plane + b_bytes(Fp);                     // [2][K] code bytes
    float *red = reinterpret_cast<float *>(cb + 2 * K);             // [2 rows][2][12 warps... 6 used per row]
    const uint32_t bar = base + 3 * plane + b_bytes(Fp) + 2 * K + 512;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + 3 * plane + b_bytes(Fp) + 2 * K + 528);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + 3 * plane + b_bytes(Fp) + 2 * K + 544);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- one-time setup: zero the A planes (padding rows stay zero), lay S out as the K-major B operand ----
    for (int i = tid; i < (3 * plane + b_bytes(Fp)) / 16; i += kThreadsF) reinterpret_cast<uint4 *>(sm)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    {
        // B[n][k'] = S[n][k']: k-atom kb = k' / 64, 8-row group g = n / 8 at (kb * Fp/8 + g) * 1024; row n % 8 of 128 bytes,
        // 16-byte chunk ((k' % 64) / 8) ^ (n % 8)
        const int cpr = Fp / 8;                                     // 16-byte chunks per row of S
        for (int i = tid; i < Fp * cpr; i += kThreadsF) {
            const int n = i / cpr, c = i - n * cpr;
            const uint4 v = *reinterpret_cast<const uint4 *>(p.sign_mat + (size_t)n * Fp + c * 8);
            const int kb = c >> 3, cc = c & 7;
            *reinterpret_cast<uint4 *>(sm + 3 * plane + (kb * (Fp / 8) + (n >> 3)) * 1024 + (n & 7) * 128 + ((cc ^ (n & 7)) << 4)) = v;
        }
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // this thread's chunk: row r of the pair, chunk k' (threads >= 2 F idle in the butterfly phase)
    const bool has_chunk = tid < 2 * F;
    const int cr = tid >= F ? 1 : 0, ck = tid - cr * F;
    const uint32_t a_off = ((ck >> 3) * 2 + cr) * 1024 + (ck & 7) * 128;   // inside a plane; chunk c at ((c ^ (ck & 7)) << 4)
    // epilogue role: TMEM lane quarter and column third
    const int eq = warp & 3, eg = warp >> 2;
    const int er = eq >> 1, ej = (eq & 1) * 32 + lane;                      // row of the pair, position inside the chunk
    const int nchunks = Fp / 16;
    const int c_lo = eg * 4, c_hi = (eg * 4 + 4 < nchunks) ? eg * 4 + 4 : nchunks;

    const long npairs = (p.M + 1) / 2;
    uint4 w[8];
    auto load_pair = [&](long pair) {
        const long row = 2 * pair + cr;
        if (has_chunk && row < p.M) {
            const uint8_t *src = p.x + row * p.ld_bytes + ck * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) w[c] = ldg_v4(src + c * 16);
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) w[c] = make_uint4(0, 0, 0, 0);
        }
    };

    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(Fp >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    bool ok = true;
    long it = 0;
    long pair = blockIdx.x;
    if (pair < npairs) load_pair(pair);

    auto epilogue = [&](long epair, int buf) {
        // values of (row er, position ej) for the factor rows k of this warp's column third: all loads first, one wait
        uint32_t v[64];
        const uint32_t taddr = tmem + ((uint32_t)(eq * 32) << 16) + buf * 256;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            if (c_lo + cc < c_hi) {
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[16 * cc + 0]), "=r"(v[16 * cc + 1]), "=r"(v[16 * cc + 2]), "=r"(v[16 * cc + 3]),
                               "=r"(v[16 * cc + 4]), "=r"(v[16 * cc + 5]), "=r"(v[16 * cc + 6]), "=r"(v[16 * cc + 7]),
                               "=r"(v[16 * cc + 8]), "=r"(v[16 * cc + 9]), "=r"(v[16 * cc + 10]), "=r"(v[16 * cc + 11]),
                               "=r"(v[16 * cc + 12]), "=r"(v[16 * cc + 13]), "=r"(v[16 * cc + 14]), "=r"(v[16 * cc + 15])
                             : "r"(taddr + (c_lo + cc) * 16) : "memory");
            }
        }
        tc_wait_ld();
        tc_fence_before();
        // columns past the factor order (padding of the last chunk, chunks this third does not have) count as 0
        const int nvalid = F - c_lo * 16;                 // valid values of this thread: indices < nvalid
        uint64_t y[32];
        if (nvalid >= 64) {               // warp-uniform: only the last column third has padding
#pragma unroll
            for (int i = 0; i < 32; ++i) y[i] = pack2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float f0 = (2 * i < nvalid) ? __uint_as_float(v[2 * i]) : 0.0f;
                const float f1 = (2 * i + 1 < nvalid) ? __uint_as_float(v[2 * i + 1]) : 0.0f;
                y[i] = pack2(f0, f1);
            }
        }
        float mn[4] = {0.0f, 0.0f, 0.0f, 0.0f}, mx[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float f0, f1;
            unpack2(y[i], f0, f1);
            mn[i & 3] = min3(mn[i & 3], f0, f1);
            mx[i & 3] = max3(mx[i & 3], f0, f1);
        }
        float vmin = warp_min(fminf(fminf(mn[0], mn[1]), fminf(mn[2], mn[3])));
        float vmax = warp_max(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
        if (lane == 0) { red[warp * 2] = vmin; red[warp * 2 + 1] = vmax; }
        __syncthreads();
        // the six warps of row er: lane quarters 2 er and 2 er + 1 of the three column thirds
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int g = 0; g < 3; ++g) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int wsrc = g * 4 + 2 * er + h;
                a = fminf(a, red[wsrc * 2]);
                b = fmaxf(b, red[wsrc * 2 + 1]);
            }
        }
        const TokenRowParams rp = token_row_params(a, b, p.clip, p.c);
        const long row = 2 * epair + er;
        if (eg == 0 && (eq & 1) == 0 && lane == 0 && row < p.M) { p.scale[row] = rp.scale; p.zero[row] = __float2half_rn(rp.zero); }
        {
            // v * rd, clamped only when the row needs it, + 1.5 * 2^23 (rint in the low mantissa bits), + zero (exact):
            // the low byte of the sum's bit pattern is the code
            const uint64_t rd2 = pack2(rp.rd, rp.rd), magic2 = pack2(12582912.0f, 12582912.0f), z2 = pack2(rp.zero, rp.zero);
#pragma unroll
            for (int i = 0; i < 32; ++i) y[i] = mul2(y[i], rd2);
            if (rp.clamp) {
                const float lo = -rp.zero, hi = 15.0f - rp.zero;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float f0, f1;
                    unpack2(y[i], f0, f1);
                    y[i] = pack2(fmaxf(fminf(f0, hi), lo), fmaxf(fminf(f1, hi), lo));
                }
            }
            uint8_t *dst = cb + er * K + ej + c_lo * 16 * 64;
            if (nvalid >= 64) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float r0, r1;
                    unpack2(add2(add2(y[i], magic2), z2), r0, r1);
                    dst[(2 * i) * 64] = (uint8_t)__float_as_uint(r0);
                    dst[(2 * i + 1) * 64] = (uint8_t)__float_as_uint(r1);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float r0, r1;
                    unpack2(add2(add2(y[i], magic2), z2), r0, r1);
                    if (2 * i < nvalid) dst[(2 * i) * 64] = (uint8_t)__float_as_uint(r0);
                    if (2 * i + 1 < nvalid) dst[(2 * i + 1) * 64] = (uint8_t)__float_as_uint(r1);
                }
            }
        }
        __syncthreads();
        // pack 16 staged codes into 8 bytes, coalesced 64-bit stores
        const int per_row = K >> 4;
        for (int i = tid; i < 2 * per_row; i += kThreadsF) {
            const int rr = i >= per_row ? 1 : 0, c16 = i - rr * per_row;
            const long orow = 2 * epair + rr;
            if (orow < p.M) {
                const uint4 cv = *reinterpret_cast<const uint4 *>(cb + rr * K + 16 * c16);
                const uint32_t ww[4] = {cv.x, cv.y, cv.z, cv.w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t tt = ww[j] | (ww[j] >> 4);
                    o[j] = __byte_perm(tt, 0, 0x4420);
                }
                reinterpret_cast<uint2 *>(p.q + orow * (long)(K >> 1))[c16] = make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
            }
        }
    };

    for (; pair < npairs && ok; pair += gridDim.x, ++it) {
        // ---- butterflies of this pair (bits 0-5 of every chunk) from the registers loaded a step ahead ----
        float x[64];
        if (p.bf16) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    x[8 * c + 2 * j] = __uint_as_float(ww[j] << 16);
                    x[8 * c + 2 * j + 1] = __uint_as_float(ww[j] & 0xffff0000u);
                }
            }
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&ww[j]));
                    x[8 * c + 2 * j] = f.x;
                    x[8 * c + 2 * j + 1] = f.y;
                }
            }
        }
        // next pair: towards L2 now; it is loaded into registers only after the epilogue below, so that the
        // epilogue does not have to keep (and wait for) 32 registers of loads in flight
        if (has_chunk && 2 * (pair + gridDim.x) + cr < p.M)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x + (2 * (pair + gridDim.x) + cr) * p.ld_bytes + ck * 128));
        if (has_chunk) bfly6(x);

        // ---- the A planes are free once MMA(it - 1) has finished ----
        if (it > 0) {
            const bool done = mbar_wait_status(g_status_tf, bar, (uint32_t)((it - 1) & 1), abort_flag, 21, nullptr);
            ok = __syncthreads_and(done) != 0;          // the whole CTA takes the same branch
            if (!ok) break;
            tc_fence_after();
        }
        if (has_chunk) {
            // exact split into three bfloat16 planes by truncation: hi = top 16 bits of x, mid = top 16 bits of x - hi,
            // lo = x - hi - mid (at most 8 significant bits are left); each difference is exact
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t pl[3][4];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const uint32_t b0 = __float_as_uint(x[8 * c + 2 * h]), b1 = __float_as_uint(x[8 * c + 2 * h + 1]);
                    pl[0][h] = __byte_perm(b0, b1, 0x7632);
                    float r0, r1;
                    unpack2(sub2(pack2(x[8 * c + 2 * h], x[8 * c + 2 * h + 1]),
                                 pack2(__uint_as_float(b0 & 0xffff0000u), __uint_as_float(b1 & 0xffff0000u))), r0, r1);
                    const uint32_t m0 = __float_as_uint(r0), m1 = __float_as_uint(r1);
                    pl[1][h] = __byte_perm(m0, m1, 0x7632);
                    float s0, s1;
                    unpack2(sub2(pack2(r0, r1), pack2(__uint_as_float(m0 & 0xffff0000u), __uint_as_float(m1 & 0xffff0000u))), s0, s1);
                    pl[2][h] = __byte_perm(__float_as_uint(s0), __float_as_uint(s1), 0x7632);
                }
                const uint32_t off = a_off + ((c ^ (ck & 7)) << 4);
#pragma unroll
                for (int sp = 0; sp < 3; ++sp)
                    *reinterpret_cast<uint4 *>(sm + sp * plane + off) = make_uint4(pl[sp][0], pl[sp][1], pl[sp][2], pl[sp][3]);
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();                 // planes written; every thread's TMEM reads of the previous epilogue are complete
        if (tid == kThreadsF - 32) {     // lane 0 of the last warp, whose column third is the short one
            tc_fence_after();
            const int buf = (int)(it & 1);
            bool first = true;
            for (int sp = 2; sp >= 0; --sp) {                        // smallest plane first
                for (int s = 0; s < Fp / 16; ++s) {
                    const uint64_t ad = umma_desc(a_base + sp * plane + s * 4096, 1024, 2048);
                    const uint64_t bd = umma_desc(b_base + (s >> 2) * (Fp / 8) * 1024 + (s & 3) * 32, 16, 1024);
                    const uint32_t acc = first ? 0u : 1u;
                    asm volatile("{\n\t.reg .pred pp;\n\tsetp.ne.b32 pp, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pp;\n\t}"
                                 ::"r"(tmem + buf * 256), "l"(ad), "l"(bd), "r"(idesc), "r"(acc) : "memory");
                    first = false;
                }
            }
            tc_commit(bar);
        }
        // ---- epilogue of the previous pair while the tensor core works on this one ----
        if (it > 0) epilogue(pair - gridDim.x, (int)((it - 1) & 1));
        if (pair + gridDim.x < npairs) load_pair(pair + gridDim.x);
    }
    if (ok && it > 0) {
        const bool done = mbar_wait_status(g_status_tf, bar, (uint32_t)((it - 1) & 1), abort_flag, 22, nullptr);
        ok = __syncthreads_and(done) != 0;
        if (ok) {
            tc_fence_after();
            epilogue(pair - gridDim.x, (int)((it - 1) & 1));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace

// K = F * 64 with F > 1 a multiple of 4 up to 176 after padding.  Returns -1000 when the shape is not one this
// kernel takes (the caller then uses the general kernel).
int launch_quant_token_factor(const void *x, int in_dtype, long M, long K, long ld, int kfac, const void *sign_mat_bf16,
                              float clip, uint8_t *q, void *scale, void *zero, cudaStream_t stream) {
    if (kfac <= 1 || K != (long)kfac * 64) return -1000;
    const int Fp = (kfac + 15) / 16 * 16;
    if (Fp > 176) return -1000;
    FactorParams p;
    p.x = static_cast<const uint8_t *>(x);
    p.ld_bytes = ld * 2;
    p.M = M;
    p.bf16 = in_dtype == FLH_B200_BF16;
    p.F = kfac; p.Fp = Fp; p.K = (int)K;
    p.sign_mat = static_cast<const __nv_bfloat16 *>(sign_mat_bf16);
    p.clip = clip;
    p.c = sqrtf((float)K);
    p.q = q;
    p.scale = static_cast<__half *>(scale);
    p.zero = static_cast<__half *>(zero);
    const int smem = factor_smem_bytes(Fp, (int)K);
    cudaError_t e = cudaFuncSetAttribute(quant_token_factor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "quant_token_factor smem attribute");
    long grid = (M + 1) / 2;
    if (grid > kNumSMs) grid = kNumSMs;
    quant_token_factor_kernel<<<(unsigned)grid, kThreadsF, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "quant_token_factor launch");
}

int quant_token_factor_status(int *out4) {
    return cuda_status(cudaMemcpyFromSymbol(out4, g_status_tf, sizeof(int) * 4), "status read");
}
int quant_token_factor_status_clear() {
    int z[4] = {0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_status_tf, z, sizeof(z)), "status clear");
}

}  // namespace flh
