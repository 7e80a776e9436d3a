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
// Two rows per step (M = 128) of a persistent CTA with warp roles (see the kernel): producer warps stream the chunks,
// run the butterflies and write the A planes; one thread issues the 3 * kp/16 MMAs into one of two TMEM buffers; the
// epilogue warps turn the other buffer into codes meanwhile.  All mbarrier waits are bounded; a timeout sets a status
// word (flh_b200_gemm_status) and the CTA runs out without touching the tensor core again.
#include "tc_common.cuh"
#include "token_common.cuh"

namespace flh {
namespace {

constexpr int kEpiWarps = 8;                       // 4: one epilogue warp per TMEM lane quarter; 8: two (column halves)
constexpr int kThreadsF = 256 + 32 * kEpiWarps;
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

// 16 packed codes -> 8 bytes
__device__ __forceinline__ uint2 pack16(const uint4 &cv) {
    const uint32_t ww[4] = {cv.x, cv.y, cv.z, cv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t tt = ww[j] | (ww[j] >> 4);
        o[j] = __byte_perm(tt, 0, 0x4420);
    }
    return make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
}

// Warp roles.  Warps 0-7 (256 threads) are PRODUCERS: they stream the chunks of a pair of rows (2 kfac chunks of 64,
// one or two per thread, the next one always in flight), run the six butterfly bits in registers, wait until the
// previous pair's MMAs have released the 16-chunk slice of the A planes they write to (one mbarrier per K step of
// the MMA, so writing overlaps the tail of the previous pair's MMAs), write the three bf16 planes, and one of them
// issues the MMAs.  Warps 8-15 (256 threads) are the EPILOGUE: TMEM lane quarter warp % 4 (row of the pair =
// quarter / 2), column half (warp - 8) / 4; they read the accumulator twice (row min/max, then codes), hand the
// TMEM buffer back, and the four warps of a row pack and store that row.  Producers and epilogue meet only through mbarriers (slice_free, acc_full,
// acc_empty) with bounded waits; named barriers join the warps of one role.  After a timeout every thread keeps
// walking its loop (without MMAs) so that no named barrier is left waiting.
__global__ void __launch_bounds__(kThreadsF, 1) quant_token_factor_kernel(const FactorParams p) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_dyn + (base - raw);
    const int Fp = p.Fp, F = p.F, K = p.K;
    const int plane = a_plane_bytes(Fp);
    const uint32_t a_base = base, b_base = base + 3 * plane;
    const int aux = 3 * plane + b_bytes(Fp) + 2 * K;
    uint8_t *cb = sm + 3 * plane + b_bytes(Fp);                     // [2][K] code bytes
    float *red = reinterpret_cast<float *>(sm + aux);               // [2 rows][2 warps][min, max]
    const uint32_t bars = base + aux + 512;
    auto acc_full = [&](int b) { return bars + 8u * b; };
    auto acc_empty = [&](int b) { return bars + 8u * (2 + b); };
    auto slice_free = [&](int sl) { return bars + 8u * (4 + sl); };   // K step sl of the MMAs has read its 16 chunks of the planes
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + aux + 512 + 192);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + aux + 512 + 208);

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
        for (int sl = 0; sl < Fp / 16; ++sl) mbar_init(slice_free(sl), 1);
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), kEpiWarps); }
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
    const long npairs = (p.M + 1) / 2;

    if (warp < 8) {
        // ================================================================= producers
        const int pt = tid;                                          // 0..255
        const int nchunks2 = 2 * F;                                  // chunks of a pair
        uint4 w[8];
        auto load_chunk = [&](long pair, int c) {
            const int r = c >= F ? 1 : 0;
            const long row = 2 * pair + r;
            if (row < p.M) {
                const uint8_t *src = p.x + row * p.ld_bytes + (c - r * F) * 128;
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = ldg_v4(src + i * 16);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = make_uint4(0, 0, 0, 0);
            }
        };
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(Fp >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        bool ok = true;
        long it = 0;
        long pair = blockIdx.x;
        if (pair < npairs && pt < nchunks2) load_chunk(pair, pt);
        for (; pair < npairs; pair += gridDim.x, ++it) {
#pragma unroll 1
            for (int rd = 0; rd < 2; ++rd) {
                const int c = pt + 256 * rd;
                if (c < nchunks2) {
                    float x[64];
                    if (p.bf16) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint32_t ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                x[8 * i + 2 * j] = __uint_as_float(ww[j] << 16);
                                x[8 * i + 2 * j + 1] = __uint_as_float(ww[j] & 0xffff0000u);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint32_t ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&ww[j]));
                                x[8 * i + 2 * j] = f.x;
                                x[8 * i + 2 * j + 1] = f.y;
                            }
                        }
                    }
                    // this thread's next chunk (same pair, or the first one of its next pair) goes in flight now
                    if (c + 256 < nchunks2) load_chunk(pair, c + 256);
                    else if (pair + gridDim.x < npairs) load_chunk(pair + gridDim.x, pt);
                    bfly6(x);
                    const int cr = c >= F ? 1 : 0, ck = c - cr * F;
                    if (it > 0) {                                    // this chunk's slice of the planes is free once K step ck / 16 of MMA(it - 1) is done
                        if (!mbar_wait_status(g_status_tf, slice_free(ck >> 4), (uint32_t)((it - 1) & 1), abort_flag, 21, nullptr)) ok = false;
                    }
                    const uint32_t a_off = ((ck >> 3) * 2 + cr) * 1024 + (ck & 7) * 128;
                    // exact split into three bfloat16 planes by truncation: hi = top 16 bits of x, mid = top 16 bits of x - hi,
                    // lo = x - hi - mid (at most 8 significant bits are left); each difference is exact
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        uint32_t pl[3][4];
#pragma unroll
                        for (int h = 0; h < 4; ++h) {
                            const uint32_t b0 = __float_as_uint(x[8 * i + 2 * h]), b1 = __float_as_uint(x[8 * i + 2 * h + 1]);
                            pl[0][h] = __byte_perm(b0, b1, 0x7632);
                            float r0, r1;
                            unpack2(sub2(pack2(x[8 * i + 2 * h], x[8 * i + 2 * h + 1]),
                                         pack2(__uint_as_float(b0 & 0xffff0000u), __uint_as_float(b1 & 0xffff0000u))), r0, r1);
                            const uint32_t m0 = __float_as_uint(r0), m1 = __float_as_uint(r1);
                            pl[1][h] = __byte_perm(m0, m1, 0x7632);
                            float s0, s1;
                            unpack2(sub2(pack2(r0, r1), pack2(__uint_as_float(m0 & 0xffff0000u), __uint_as_float(m1 & 0xffff0000u))), s0, s1);
                            pl[2][h] = __byte_perm(__float_as_uint(s0), __float_as_uint(s1), 0x7632);
                        }
                        const uint32_t off = a_off + ((i ^ (ck & 7)) << 4);
#pragma unroll
                        for (int sp = 0; sp < 3; ++sp)
                            *reinterpret_cast<uint4 *>(sm + sp * plane + off) = make_uint4(pl[sp][0], pl[sp][1], pl[sp][2], pl[sp][3]);
                    }
                }
            }
            fence_proxy_async();
            bar_sync_named(1, 256);                                  // all planes of this pair are written
            if (pt == 255) {             // in a producer warp with one chunk per pair
                const int buf = (int)(it & 1);
                if (ok && it >= 2 &&
                    !mbar_wait_status(g_status_tf, acc_empty(buf), (uint32_t)((((it >> 1) - 1) & 1)), abort_flag, 23, nullptr)) ok = false;
                if (ok && !*abort_flag) {
                    tc_fence_after();
                    bool first = true;
                    for (int s = 0; s < Fp / 16; ++s) {              // K step s: chunks 16 s .. 16 s + 15 of both rows
                        const uint64_t bd = umma_desc(b_base + (s >> 2) * (Fp / 8) * 1024 + (s & 3) * 32, 16, 1024);
                        for (int sp = 2; sp >= 0; --sp) {            // smallest plane first
                            const uint64_t ad = umma_desc(a_base + sp * plane + s * 4096, 1024, 2048);
                            const uint32_t acc = first ? 0u : 1u;
                            asm volatile("{\n\t.reg .pred pp;\n\tsetp.ne.b32 pp, %4, 0;\n\t"
                                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pp;\n\t}"
                                         ::"r"(tmem + buf * 256), "l"(ad), "l"(bd), "r"(idesc), "r"(acc) : "memory");
                            first = false;
                        }
                        tc_commit(slice_free(s));
                    }
                    tc_commit(acc_full(buf));
                }
            }
        }
    } else {
        // ================================================================= epilogue
        constexpr int kH = kEpiWarps / 4;                            // column parts per lane quarter
        constexpr int kRowThreads = 64 * kH;                         // epilogue threads of one row
        const int eq = warp & 3, eh = (warp - 8) >> 2;               // TMEM lane quarter, column part
        const int er = eq >> 1, ej = (eq & 1) * 32 + lane;           // row of the pair, position inside the chunk
        const int et = eh * 64 + ej;                                 // index among the epilogue threads of this row
        const int nch = Fp / 16;
        const int c_lo = kH == 1 ? 0 : (eh == 0 ? 0 : (nch + 1) / 2), c_hi = kH == 1 ? nch : (eh == 0 ? (nch + 1) / 2 : nch);
        const int rslot = (eq & 1) * kH + eh;                        // this warp's slot in the row's reduction
        bool ok = true;
        long it = 0;
        for (long pair = blockIdx.x; pair < npairs; pair += gridDim.x, ++it) {
            const int buf = (int)(it & 1);
            if (!mbar_wait_status(g_status_tf, acc_full(buf), (uint32_t)((it >> 1) & 1), abort_flag, 22, nullptr)) ok = false;
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(eq * 32) << 16) + buf * 256;
            // ---- pass 1: row minimum / maximum (the next chunk's TMEM load is in flight while this one is reduced) ----
            float mn[2] = {0.0f, 0.0f}, mx[2] = {0.0f, 0.0f};
            {
                uint32_t va[16], vb[16];
                tmem_ld16(taddr + c_lo * 16, va);
                for (int c = c_lo; c < c_hi; c += 2) {
                    tc_wait_ld();
                    if (c + 1 < c_hi) tmem_ld16(taddr + (c + 1) * 16, vb);
                    if (F - c * 16 >= 16) {
#pragma unroll
                        for (int j = 0; j < 16; j += 2) {
                            mn[(j >> 1) & 1] = min3(mn[(j >> 1) & 1], __uint_as_float(va[j]), __uint_as_float(va[j + 1]));
                            mx[(j >> 1) & 1] = max3(mx[(j >> 1) & 1], __uint_as_float(va[j]), __uint_as_float(va[j + 1]));
                        }
                    } else {
                        const int nv = F - c * 16;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float f = j < nv ? __uint_as_float(va[j]) : 0.0f;
                            mn[0] = fminf(mn[0], f);
                            mx[0] = fmaxf(mx[0], f);
                        }
                    }
                    if (c + 1 < c_hi) {
                        tc_wait_ld();
                        if (c + 2 < c_hi) tmem_ld16(taddr + (c + 2) * 16, va);
                        if (F - (c + 1) * 16 >= 16) {
#pragma unroll
                            for (int j = 0; j < 16; j += 2) {
                                mn[(j >> 1) & 1] = min3(mn[(j >> 1) & 1], __uint_as_float(vb[j]), __uint_as_float(vb[j + 1]));
                                mx[(j >> 1) & 1] = max3(mx[(j >> 1) & 1], __uint_as_float(vb[j]), __uint_as_float(vb[j + 1]));
                            }
                        } else {
                            const int nv = F - (c + 1) * 16;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float f = j < nv ? __uint_as_float(vb[j]) : 0.0f;
                                mn[0] = fminf(mn[0], f);
                                mx[0] = fmaxf(mx[0], f);
                            }
                        }
                    }
                }
            }
            const float vmin = warp_min(fminf(mn[0], mn[1])), vmax = warp_max(fmaxf(mx[0], mx[1]));
            if (lane == 0) { red[(er * 2 * kH + rslot) * 2] = vmin; red[(er * 2 * kH + rslot) * 2 + 1] = vmax; }
            bar_sync_named(2 + er, kRowThreads);                     // the epilogue warps of this row
            float a = 0.0f, b = 0.0f;
#pragma unroll
            for (int g = 0; g < 2 * kH; ++g) { a = fminf(a, red[(er * 2 * kH + g) * 2]); b = fmaxf(b, red[(er * 2 * kH + g) * 2 + 1]); }
            const TokenRowParams rp = token_row_params(a, b, p.clip, p.c);
            const long row = 2 * pair + er;
            if (et == 0 && row < p.M && ok) { p.scale[row] = rp.scale; p.zero[row] = __float2half_rn(rp.zero); }
            // ---- pass 2: codes.  v * rd, clamped only when the row needs it, + 1.5 * 2^23 (rint in the low mantissa bits),
            //      + zero (exact): the low byte of the sum's bit pattern is the code ----
            {
                const uint64_t rd2 = pack2(rp.rd, rp.rd), magic2 = pack2(12582912.0f, 12582912.0f), z2 = pack2(rp.zero, rp.zero);
                const float lo = -rp.zero, hi = 15.0f - rp.zero;
                uint8_t *dst = cb + er * K + ej;
                const bool clamp = rp.clamp;                         // row-uniform; almost never set when nothing is clipped
                auto codes16 = [&](const uint32_t (&v)[16], int c) {
                    uint8_t *d = dst + c * 1024;
                    const int nv = F - c * 16;
                    uint64_t y[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) y[j] = mul2(pack2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), rd2);
                    if (__builtin_expect(clamp, 0)) {                // a real branch: the common path carries no min/max instructions
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float f0, f1;
                            unpack2(y[j], f0, f1);
                            y[j] = pack2(fmaxf(fminf(f0, hi), lo), fmaxf(fminf(f1, hi), lo));
                        }
                    }
                    uint32_t r[16];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float r0, r1;
                        unpack2(add2(add2(y[j], magic2), z2), r0, r1);
                        r[2 * j] = __float_as_uint(r0); r[2 * j + 1] = __float_as_uint(r1);
                    }
                    if (nv >= 16) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) d[j * 64] = (uint8_t)r[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (j < nv) d[j * 64] = (uint8_t)r[j];
                    }
                };
                uint32_t va[16], vb[16];
                tmem_ld16(taddr + c_lo * 16, va);
                for (int c = c_lo; c < c_hi; c += 2) {
                    tc_wait_ld();
                    if (c + 1 < c_hi) tmem_ld16(taddr + (c + 1) * 16, vb);
                    codes16(va, c);
                    if (c + 1 < c_hi) {
                        tc_wait_ld();
                        if (c + 2 < c_hi) tmem_ld16(taddr + (c + 2) * 16, va);
                        codes16(vb, c + 1);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));              // this warp is done with the TMEM buffer
            bar_sync_named(2 + er, kRowThreads);                     // the codes of this row are staged
            if (row < p.M && ok) {
                const int per_row = K >> 4;
                uint2 *qrow = reinterpret_cast<uint2 *>(p.q + row * (long)(K >> 1));
                for (int i = et; i < per_row; i += kRowThreads) qrow[i] = pack16(*reinterpret_cast<const uint4 *>(cb + er * K + 16 * i));
            }
            // (the next pair's first named barrier orders these reads before the next writes of cb and red)
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
