// Full-width online Hadamard (binary32, matmul_hadU's order) fused with the per-token asymmetric
// int4 quantiser and nibble packing.
//
// One CTA per token row, T = K/64 threads, every thread owns 64 values in registers at each step:
//   pass 1  the row arrives in shared memory by coalesced 16-byte cp.async; butterfly bits 0-5 on 64
//           consecutive inputs per thread (eight 128-bit shared loads);
//   pass 2  bits 6..6+B2-1 after one transpose through padded shared memory;
//   pass 3  bits 12..12+B3-1 (K > 4096 only) after a second transpose;
//   factor  the kfac x kfac +-1 matrix across the K/kfac-long chunks (K = 11008, 14336, 28672 ...),
//           accumulated k' ascending in binary32, signs kept as bit rows in shared memory;
//   quant   row min/max -> scale (f16), zero-point, codes from the registers, staged as bytes in
//           shared memory only to be packed two per byte and stored with 64-bit writes.
// All butterflies run on packed binary32 pairs (add.rn.f32x2 / fma.rn.f32x2), so every result is
// the IEEE sum or difference of its two inputs, in ascending bit order: bit-exact with the oracle.
// Shared memory is used only for the transposes between register passes.
#include "token_common.cuh"
#include <stdlib.h>

namespace flh {
namespace {

// ---- 64 registers, butterfly over the low NST bits of the register index --------------------
template <int NST>
__device__ __forceinline__ void bfly_regs(float (&x)[64]) {
    if (NST >= 1) {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const float a = x[2 * k], b = x[2 * k + 1];
            x[2 * k] = __fadd_rn(a, b);
            x[2 * k + 1] = __fsub_rn(a, b);
        }
    }
    if (NST >= 2) {
        uint64_t p[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) p[k] = pack2(x[2 * k], x[2 * k + 1]);
#pragma unroll
        for (int s = 1; s < NST; ++s) {
            const int h = 1 << (s - 1);
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
}

// Shared-memory position of element e (0..63) of 64-chunk `chunk`: 68 words per chunk keeps the
// 128-bit stores of pass 1 conflict-free; for B2 < 5 one more word per chunk (two for B2 = 1),
// granted in blocks of 2^B2 chunks, spreads the 2^B2-strided reads of pass 2 over the banks.
// A row never needs more than 70 words per chunk.
template <int B2>
__device__ __forceinline__ int phys(int chunk, int e) {
    if (B2 == 1) return 68 * chunk + ((chunk >> 1) << 2) + e;      // keeps 16-byte alignment
    if (B2 > 1 && B2 < 5) return 68 * chunk + ((chunk >> B2) << B2) + e;
    return 68 * chunk + e;
}

// 32-bit words of the transpose buffer of a row of T 64-chunks (see phys): 68 per chunk, plus the extra
// padding of the small-B2 layouts, plus slack.
template <int B2>
__host__ __device__ inline size_t buf_words(int T) {
    return (size_t)T * (B2 == 1 ? 70 : ((B2 > 1 && B2 < 5) ? 69 : 68)) + 64;
}

struct TokenParams {
    const void *x;
    long ld;
    int bf16;
    int n;         // K
    int T;         // n / 64 working threads
    int kfac;
    int P;         // n / kfac
    const uint32_t *sign_bits;
    long M;                          // rows; CTAs walk rows blockIdx.x, blockIdx.x + gridDim.x, ...
    const __nv_bfloat16 *sign_mat;   // kp x kp matrix of +-1 (0 in the padding), row-major; tensor-core factor stage
    int kp;                          // kfac rounded up to a multiple of 16
    int factor_exact;                // 1: sequential binary32 factor stage on the CUDA cores (bit-exact with the oracle)
    float clip;
    float c;       // sqrtf(n) with the transform, 1 without
    uint8_t *q;
    __half *scale;
    __half *zero;
};

// B2/B3: bits handled by passes 2/3.  FACTOR: kfac > 1.  HAD: transform at all.
// With the transform, K <= 4096 and no factor stage mean at most 64 working threads: ask for ten CTAs per SM (twelve fit only with spills and measured slower).
template <int B2, int B3, bool FACTOR, bool HAD>
__global__ void __launch_bounds__((HAD && B3 == 0 && !FACTOR) ? 64 : 512, (HAD && B3 == 0 && !FACTOR) ? 10 : 1)
quant_token_asym_kernel(const TokenParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *buf = reinterpret_cast<float *>(smem_raw);
    __shared__ float red[2][32];
    __shared__ float bcast[3];

    const int t = threadIdx.x;
    const int lane = t & 31, warp = t >> 5;
    const bool active = t < p.T;

    // Tensor-core factor stage: the sign matrix lives in shared memory for the whole (persistent) CTA,
    // rows padded by 16 bytes so that ldmatrix reads are conflict-free.
    const int smat_ld = p.kp + 8;                                              // bf16 elements per row
    __nv_bfloat16 *smat = reinterpret_cast<__nv_bfloat16 *>(smem_raw + ((buf_words<B2>(p.T) * 4 + 15) & ~(size_t)15));
    if (HAD && FACTOR && !p.factor_exact) {
        const int cpr = p.kp >> 3;                                             // 16-byte chunks per row
        for (int i = t; i < p.kp * cpr; i += blockDim.x) {
            const int r = i / cpr, c = i - r * cpr;
            *reinterpret_cast<uint4 *>(smat + r * smat_ld + c * 8) =
                *reinterpret_cast<const uint4 *>(p.sign_mat + (size_t)r * p.kp + c * 8);
        }
        __syncthreads();
    }

    for (long row = blockIdx.x; row < p.M; row += gridDim.x) {
    float x[64];

    // ---------------- pass 1: load 64 consecutive inputs, bits 0-5 -------------------------
    // The row is copied into shared memory with coalesced 16-byte cp.async (chunk c of 128-byte line L
    // lands at chunk c ^ (L & 7), so that a thread reading its own line is conflict-free), then every
    // thread picks up its 64 consecutive values.
    {
        const uint16_t *src = static_cast<const uint16_t *>(p.x) + row * p.ld + t * 8;
        const uint32_t sbase = smem_u32(smem_raw);
        const int c = t & 7, dl = blockDim.x >> 3, nch = p.n >> 3;
        int line = t >> 3;
        for (int ch = t; ch < nch; ch += blockDim.x, line += dl, src += blockDim.x * 8) {
            const uint32_t dst = sbase + (((line << 3) + (c ^ (line & 7))) << 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
        }
        asm volatile("cp.async.commit_group;" ::);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }
    if (active) {
        uint4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
            v[c] = *reinterpret_cast<const uint4 *>(smem_raw + ((t << 3) + (c ^ (t & 7))) * 16);
        if (p.bf16) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    x[8 * c + 2 * j] = __uint_as_float(w[j] << 16);
                    x[8 * c + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                }
            }
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
                    x[8 * c + 2 * j] = f.x;
                    x[8 * c + 2 * j + 1] = f.y;
                }
            }
        }
        if (HAD) bfly_regs<6>(x);
    }
    __syncthreads();      // the staged row is consumed; its space is reused below

    // element index of register idx once all passes are done: base + stride pattern below
    // (computed per section); codes are staged at cb[element index].
    int ebase = 64 * t;      // pass-1 layout: idx -> 64 t + idx

    if (HAD && (B2 > 0 || FACTOR)) {
        if (active) {
#pragma unroll
            for (int e = 0; e < 64; e += 4)
                *reinterpret_cast<float4 *>(buf + phys<B2>(t, e)) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
        }
        __syncthreads();
    }

    // ---------------- pass 2: bits 6 .. 6+B2-1 ---------------------------------------------
    // register idx = r * 2^B2 + m  <->  element hi * 2^(6+B2) + m * 64 + r * 2^B2 + w
    if (HAD && B2 > 0) {
        constexpr int NM = 1 << B2;
        const int w = t & (NM - 1), hi = t >> B2;
        if (active) {
#pragma unroll
            for (int idx = 0; idx < 64; ++idx) {
                const int m = idx & (NM - 1), r = idx >> B2;
                x[idx] = buf[phys<B2>(hi * NM + m, r * NM + w)];
            }
            bfly_regs<B2>(x);
        }
        ebase = (hi << (6 + B2)) + w;
        if (B3 > 0 || FACTOR) {
            __syncthreads();   // everyone has read before anyone overwrites
            if (active) {
#pragma unroll
                for (int idx = 0; idx < 64; ++idx) {
                    const int m = idx & (NM - 1), r = idx >> B2;
                    buf[phys<B2>(hi * NM + m, r * NM + w)] = x[idx];
                }
            }
            __syncthreads();
        }
    }

    // ---------------- pass 3: bits 12 .. 12+B3-1 (B2 == 6) ----------------------------------
    // register idx = r * 2^B3 + m  <->  element hi * 2^(12+B3) + m * 4096 + r * 64 * 2^B3 + w
    if (HAD && B3 > 0) {
        constexpr int NM = 1 << B3;
        const int w = t & (64 * NM - 1), hi = t >> (6 + B3);
        if (active) {
#pragma unroll
            for (int idx = 0; idx < 64; ++idx) {
                const int m = idx & (NM - 1), r = idx >> B3;
                const int chunk = (hi << (6 + B3)) + m * 64 + r * NM + (w >> 6);
                x[idx] = buf[phys<B2>(chunk, w & 63)];
            }
            bfly_regs<B3>(x);
        }
        ebase = (hi << (12 + B3)) + w;
        if (FACTOR) {
            __syncthreads();
            if (active) {
#pragma unroll
                for (int idx = 0; idx < 64; ++idx) {
                    const int m = idx & (NM - 1), r = idx >> B3;
                    const int chunk = (hi << (6 + B3)) + m * 64 + r * NM + (w >> 6);
                    buf[phys<B2>(chunk, w & 63)] = x[idx];
                }
            }
            __syncthreads();
        }
    }

    // ---------------- factor stage: y[k P + j] = sum_k' S[k][k'] in[k' P + j] ----------------
    // thread <-> (kb, w): k = 4 kb + v (v < 4); j = 2 w + b + (P/8) u (b < 2, u < 8);
    // register idx = v * 16 + 2 u + b.
    int f_kb = 0, f_w = 0;
    if (HAD && FACTOR && p.factor_exact) {
        const int words = (p.kfac + 31) >> 5;
        uint32_t *sgn = reinterpret_cast<uint32_t *>(buf + buf_words<B2>(p.T));   // after the data area
        for (int i = t; i < p.kfac * words; i += blockDim.x) sgn[i] = p.sign_bits[i];
        __syncthreads();
        const int Wd = p.P >> 4;
        f_w = t % Wd;
        f_kb = t / Wd;
        if (active) {
            uint64_t acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0ull;
            const int jstep = p.P >> 3;
            for (int kk0 = 0; kk0 < p.kfac; kk0 += 32) {
                uint32_t sw[4];
#pragma unroll
                for (int v = 0; v < 4; ++v) sw[v] = sgn[(4 * f_kb + v) * words + (kk0 >> 5)];
                const int kend = min(32, p.kfac - kk0);
                for (int kb = 0; kb < kend; ++kb) {
                    const int kk = kk0 + kb;
                    uint64_t in[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int j = 2 * f_w + jstep * u;
                        const int i = kk * p.P + j;
                        in[u] = *reinterpret_cast<const uint64_t *>(buf + phys<B2>(i >> 6, i & 63));
                    }
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const uint32_t s = 0x3f800000u | ((sw[v] >> kb) << 31);
                        uint64_t s2;
                        asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "r"(s));
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[v * 8 + u]) : "l"(s2), "l"(in[u]));
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) unpack2(acc[i], x[2 * i], x[2 * i + 1]);
        }
    }

    // ---------------- factor stage on the tensor cores ---------------------------------------
    // y = S x with S the kfac x kfac sign matrix: mma.sync m16n8k16 bf16 -> f32, rows = output chunk k,
    // contraction = input chunk k', columns = position j inside the chunk.  x is binary32; it is split
    // EXACTLY into three bfloat16 terms (8 + 8 + 8 significand bits), the products with +-1 are exact and
    // the sums accumulate in binary32, so the result differs from the sequential sum only by the order of
    // the binary32 roundings.  A warp owns 8 columns: it reads them for every k', keeps all output rows in
    // registers (up to 11 tiles x 4), then writes them back in place.
    if (HAD && FACTOR && !p.factor_exact) {
        const int MTr = p.kp >> 4;
        const int ntiles = p.P >> 3, nwarps = blockDim.x >> 5;
        const int g = lane >> 2, tq = lane & 3;
        for (int nt = warp; nt < ntiles; nt += nwarps) {
            float acc[11][4];
#pragma unroll
            for (int mt = 0; mt < 11; ++mt)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[mt][q] = 0.0f;
            const int j = nt * 8 + g;
            for (int kt = 0; kt < MTr; ++kt) {
                float v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int kq = kt * 16 + 2 * tq + (q & 1) + 8 * (q >> 1);
                    const int i = kq * p.P + j;
                    v[q] = kq < p.kfac ? buf[phys<B2>(i >> 6, i & 63)] : 0.0f;
                }
                uint32_t b[3][2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float lo = v[2 * h], hi = v[2 * h + 1];
#pragma unroll
                    for (int sp = 0; sp < 3; ++sp) {
                        const __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
                        const uint32_t bits = *reinterpret_cast<const uint32_t *>(&pr);
                        b[sp][h] = bits;
                        lo = __fsub_rn(lo, __uint_as_float(bits << 16));
                        hi = __fsub_rn(hi, __uint_as_float(bits & 0xffff0000u));
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 11; ++mt) {
                    if (mt < MTr) {
                        uint32_t a0, a1, a2, a3;
                        const uint32_t addr = smem_u32(smat + (mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * smat_ld + kt * 16 + 8 * (lane >> 4));
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(addr));
#pragma unroll
                        for (int sp = 0; sp < 3; ++sp)
                            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                         : "+f"(acc[mt][0]), "+f"(acc[mt][1]), "+f"(acc[mt][2]), "+f"(acc[mt][3])
                                         : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b[sp][0]), "r"(b[sp][1]));
                    }
                }
            }
            __syncwarp();           // every lane has read its columns before any lane overwrites them
            const int j0 = nt * 8 + 2 * tq;
#pragma unroll
            for (int mt = 0; mt < 11; ++mt) {
                if (mt < MTr) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int k = mt * 16 + g + 8 * h;
                        if (k < p.kfac) {
                            const int i = k * p.P + j0;
                            *reinterpret_cast<float2 *>(buf + phys<B2>(i >> 6, i & 63)) = make_float2(acc[mt][2 * h], acc[mt][2 * h + 1]);
                        }
                    }
                }
            }
        }
        __syncthreads();
        if (active) {               // back to 64 consecutive values per thread for the quantiser
#pragma unroll
            for (int e = 0; e < 64; e += 4) {
                const float4 f = *reinterpret_cast<const float4 *>(buf + phys<B2>(t, e));
                x[e] = f.x; x[e + 1] = f.y; x[e + 2] = f.z; x[e + 3] = f.w;
            }
        }
    }

    // ---------------- row min / max ---------------------------------------------------------
    float vmin = 0.0f, vmax = 0.0f;
    if (active) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) { vmin = min3(vmin, x[i], x[i + 1]); vmax = max3(vmax, x[i], x[i + 1]); }
    }
    vmin = warp_min(vmin); vmax = warp_max(vmax);
    if (lane == 0) { red[0][warp] = vmin; red[1][warp] = vmax; }
    __syncthreads();            // also: all reads of buf are complete, cb may alias it
    if (warp == 0) {
        // one warp finishes the reduction and derives scale, reciprocal and zero-point for the row
        const int nw = (blockDim.x + 31) >> 5;
        float a = lane < nw ? red[0][lane] : 0.0f;
        float b = lane < nw ? red[1][lane] : 0.0f;
        a = warp_min(a); b = warp_max(b);
        if (lane == 0) {
            const TokenRowParams rp = token_row_params(a, b, p.clip, p.c);
            bcast[0] = rp.rd; bcast[1] = rp.zero; bcast[2] = rp.clamp ? 1.0f : 0.0f;
            p.scale[row] = rp.scale; p.zero[row] = __float2half_rn(rp.zero);
        }
    }
    __syncthreads();
    const float rd = bcast[0], zf = bcast[1];
    const bool clamp_codes = bcast[2] != 0.0f;

    // codes: clamp(rint(z * rd), -zero, 15 - zero) + zero; adding 1.5 * 2^23 rounds to the
    // nearest integer (ties to even) and leaves it in the low mantissa bits.
    uint8_t *cb = smem_raw;
    if (active) {
        const float lo = -zf, hi = 15.0f - zf;
        const float magic = 12582912.0f;
        const int zi = (int)zf;
        const uint64_t rd2 = pack2(rd, rd), magic2 = pack2(magic, magic);
        // The row leader has checked whether any code of this row can leave 0..15 (it cannot, for almost
        // every row, when nothing is clipped); only then are the values clamped before rounding.
#pragma unroll
        for (int idx = 0; idx < 64; idx += 2) {
            float v0, v1;
            unpack2(mul2(pack2(x[idx], x[idx + 1]), rd2), v0, v1);
            if (clamp_codes) { v0 = fmaxf(fminf(v0, hi), lo); v1 = fmaxf(fminf(v1, hi), lo); }
            float r0, r1;
            unpack2(add2(pack2(v0, v1), magic2), r0, r1);
            // low byte of (bits + zero) = rint(v) + zero, already in 0..15
            const int code[2] = {__float_as_int(r0) + zi, __float_as_int(r1) + zi};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int id = idx + u;
                int e;
                if (HAD && FACTOR && p.factor_exact) {
                    const int v4 = id >> 4, uu = (id >> 1) & 7, b = id & 1;
                    e = (4 * f_kb + v4) * p.P + 2 * f_w + b + (p.P >> 3) * uu;
                } else if (HAD && FACTOR) {
                    e = 64 * t + id;
                } else if (HAD && B3 > 0) {
                    const int m = id & ((1 << B3) - 1), r = id >> B3;
                    e = ebase + m * 4096 + r * (64 << B3);
                } else if (HAD && B2 > 0) {
                    const int m = id & ((1 << B2) - 1), r = id >> B2;
                    e = ebase + m * 64 + (r << B2);
                } else {
                    e = ebase + id;
                }
                cb[e] = (uint8_t)code[u];
            }
        }
    }
    __syncthreads();
    // pack 16 staged codes into 8 bytes, coalesced 64-bit stores
    uint2 *qrow = reinterpret_cast<uint2 *>(p.q + row * (long)(p.n >> 1));
    for (int c = t; c < (p.n >> 4); c += blockDim.x) {
        const uint4 cv = *reinterpret_cast<const uint4 *>(cb + 16 * c);
        const uint32_t w[4] = {cv.x, cv.y, cv.z, cv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t tt = w[j] | (w[j] >> 4);
            o[j] = __byte_perm(tt, 0, 0x4420);            // bytes 0 and 2 -> a 16-bit pair
        }
        qrow[c] = make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
    }
    __syncthreads();            // the staged codes are consumed before the next row reuses the space
    }                           // row loop
}

template <int B2, int B3, bool FACTOR, bool HAD>
int launch_one(const TokenParams &p, long M, cudaStream_t stream) {
    int threads = ((p.T + 31) / 32) * 32;
    if (FACTOR && !p.factor_exact && threads < 256) threads = 256;     // eight warps for the tensor-core factor stage
    size_t smem = (size_t)p.n * 2;                               // staged input row (codes reuse it)
    if (HAD && (B2 > 0 || FACTOR)) {
        smem = buf_words<B2>(p.T) * 4;
        if (FACTOR && p.factor_exact) smem += (size_t)p.kfac * ((p.kfac + 31) / 32) * 4;
        if (FACTOR && !p.factor_exact) smem = ((smem + 15) & ~(size_t)15) + (size_t)p.kp * (p.kp + 8) * 2;
        if (smem < (size_t)p.n * 2) smem = (size_t)p.n * 2;
    }
    auto kern = quant_token_asym_kernel<B2, B3, FACTOR, HAD>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "quant_token smem attribute");
    }
    long grid = M;
    if (FACTOR && !p.factor_exact) {        // persistent: the sign matrix is staged once per CTA
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, smem) != cudaSuccess || occ < 1) occ = 1;
        if (grid > (long)occ * kNumSMs) grid = (long)occ * kNumSMs;
    }
    TokenParams q = p;
    q.M = M;
    kern<<<(unsigned)grid, threads, smem, stream>>>(q);
    return cuda_status(cudaGetLastError(), "quant_token_asym launch");
}

}  // namespace

int launch_quant_token_warp(const void *x, int in_dtype, long M, long K, long ld, int hadamard, float norm_eps, float clip,
                            uint8_t *q, void *scale, void *zero, cudaStream_t stream);

int launch_quant_token_factor(const void *x, int in_dtype, long M, long K, long ld, int kfac, const void *sign_mat_bf16,
                              float clip, uint8_t *q, void *scale, void *zero, cudaStream_t stream);

// Rows from which the warp-per-row kernel (K = 4096) is used; below it the 64-thread kernel spreads a
// small batch over more SMs.  FLH_B200_TOKEN_WARP_MIN_M overrides it (tuning aid).
static long token_warp_min_rows() {
    static long v = -1;
    if (v < 0) {
        const char *e = getenv("FLH_B200_TOKEN_WARP_MIN_M");
        v = e ? atol(e) : 512;
        if (v < 0) v = 0;
    }
    return v;
}

int launch_quant_token_tc(const void *x, int in_dtype, long M, long K, long ld, int kfac, const uint32_t *sign_bits,
                          float clip, uint8_t *q, void *scale, void *zero, cudaStream_t stream);

int launch_quant_token_asym(const void *x, int in_dtype, long M, long K, long ld, int hadamard,
                            int kfac, const uint32_t *sign_bits, float clip, uint8_t *q,
                            void *scale, void *zero, cudaStream_t stream) {
    if (hadamard == 1) {
        // default transform: the high part on the tensor cores, for every batch size (K = P * 64, P <= 512)
        int rc;
        rc = launch_quant_token_tc(x, in_dtype, M, K, ld, kfac, sign_bits, clip, q, scale, zero, stream);
        if (rc != -1000) return rc;
    }
    if ((!hadamard || kfac == 1) && (K == 4096 || K == 8192) && M >= token_warp_min_rows() &&
        (hadamard || (reinterpret_cast<uintptr_t>(q) & 15) == 0))          // its untransformed form stores 16 bytes at a time
        return launch_quant_token_warp(x, in_dtype, M, K, ld, hadamard, -1.0f, clip, q, scale, zero, stream);
    if (hadamard == 1 && kfac >= 64 && K == (long)kfac * 64 && M >= 256) {
        // K = kfac * 64 with a large factor (11008 = 172 * 64), prefill-size batches: butterflies + the factor on
        // tcgen05, two rows per step of a persistent CTA (its set-up costs more than a decode-size batch)
        const size_t bits_bytes = ((size_t)kfac * ((kfac + 31) / 32) * 4 + 15) / 16 * 16;
        const int rc = launch_quant_token_factor(x, in_dtype, M, K, ld, kfac, reinterpret_cast<const uint8_t *>(sign_bits) + bits_bytes,
                                                 clip, q, scale, zero, stream);
        if (rc != -1000) return rc;
    }
    TokenParams p;
    // factor table layout (flh_b200_pack_signs): bit rows, then (16-byte aligned) the bf16 matrix
    p.kp = (kfac + 15) / 16 * 16;
    // the tensor-core factor stage pays off for the large orders (108 ... 172); the small ones (12 ... 60) are
    // cheaper summed directly, which is also the oracle's order
    {
        static int min_kfac = -1;
        if (min_kfac < 0) { const char *e = getenv("FLH_B200_FACTOR_TC_MIN_KFAC"); min_kfac = e ? atoi(e) : 64; }
        p.factor_exact = hadamard == 2 || kfac < min_kfac;
    }
    {
        const size_t bits_bytes = ((size_t)kfac * ((kfac + 31) / 32) * 4 + 15) / 16 * 16;
        p.sign_mat = reinterpret_cast<const __nv_bfloat16 *>(reinterpret_cast<const uint8_t *>(sign_bits) + bits_bytes);
    }
    p.x = x; p.ld = ld; p.bf16 = in_dtype == FLH_B200_BF16; p.n = (int)K; p.T = (int)(K / 64);
    p.kfac = kfac; p.P = (int)(K / kfac); p.sign_bits = sign_bits; p.clip = clip;
    p.c = hadamard ? sqrtf((float)K) : 1.0f;
    p.q = q; p.scale = static_cast<__half *>(scale); p.zero = static_cast<__half *>(zero);
    if (!hadamard) return launch_one<0, 0, false, false>(p, M, stream);
    int logp = 0;
    while ((1 << logp) < p.P) ++logp;
    const int b2 = logp - 6 > 6 ? 6 : logp - 6;
    const int b3 = logp - 12 > 0 ? logp - 12 : 0;
    if (kfac > 1) {
        switch (b2) {
            case 0: return launch_one<0, 0, true, true>(p, M, stream);
            case 1: return launch_one<1, 0, true, true>(p, M, stream);
            case 2: return launch_one<2, 0, true, true>(p, M, stream);
            case 3: return launch_one<3, 0, true, true>(p, M, stream);
            case 4: return launch_one<4, 0, true, true>(p, M, stream);
            case 5: return launch_one<5, 0, true, true>(p, M, stream);
            default: return launch_one<6, 0, true, true>(p, M, stream);
        }
    }
    if (b3 == 0) {
        switch (b2) {
            case 0: return launch_one<0, 0, false, true>(p, M, stream);
            case 1: return launch_one<1, 0, false, true>(p, M, stream);
            case 2: return launch_one<2, 0, false, true>(p, M, stream);
            case 3: return launch_one<3, 0, false, true>(p, M, stream);
            case 4: return launch_one<4, 0, false, true>(p, M, stream);
            case 5: return launch_one<5, 0, false, true>(p, M, stream);
            default: return launch_one<6, 0, false, true>(p, M, stream);
        }
    }
    switch (b3) {
        case 1: return launch_one<6, 1, false, true>(p, M, stream);
        case 2: return launch_one<6, 2, false, true>(p, M, stream);
        default: return launch_one<6, 3, false, true>(p, M, stream);
    }
}

bool quant_token_tc_takes(long K, int kfac);

// The __global__ function launch_quant_token_asym picks for a shape (for pointers aligned to 16 bytes).
const char *quant_token_kernel_name(long M, long K, int hadamard, int kfac) {
    if (!hadamard) kfac = 1;
    if (hadamard == 1 && quant_token_tc_takes(K, kfac)) return "quant_token_tc_kernel";
    if ((!hadamard || kfac == 1) && (K == 4096 || K == 8192) && M >= token_warp_min_rows()) return "quant_token_warp_kernel";
    if (hadamard == 1 && kfac >= 64 && K == (long)kfac * 64 && M >= 256) return "quant_token_factor_kernel";
    return "quant_token_asym_kernel";
}

}  // namespace flh
