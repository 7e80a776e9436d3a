/*
 * CPU oracle for the FLH W4A4 hot path: online Hadamard + int4 activation
 * quantiser + int4 x int4 GEMM with fused dequantisation.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is a plain-C restatement of the
 * reference's algorithms, used only as the checker by the tests, by the smoke
 * entry and by the CPU-baseline leg of the benchmark.  Nothing in the shipped
 * library links, imports or calls it.
 *
 * Every function names the reference source it restates (paths are relative to
 * the FLH repository root).
 *
 * Arithmetic conventions
 *   - binary16 values travel as uint16_t bit patterns; all binary16 arithmetic
 *     is "exact operation, one rounding to nearest-even", which is what the
 *     device's add.f16 / sub.f16 / cvt.rn.f16.f32 do.
 *   - compile with -ffp-contract=off so that no multiply-add is fused unless
 *     fmaf() is written out.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

static inline f16 h_from_bits(uint16_t b) { f16 h; memcpy(&h, &b, 2); return h; }
static inline uint16_t h_bits(f16 h) { uint16_t b; memcpy(&b, &h, 2); return b; }
static inline float h2f(uint16_t b) { return (float)h_from_bits(b); }
static inline uint16_t f2h(float f) { return h_bits((f16)f); }            /* cvt.rn.f16.f32 */

static inline float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t f2bf(float f) {                                       /* cvt.rn.bf16.f32 */
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* binary16 add/sub: the float sum of two binary16 values rounded once to float
 * and once more to binary16 equals the correctly rounded binary16 sum
 * (24 >= 2*11+2), i.e. __hadd / __hsub. */
static inline uint16_t hadd(uint16_t a, uint16_t b) { return f2h(h2f(a) + h2f(b)); }
static inline uint16_t hsub(uint16_t a, uint16_t b) { return f2h(h2f(a) - h2f(b)); }

/* __hdiv as cuda_fp16.hpp defines it for device code: reciprocal, multiply,
 * round to binary16, and one Newton correction when the result is a tiny
 * subnormal.  The device takes the reciprocal with rcp.approx.ftz.f32 (error
 * <= 1 ulp, not reproducible on a CPU); this restatement and the B200 kernels
 * use the correctly rounded reciprocal instead. */
static inline uint16_t hdiv_rcp(float fa, float fb, float rcp) {
    float fv = rcp * fa;
    uint16_t v = f2h(fv);
    uint16_t a = v & 0x7fffu;
    if (a != 0 && a < 0x008Fu) {
        float err = fmaf(-fb, fv, fa);
        fv = fmaf(rcp, err, fv);
        v = f2h(fv);
    }
    return v;
}
static inline uint16_t hdiv(uint16_t a, uint16_t b) {
    float fb = h2f(b);
    return hdiv_rcp(h2f(a), fb, 1.0f / fb);
}

/* __half2int_rn */
static inline int h2i_rn(uint16_t h) { return (int)nearbyintf(h2f(h)); }

static inline int ilog2(long n) { int l = 0; while ((1L << l) < n) ++l; return l; }

/* ------------------------------------------------------------------------- */
/* In-place un-normalised binary16 Walsh-Hadamard transform of rows of n
 * (n = 32, 64 or 128; any power of two works).
 * Restates hadamard_transform_kernel_optimized, flh/kernels/cuda_had_kernel.cu:190-268
 * (and the 64/32 copies): stage s pairs the elements whose index differs in
 * bit s, s ascending; the lower index receives a+b, the upper a-b; every
 * add/sub rounds to binary16 (hadamard_mult_thread :124-146, hadamard_mult_warp
 * :150-186 of that file; the same order as flh/kernels/had_and_quant.cu:13-56). */
static void fht_row_f16(uint16_t *x, int n) {
    for (int s = 1; s < n; s <<= 1)
        for (int i = 0; i < n; ++i)
            if (!(i & s)) {
                uint16_t a = x[i], b = x[i + s];
                x[i] = hadd(a, b);
                x[i + s] = hsub(a, b);
            }
}

void flh_oracle_fht_f16(uint16_t *x, long rows, int n) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) fht_row_f16(x + r * n, n);
}

/* ------------------------------------------------------------------------- */
/* Fused (optional) Hadamard + symmetric int4 quantiser + nibble packing on rows
 * of gs binary16 values (gs = 32, 64 or 128).
 * Restates had_and_quant_kernel, flh/kernels/had_and_quant.cu:61-155 (and
 * had_and_quant_kernel_gs, flh/kernels/had_and_quant_gs.cu:84-185; without the
 * transform: quant_and_pack_kernel, flh/kernels/quant_and_pack.cu:8-96):
 *   max = max |x| in binary16; scale = __hdiv(max, 7); scale <= half(1e-6) -> 1;
 *   q = clamp(__half2int_rn(__hdiv(x, scale)), -8, 7);
 *   byte j = (q[2j] & 15) | (q[2j+1] << 4); the raw scale is returned. */
void flh_oracle_quant_group_sym(const uint16_t *x, long rows, int gs, int hadamard,
                                uint8_t *q_out, uint16_t *scale_out) {
    const uint16_t seven = f2h(7.0f), tiny = f2h(1e-6f), one = f2h(1.0f);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        uint16_t v[128];
        memcpy(v, x + r * gs, (size_t)gs * 2);
        if (hadamard) fht_row_f16(v, gs);
        float m = 0.0f;
        for (int i = 0; i < gs; ++i) { float a = fabsf(h2f(v[i])); if (a > m) m = a; }
        uint16_t scale = hdiv(f2h(m), seven);
        if (h2f(scale) <= h2f(tiny)) scale = one;
        scale_out[r] = scale;
        float fs = h2f(scale), rcp = 1.0f / fs;
        for (int i = 0; i < gs; i += 2) {
            int q0 = h2i_rn(hdiv_rcp(h2f(v[i]), fs, rcp));
            int q1 = h2i_rn(hdiv_rcp(h2f(v[i + 1]), fs, rcp));
            q0 = q0 < -8 ? -8 : (q0 > 7 ? 7 : q0);
            q1 = q1 < -8 ? -8 : (q1 > 7 ? 7 : q1);
            q_out[r * (gs / 2) + i / 2] = (uint8_t)((q0 & 15) | ((q1 & 15) << 4));
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Full-width Hadamard in binary32, un-normalised: n = kfac * p, p a power of two.
 * Restates matmul_hadU, flh/functional/hadamard.py:92-113: butterflies over the
 * contiguous chunks of p (stage s pairs indices differing in bit s, s ascending,
 * sum to the lower index), then y[k*p+j] = sum_k' hadK[k][k'] * x[k'*p+j].
 * The reference evaluates that last product with a library matmul whose
 * summation order is unspecified; here it is k' ascending in binary32 starting
 * from +0, which is also the order of the B200 kernel.
 * signs: kfac*kfac int8 entries (+1/-1), row-major; NULL when kfac == 1. */
static void had_full_row_f32(float *x, float *tmp, long n, int kfac, const int8_t *signs) {
    long p = n / kfac;
    for (long c = 0; c < kfac; ++c) {
        float *y = x + c * p;
        for (long s = 1; s < p; s <<= 1)
            for (long i = 0; i < p; ++i)
                if (!(i & s)) { float a = y[i], b = y[i + s]; y[i] = a + b; y[i + s] = a - b; }
    }
    if (kfac > 1) {
        for (int k = 0; k < kfac; ++k)
            for (long j = 0; j < p; ++j) {
                float acc = 0.0f;
                for (int kk = 0; kk < kfac; ++kk) {
                    float v = x[kk * p + j];
                    acc = acc + (signs[k * kfac + kk] < 0 ? -v : v);
                }
                tmp[k * p + j] = acc;
            }
        memcpy(x, tmp, (size_t)n * 4);
    }
}

/* Normalised full Hadamard, binary32 in/out: y = H x / sqrt(n), the division as
 * the reference writes it (flh/functional/hadamard.py:113). */
void flh_oracle_had_full_f32(float *x, long rows, long n, int kfac, const int8_t *signs) {
    const float c = sqrtf((float)n);
#pragma omp parallel
    {
        float *tmp = (float *)malloc((size_t)n * 4);
#pragma omp for schedule(static)
        for (long r = 0; r < rows; ++r) {
            float *y = x + r * n;
            had_full_row_f32(y, tmp, n, kfac, signs);
            for (long i = 0; i < n; ++i) y[i] = y[i] / c;
        }
        free(tmp);
    }
}

/* ------------------------------------------------------------------------- */
/* (Optional full Hadamard +) per-token asymmetric int4 quantiser + packing.
 * Restates ActQuantizer.find_params / asym_quant, fake_quant/quant_utils.py:94-128
 * and :17-21, applied to matmul_hadU's output:
 *   xmin = min(row, 0) * clip, xmax = max(row, 0) * clip; both 0 -> (-1, +1);
 *   scale = (xmax - xmin) / 15; zero = round(-xmin / scale);
 *   q = clamp(round(x / scale) + zero, 0, 15).
 * The reference keeps the scale in binary32; the packed interface stores it as
 * binary16, so the scale is rounded to binary16 FIRST and the codes and the
 * zero-point are computed against the rounded value (the stored triple then
 * dequantises consistently).
 *
 * exact_norm = 1: y = Hx / sqrt(n) is formed per element as the reference does,
 *                 then quantised (used to pin this file against the reference).
 * exact_norm = 0: the B200 kernel's arithmetic: the un-normalised transform z is
 *                 quantised directly and 1/sqrt(n) is folded into the scale:
 *                   scale32 = ((zmax - zmin) / 15) / c;  scale = half(scale32);
 *                   d = c * float(scale);  rd = 1 / d;
 *                   zero = rint(-zmin * rd);  q = clamp(rint(z * rd) + zero, 0, 15)
 *                 with c = sqrtf(n) (c = 1 without the transform).
 * in_dtype: 0 = binary16, 1 = bfloat16.  ld = row stride of x in elements.
 * q_out [M, n/2] bytes, scale_out/zero_out [M] binary16. */
void flh_oracle_quant_token_asym(const uint16_t *x, int in_dtype, long M, long n, long ld,
                                 int hadamard, int kfac, const int8_t *signs, float clip,
                                 int exact_norm, uint8_t *q_out, uint16_t *scale_out,
                                 uint16_t *zero_out) {
    const float c = hadamard ? sqrtf((float)n) : 1.0f;
#pragma omp parallel
    {
        float *z = (float *)malloc((size_t)n * 4);
        float *tmp = (float *)malloc((size_t)n * 4);
#pragma omp for schedule(static)
        for (long r = 0; r < M; ++r) {
            for (long i = 0; i < n; ++i)
                z[i] = in_dtype ? bf2f(x[r * ld + i]) : h2f(x[r * ld + i]);
            if (hadamard) had_full_row_f32(z, tmp, n, kfac, signs);
            if (exact_norm && hadamard) for (long i = 0; i < n; ++i) z[i] = z[i] / c;
            float zmin = 0.0f, zmax = 0.0f;
            for (long i = 0; i < n; ++i) { if (z[i] < zmin) zmin = z[i]; if (z[i] > zmax) zmax = z[i]; }
            zmin = zmin * clip; zmax = zmax * clip;
            if (zmin == 0.0f && zmax == 0.0f) { zmin = -1.0f; zmax = 1.0f; }
            float scale32 = (zmax - zmin) / 15.0f;
            if (!exact_norm) scale32 = scale32 / c;
            uint16_t sh = f2h(scale32);
            if ((sh & 0x7fffu) == 0) sh = 0x0001u;          /* keep the stored scale non-zero */
            float s = h2f(sh);
            scale_out[r] = sh;
            if (exact_norm) {
                float zero = nearbyintf(-zmin / s);
                zero_out[r] = f2h(zero);
                for (long i = 0; i < n; i += 2) {
                    float a = nearbyintf(z[i] / s) + zero, b = nearbyintf(z[i + 1] / s) + zero;
                    int q0 = (int)(a < 0.f ? 0.f : (a > 15.f ? 15.f : a));
                    int q1 = (int)(b < 0.f ? 0.f : (b > 15.f ? 15.f : b));
                    q_out[r * (n / 2) + i / 2] = (uint8_t)(q0 | (q1 << 4));
                }
            } else {
                float d = c * s, rd = 1.0f / d;
                float zf = nearbyintf(-zmin * rd);
                int zero = (int)zf;
                zero_out[r] = f2h(zf);
                for (long i = 0; i < n; i += 2) {
                    float ta = nearbyintf(z[i] * rd), tb = nearbyintf(z[i + 1] * rd);
                    /* clamp in float first so that the int conversion cannot overflow */
                    ta = ta < -64.f ? -64.f : (ta > 64.f ? 64.f : ta);
                    tb = tb < -64.f ? -64.f : (tb > 64.f ? 64.f : tb);
                    int q0 = (int)ta + zero, q1 = (int)tb + zero;
                    q0 = q0 < 0 ? 0 : (q0 > 15 ? 15 : q0);
                    q1 = q1 < 0 ? 0 : (q1 > 15 ? 15 : q1);
                    q_out[r * (n / 2) + i / 2] = (uint8_t)(q0 | (q1 << 4));
                }
            }
        }
        free(z); free(tmp);
    }
}

/* ------------------------------------------------------------------------- */
static inline int nib_s(const uint8_t *row, long k) {        /* signed nibble */
    int v = (row[k >> 1] >> ((k & 1) * 4)) & 15;
    return v >= 8 ? v - 16 : v;
}
static inline int nib_u(const uint8_t *row, long k) { return (row[k >> 1] >> ((k & 1) * 4)) & 15; }

/* Per-(row, group) sums of the signed weight codes: rs[n][g] = sum_{k in g} qw[n][k].
 * Needed for the zero-point term of the asymmetric epilogue; no counterpart in
 * the reference CUDA path (its GEMM has no zero-point). group = K for one sum per row. */
void flh_oracle_weight_rowsum(const uint8_t *B, long N, long K, long group, int32_t *rs) {
    long G = K / group;
#pragma omp parallel for schedule(static)
    for (long n = 0; n < N; ++n)
        for (long g = 0; g < G; ++g) {
            int32_t s = 0;
            for (long k = g * group; k < (g + 1) * group; ++k) s += nib_s(B + n * (K / 2), k);
            rs[n * G + g] = s;
        }
}

/* Exact integer group partial sums: C[m][n][g] = sum_{k in g} qa[m][k] * qw[n][k].
 * The int32 accumulators of flh_gemm_i4_dequant_o16_kernel,
 * flh/kernels/gemm_and_dequant_i4.cu:199-240 (mma.sync s4.s4 -> s32). */
void flh_oracle_gemm_i4_int32(const uint8_t *A, const uint8_t *B, long M, long N, long K,
                              long group, int a_unsigned, int32_t *C) {
    long G = K / group;
#pragma omp parallel for schedule(static)
    for (long n = 0; n < N; ++n) {
        int8_t *w = (int8_t *)malloc((size_t)K);
        for (long k = 0; k < K; ++k) w[k] = (int8_t)nib_s(B + n * (K / 2), k);
        for (long m = 0; m < M; ++m) {
            const uint8_t *a = A + m * (K / 2);
            for (long g = 0; g < G; ++g) {
                int32_t s = 0;
                for (long k = g * group; k < (g + 1) * group; ++k)
                    s += (a_unsigned ? nib_u(a, k) : nib_s(a, k)) * (int32_t)w[k];
                C[(m * N + n) * G + g] = s;
            }
        }
        free(w);
    }
}

/* int4 x int4 GEMM with fused dequantisation.
 * Restates flh_gemm_i4_dequant_o16_kernel, flh/kernels/gemm_and_dequant_i4.cu:315-469,
 * whose epilogue is dequant_accumulate :287-313 — per 128-K group, ascending,
 *     acc += float(int32 group sum) * (sa[m][g] * sb[n][g])      (binary32)
 * (the reference is built with --use_fast_math, which contracts this to one
 * fused multiply-add; it is written as fmaf here and in the B200 kernels) — and a
 * round-to-nearest binary16 store (:179-197).
 *
 * Extended the way the activation modes need (no counterpart in the reference
 * CUDA path, arithmetic from LinearFLH.forward_torch, flh/nn/linear.py:134-152,
 * (q - zero) * scale on both operands):
 *   a_group / b_group = scale granularity along K of the activations / weights
 *                       (128 or K for a; 32, 64, 128 or K for b);
 *   the accumulation group is min(a_group, b_group);
 *   a_zero != NULL: activation codes are unsigned 0..15 with an integer
 *                   zero-point per scale group of a, and
 *                   I_g = C_g - zero[m][ga] * rowsum_w[n][g] replaces C_g;
 *   acc = fmaf(float(I_g), sa[m][ga] * sb[n][gb], acc), g ascending, from +0;
 *   bias != NULL: acc + float(bias[n]) before the final rounding;
 *   out_dtype 0 = binary16, 1 = bfloat16.
 * A [M, K/2], B [N, K/2] packed; a_scale [M, K/a_group]; a_zero same shape;
 * b_scale [N, K/b_group]; D [M, N]. */
void flh_oracle_gemm_i4_dequant(const uint8_t *A, const uint8_t *B, const uint16_t *a_scale,
                                const uint16_t *a_zero, const uint16_t *b_scale,
                                const uint16_t *bias, uint16_t *D, long M, long N, long K,
                                long a_group, long b_group, int out_dtype) {
    long group = a_group < b_group ? a_group : b_group;
    long G = K / group, GA = K / a_group, GB = K / b_group;
#pragma omp parallel for schedule(static)
    for (long n = 0; n < N; ++n) {
        int8_t *w = (int8_t *)malloc((size_t)K);
        int32_t *rs = (int32_t *)malloc((size_t)G * 4);
        for (long k = 0; k < K; ++k) w[k] = (int8_t)nib_s(B + n * (K / 2), k);
        for (long g = 0; g < G; ++g) {
            int32_t s = 0;
            for (long k = g * group; k < (g + 1) * group; ++k) s += w[k];
            rs[g] = s;
        }
        for (long m = 0; m < M; ++m) {
            const uint8_t *a = A + m * (K / 2);
            float acc = 0.0f;
            for (long g = 0; g < G; ++g) {
                long ga = g * group / a_group, gb = g * group / b_group;
                int32_t c = 0;
                if (a_zero) {
                    for (long k = g * group; k < (g + 1) * group; ++k) c += nib_u(a, k) * (int32_t)w[k];
                    c -= (int32_t)h2f(a_zero[m * GA + ga]) * rs[g];
                } else {
                    for (long k = g * group; k < (g + 1) * group; ++k) c += nib_s(a, k) * (int32_t)w[k];
                }
                float p = h2f(a_scale[m * GA + ga]) * h2f(b_scale[n * GB + gb]);   /* exact */
                acc = fmaf((float)c, p, acc);
            }
            if (bias) acc = acc + h2f(bias[n]);
            D[m * N + n] = out_dtype ? f2bf(acc) : f2h(acc);
        }
        free(w); free(rs);
    }
}

/* Conversions exported for the Python side of the tests. */
/* RMS-normalisation (weight 1) into the input's 16-bit type, with the summation order the fused B200 kernel
 * defines (include/flh_b200.h, flh_b200_rmsnorm_quant_token_asym_i4): lanes of 128 consecutive values added in order
 * with fma, 32 lanes joined by an xor tree (16, 8, 4, 2, 1), the warps of a row added last; then
 * c = 1 / sqrt(s / K + eps) with correctly rounded sqrt and division, y = round16(x * c).
 * Restates flh/nn/normalization.py (x * rsqrt(mean(x^2) + eps), weight folded to 1) up to that order. */
void flh_oracle_rmsnorm16(const uint16_t *x, int bf16, long M, long K, long ld, float eps, uint16_t *y) {
    const long lanes = K / 128, warps = lanes / 32;
    for (long r = 0; r < M; ++r) {
        const uint16_t *row = x + r * ld;
        float total = 0.0f;
        for (long w = 0; w < warps; ++w) {
            float s[32], t[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.0f;
                const uint16_t *v = row + (w * 32 + l) * 128;
                for (int i = 0; i < 128; ++i) { const float f = bf16 ? bf2f(v[i]) : h2f(v[i]); acc = fmaf(f, f, acc); }
                s[l] = acc;
            }
            for (int sft = 16; sft > 0; sft >>= 1) {
                for (int l = 0; l < 32; ++l) t[l] = s[l] + s[l ^ sft];
                memcpy(s, t, sizeof(s));
            }
            total = w == 0 ? s[0] : total + s[0];
        }
        const float c = 1.0f / sqrtf(total * (1.0f / (float)K) + eps);
        for (long i = 0; i < K; ++i) {
            const float f = bf16 ? bf2f(row[i]) : h2f(row[i]);
            y[r * K + i] = bf16 ? f2bf(f * c) : f2h(f * c);
        }
    }
}

void flh_oracle_f32_to_f16(const float *in, uint16_t *out, long n) { for (long i = 0; i < n; ++i) out[i] = f2h(in[i]); }
void flh_oracle_f16_to_f32(const uint16_t *in, float *out, long n) { for (long i = 0; i < n; ++i) out[i] = h2f(in[i]); }

/* ---- SiLU(gate) * up of the MLP (flh/quantized_model/modeling_llama.py:522-526), as the fused kernels define it:
 *   e = exp32(-g);  s = round16(g / (1 + e));  out = round16(s * u), every step one IEEE binary32 operation.
 *   exp32(t), t clamped to [-87, 88]: n = rint(t log2 e); r = t - n ln2 in two fma; y = 1 + r + r^2 P(r) (Cephes expf's
 *   degree-5 polynomial, Horner with fma); result = y * 2^n.                                                            */
static inline float exp32(float t) {
    t = fminf(fmaxf(t, -87.0f), 88.0f);
    const float n = nearbyintf(t * 1.44269504088896341f);
    float r = fmaf(n, -0.693359375f, t);
    r = fmaf(n, 2.12194440e-4f, r);
    const float z = r * r;
    float y = 1.9875691500e-4f;
    y = fmaf(y, r, 1.3981999507e-3f);
    y = fmaf(y, r, 8.3334519073e-3f);
    y = fmaf(y, r, 4.1665795894e-2f);
    y = fmaf(y, r, 1.6666665459e-1f);
    y = fmaf(y, r, 5.0000001201e-1f);
    y = fmaf(y, z, r);
    y = y + 1.0f;
    uint32_t sb = (uint32_t)((int)n + 127) << 23;
    float sc; memcpy(&sc, &sb, 4);
    return y * sc;
}

/* gu [M][ld] 16-bit values: gate = columns [0, F), up = columns [F, 2F); out [M][F] */
void flh_oracle_silu_mul16(const uint16_t *gu, int bf16, long M, long F, long ld, uint16_t *out) {
    for (long m = 0; m < M; ++m)
        for (long f = 0; f < F; ++f) {
            const uint16_t gb = gu[m * ld + f], ub = gu[m * ld + F + f];
            const float g = bf16 ? bf2f(gb) : h2f(gb), u = bf16 ? bf2f(ub) : h2f(ub);
            const float s = g / (1.0f + exp32(-g));
            if (bf16) out[m * F + f] = f2bf(bf2f(f2bf(s)) * u);
            else out[m * F + f] = f2h(h2f(f2h(s)) * u);
        }
}
