/*
 * flh_b200 — C ABI of the B200 (sm_100a) implementation of FLH's W4A4 hot path:
 * online Hadamard + int4 activation quantiser + int4 x int4 GEMM with fused
 * dequantisation.
 *
 * Conventions (all entry points unless stated otherwise)
 *   - plain pointers and sizes; every data pointer is a DEVICE pointer on the
 *     current device; inputs are borrowed, outputs are caller-allocated;
 *   - no entry point allocates, frees or synchronises; work is enqueued on
 *     `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream);
 *   - return value: 0 = ok, > 0 = rejected argument (FLH_B200_EINVAL...),
 *     < 0 = minus the cudaError_t of a failed runtime call or launch;
 *     flh_b200_last_error() returns a per-thread message for the last non-zero
 *     return;
 *   - "f16" is IEEE binary16, "bf16" bfloat16, both passed as void*;
 *   - packed int4: byte j of a row holds element 2j in its low nibble and
 *     element 2j+1 in its high nibble (pack_i4, flh/functional/quantization.py:42-49;
 *     had_and_quant_kernel, flh/kernels/had_and_quant.cu:141-148).
 *
 * File:line citations name the FLH interface each entry point replaces; paths
 * are relative to the FLH repository root.
 */
#ifndef FLH_B200_H
#define FLH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLH_B200_OK 0
#define FLH_B200_EINVAL 1      /* bad size, mode or null pointer            */
#define FLH_B200_EALIGN 2      /* pointer or stride not aligned as required */
#define FLH_B200_EUNSUPPORTED 3 /* valid request this build cannot serve    */
#define FLH_B200_EDEVICE 4     /* kernel reported a device-side error word  */

#define FLH_B200_F16 0
#define FLH_B200_BF16 1

/* GEMM algorithm selector */
#define FLH_B200_GEMM_AUTO 0
#define FLH_B200_GEMM_TCGEN05 1 /* TMA + int4->int8 expand in smem + tcgen05.mma kind::i8, TMEM accumulators */
#define FLH_B200_GEMM_MMA_SYNC 2 /* legacy mma.sync m16n8k32 s8 path (bring-up cross-check, any M)           */
#define FLH_B200_GEMM_STREAM 3  /* weight-streaming small-M path (M <= 64)                                    */
#define FLH_B200_GEMM_TCGEN05_DIRECT 5 /* tcgen05 path whose converter warps load the packed operands from L2
                                         straight into registers (no TMA staging): less shared-memory traffic */
#define FLH_B200_GEMM_STREAM_SPLITK 4 /* the same with K cut across CTAs; needs workspace (see below)           */
#define FLH_B200_GEMM_TCGEN05_I8 6 /* large M without group scales: both operands expanded to int8 in the workspace
                                     first, then TMA + tcgen05.mma on int8 tiles (no conversion inside the GEMM)  */
#define FLH_B200_GEMM_TCGEN05_I8_PAIR 7 /* the same on two-CTA clusters (tcgen05 cta_group::2, 256 x 256 tiles);
                                          N % 256 == 0                                                         */
#define FLH_B200_GEMM_DECODE_TC 8 /* M <= 64 on the tensor cores with the operands swapped (weights on the MMA's M side),
                                    K-ranges balanced across CTAs; needs zero-initialised workspace like split-K */

int flh_b200_version(void);
const char *flh_b200_last_error(void);

/* 0 when the current device is an sm_100 part this library was built for. */
int flh_b200_device_check(void);

/* ---- activation quantisers ------------------------------------------------------------- */

/* Fused (optional) group Hadamard + symmetric int4 quantiser + packing.
 * x [rows, gs] f16 contiguous, gs in {32, 64, 128}; q [rows, gs/2]; scales [rows] f16 (raw,
 * un-normalised: the caller folds 1/sqrt(gs), as ActQuantizer.forward does,
 * flh/nn/quantization.py:156-162).
 * Replaces had_and_quant_host (flh/kernels/had_and_quant.h:19-24, kernel
 * flh/kernels/had_and_quant.cu:61-155), quant_and_pack_host (flh/kernels/quant_and_pack.h:19-24)
 * and their _gs forms (flh/kernels/had_and_quant_gs.h, quant_and_pack_gs.h); bound as
 * hadamard_and_quantize_i4 / quant_and_pack_i4 (flh/cuda/flh_cuda_bindings.cpp:154-198). */
int flh_b200_quant_group_sym_i4(const void *x, long rows, int gs, int hadamard,
                                uint8_t *q, void *scales, void *stream);

/* In-place un-normalised f16 Walsh-Hadamard transform of rows of n in {32, 64, 128}.
 * Replaces had_trans_half_cuda / had_trans_64_half_cuda / had_trans_32_half_cuda
 * (flh/kernels/cuda_had_kernel.cu:296-354 and the 64/32 copies), bound as
 * hadamard_transform_half / _64_half / _32_half (flh/cuda/flh_cuda_bindings.cpp:115-152). */
int flh_b200_hadamard_f16_inplace(void *x, long rows, int n, void *stream);

/* (Optional full-width Hadamard +) per-token asymmetric int4 quantiser + packing.
 * x [M, K] f16 or bf16 with row stride ld (elements, multiple of 8; x 16-byte aligned).
 * hadamard = 0: quantise x itself.  hadamard = 1 or 2: quantise (hadK (x) H_p) x / sqrt(K) with
 * K = kfac * p, p a power of two >= 64; kfac = 1 for a power-of-two K, otherwise one of the
 * orders get_hadK knows (flh/functional/hadamard.py:39-89) with sign_bits = the factor table made
 * by flh_b200_pack_signs (copied to the device, 16-byte aligned); 1/sqrt(K) is folded into the scale.
 *   hadamard = 2: binary32 butterflies in the order of matmul_hadU (flh/functional/hadamard.py:92-113), the
 *     kfac x kfac factor summed k' ascending: bit-exact with the CPU oracle for every K.
 *   hadamard = 1 (default of the Python layer): for K = P * 64 with P <= 512 (4096, 8192, 11008, 14336, 16384, 28672, 32768
 *     and the tensor-parallel shards 7168 / 3584 ...) the part of the transform above the lowest six bits — a P x P matrix of
 *     +-1 — is applied first, to the raw 16-bit inputs, by tcgen05.mma (products exact, binary32 accumulation in the
 *     tensor core's order); the lowest six bits follow as binary32 butterflies.  Same values up to the order of the
 *     binary32 additions (the reference's own matmul has no fixed order either); measured against the oracle: at most
 *     0.1 % of all codes differ, by one step, scales within one f16 ulp.  Every M takes the same kernel, so a row's
 *     codes do not depend on the batch it arrives in.  Above P = 256 the row is read as the two halves of its top
 *     Sylvester bit and the +-1 matrix of order P / 2 is applied to both, added and subtracted in the accumulators.
 *     Other K: as hadamard = 2, except that factors of order >= 64 are summed by mma.sync.
 * Quantiser: ActQuantizer.find_params / asym_quant (fake_quant/quant_utils.py:94-128, 17-21)
 * with the scale rounded to f16 before use.  q [M, K/2] codes 0..15; scale, zero [M] f16.
 * clip = the quantiser's clip_ratio in (0, 1]. */
int flh_b200_quant_token_asym_i4(const void *x, int in_dtype, long M, long K, long ld,
                                 int hadamard, int kfac, const uint32_t *sign_bits, float clip,
                                 uint8_t *q, void *scale, void *zero, void *stream);

/* Diagnostic: the name of the kernel flh_b200_quant_token_asym_i4 launches for this shape (16-byte aligned pointers
 * assumed).  A static string.  No counterpart in FLH. */
const char *flh_b200_quant_token_kernel(long M, long K, int hadamard, int kfac);

/* RMS-norm (weight 1, as FLH leaves it after folding the norm weight into the next linear) fused in front of the
 * per-token asymmetric quantiser, K = 4096 or 8192: the decoder's "norm -> quantise" pair as one pass over the row.
 * Equal to normalising into the input's 16-bit type and then calling flh_b200_quant_token_asym_i4(hadamard) on
 * the result, with the normalisation defined as: s = sum x^2 in binary32 (each of the 32 K / 4096 lanes of a row
 * adds its 128 consecutive values in order with fma; lanes are joined by xor-shuffles 16, 8, 4, 2, 1, then the
 * two halves of a K = 8192 row), c = 1 / sqrt(s / K + eps) with correctly rounded sqrt and reciprocal,
 * y = round_to_input_type(x * c).  q must be 16-byte aligned.  FLH_B200_EUNSUPPORTED for other K (normalise
 * separately).  The reference has no fused form: `flh/nn/normalization.py` + `flh/nn/quantization.py:143-291`
 * run back to back in `flh/quantized_model/modeling_llama.py:389-393, 522-526`. */
int flh_b200_rmsnorm_quant_token_asym_i4(const void *x, int in_dtype, long M, long K, long ld, float eps,
                                         int hadamard, float clip, uint8_t *q, void *scale, void *zero,
                                         void *stream);

/* The same fusion for the group-128 symmetric mode (the flh._CUDA contract): x f16 [M, 4096] contiguous ->
 * q [M * 32, 64], scales [M * 32], equal to normalising into f16 (same definition as above) and then calling
 * flh_b200_quant_group_sym_i4(gs = 128, hadamard).  K = 4096 only (a warp owns a whole row). */
int flh_b200_rmsnorm_quant_group_sym_i4(const void *x, long M, long K, float eps, int hadamard, uint8_t *q,
                                        void *scales, void *stream);

/* ---- the decoder wiring either side of the quantised linears (flh/quantized_model/modeling_llama.py:389-470, 522-526) ---- */

/* SiLU(gate) * up of the MLP.  gu [M, 2F] f16 or bf16 with row stride ld (elements): gate = columns [0, F), up = columns
 * [F, 2F) — the output of the merged gate/up GEMM; out [M, F] contiguous, same type.  F % 8 == 0, 16-byte aligned pointers.
 * Defined bit for bit (so that the CPU restatement agrees): e = exp32(-g), s = round16(g / (1 + e)), out = round16(s * u),
 * every step one IEEE binary32 operation; exp32 is a fixed range reduction + degree-5 polynomial (csrc/act_common.cuh),
 * within 1 ulp of expf, so the result equals torch's silu(gate) * up except where torch's own expf differs in the last bit.
 * The reference runs act_fn and the product as separate PyTorch kernels (modeling_llama.py:524). */
int flh_b200_silu_mul(const void *gu, int in_dtype, long M, long F, long ld, void *out, void *stream);

/* The same followed by the full-width transform and the per-token asymmetric quantiser of flh_b200_quant_token_asym_i4
 * (hadamard = 1), as ONE kernel: the MLP's "act_fn(gate) * up -> quantizer2" (modeling_llama.py:524-525) with the online
 * transform of the per-token mode.  The product never reaches global memory: the epilogue warps of the tensor-core
 * quantiser make the rows in shared memory in place of its TMA loads.  Result: equal to flh_b200_silu_mul followed by
 * flh_b200_quant_token_asym_i4(hadamard = 1) on its output.  FLH_B200_EUNSUPPORTED when the width is not one the
 * tensor-core kernel takes (F = P * 64, P <= 256) or hadamard != 1: run the two steps separately then. */
int flh_b200_silu_mul_quant_token_asym_i4(const void *gu, int in_dtype, long M, long F, long ld, int hadamard, int kfac,
                                          const uint32_t *sign_bits, float clip, uint8_t *q, void *scale, void *zero,
                                          void *stream);

/* Rotary embedding + KV-cache write in one pass over the merged QKV GEMM output (f16).
 * qkv [B * S, (nh + 2 nkv) * D]: per token nh query heads, nkv key heads, nkv value heads of D values; cos, sin [S, D / 2]
 * binary32 for the S positions of this step; half-split convention (element i pairs with i + D / 2):
 *   out[i] = x[i] cos[i] - x[i + D/2] sin[i],  out[i + D/2] = x[i + D/2] cos[i] + x[i] sin[i]   (each product and sum rounded
 *   to binary32 on its own, the result to f16 — the bits separate tensor operations give).
 * q goes to q_out [B, nh, S, D]; rotated k and plain v go into k_cache / v_cache [B, nkv, T, D] at positions cur .. cur + S - 1.
 * D % 8 == 0, cur + S <= T.  The reference does this as split, rotary, transpose and cache update (modeling_llama.py:396-440). */
int flh_b200_rope_kv_f16(const void *qkv, const float *cos, const float *sin, void *q_out, void *k_cache, void *v_cache,
                         int B, int S, int nh, int nkv, int D, int T, int cur, void *stream);

/* HOST helpers: build the factor table of a kfac x kfac matrix of +1/-1 (int8, row-major, host
 * memory).  Layout: bit rows out[k * words + w], bit b = 1 when signs[k][32 w + b] < 0,
 * words = (kfac + 31) / 32; then, at the next 16-byte boundary, the same matrix as bfloat16 +-1.0
 * padded with zeros to kp x kp, kp = kfac rounded up to a multiple of 16.
 * out: flh_b200_sign_table_bytes(kfac) bytes of host memory. */
size_t flh_b200_sign_table_bytes(int kfac);
int flh_b200_pack_signs(const int8_t *signs, int kfac, uint32_t *out);

/* ---- weights ---------------------------------------------------------------------------- */

/* rowsum[n, g] = sum of the signed int4 codes of weight row n over K-group g (int32,
 * [N, K/group]); the zero-point term of the asymmetric epilogue needs it.  Offline, once per
 * weight.  No counterpart in FLH (its GEMM has no zero-point, flh/nn/linear.py:125-133). */
int flh_b200_weight_rowsum(const uint8_t *B, long N, long K, long group, int32_t *rowsum,
                           void *stream);

/* ---- GEMM ------------------------------------------------------------------------------- */

/* D[M, N] = dequantising int4 x int4 GEMM.
 *   A [M, K/2], B [N, K/2] packed int4 (B signed; A signed when a_zero == NULL, else unsigned);
 *   a_scale [M, K/a_group] f16, a_group in {g, K};  a_zero NULL or f16 like a_scale (integer
 *   values 0..15);  b_scale [N, K/b_group] f16, b_group in {g, K};  g in {32, 64, 128} is the K-group the
 *   integer sums are cut into (groups of 32 and 64 — the reference's *_gs entry points — are served by the
 *   mma.sync tile kernel, algo AUTO or MMA_SYNC; every group is scaled with its own scales, where the reference
 *   kernel flh/kernels/gemm_and_dequant_i4_gs.cu:408 takes the first scale of each 128-K block for the whole block);
 *   b_rowsum [N, K/min(a_group, b_group)] int32, required when a_zero != NULL;
 *   bias NULL or [N] f16;  D f16 or bf16 (out_dtype).
 *   With g running over K-groups of min(a_group, b_group) in ascending order:
 *     I_g = sum_{k in g} qa[m,k] qw[n,k]  -  zero[m, ga] * rowsum[n, g]
 *     acc = fmaf((float) I_g, sa[m, ga] * sb[n, gb], acc)        (binary32, acc starts at +0)
 *     D[m, n] = round(acc + bias[n])
 *   which with a_zero = NULL, a_group = b_group = 128, f16 output is the arithmetic of
 *   flh_gemm_i4_dequant_o16_kernel (flh/kernels/gemm_and_dequant_i4.cu:287-313, 315-469).
 *   N % 128 == 0 and K % 128 == 0 are required (as the reference kernel assumes), K <= 65536.
 *   algo: FLH_B200_GEMM_*.  workspace: device scratch of at least
 *   flh_b200_gemm_workspace_bytes(...) bytes, 256-byte aligned (may be NULL when that is 0).  The two decode
 *   kernels that share output tiles between CTAs use it: the split-K streaming kernel (decode shapes whose N
 *   alone cannot fill the GPU) and the tensor-core decode kernel (DECODE_TC; AUTO picks it for M <= 64 when
 *   the packed weights reach 64 MiB, 32 MiB above 16 tokens, 12 MiB above 32).  Its first 4 KB are arrival
 *   counters that must be ZERO before the first launch and are left zero by every launch; launches that
 *   share a workspace must not overlap on the GPU.  With AUTO and no (or too small a) workspace the plain
 *   streaming kernel (or, for large batches, the converting tcgen05 kernel) runs instead.  Both kernels add
 *   the binary32 chains of the CTAs that share a tile in K order, so with group scales their outputs can
 *   differ from the single chain in the last bit (<= 1e-3 relative, the same bits on every run); without
 *   group scales the partial sums are int32 and the result is identical.  STREAM and TCGEN05 never split a chain.
 *   The int8-operand kernels (TCGEN05_I8, TCGEN05_I8_PAIR; a_group = b_group = K only) write the expanded
 *   operands, (M + N) * K bytes, into the workspace; it needs no initial contents, results are bit-identical
 *   to the other kernels, and launches that share a workspace must not overlap on the GPU.
 * Replaces flhDenseLayerGEMM_i4_o16 (flh/kernels/gemm_and_dequant_i4.cu:471-508) and
 * flhDenseLayerGEMM_i4_o16_gs (flh/kernels/gemm_and_dequant_i4_gs.h); bound as
 * gemm_i4_dequant_o16(_gs) (flh/cuda/flh_cuda_bindings.cpp:75-113, 253-299). */
int flh_b200_gemm_i4_dequant(const uint8_t *A, const uint8_t *B, const void *a_scale,
                             const void *a_zero, const void *b_scale, const int32_t *b_rowsum,
                             const void *bias, void *D, long M, long N, long K, long a_group,
                             long b_group, int out_dtype, int algo, void *workspace,
                             size_t workspace_bytes, void *stream);

size_t flh_b200_gemm_workspace_bytes(long M, long N, long K, long a_group, long b_group, int algo);

/* Weights expanded once, ahead of time, for large-batch (prefill) GEMMs with per-token / per-channel scales.
 * flh_b200_expand_i4 turns packed int4 [rows, K/2] into int8 [rows, K] holding 16 * q (for unsigned codes:
 * 16 * code as uint8), in the element order the int8-operand kernels use (per 32 elements: the 16 even ones,
 * then the 16 odd ones); out is 128-byte aligned.  flh_b200_gemm_i8w_dequant is flh_b200_gemm_i4_dequant with
 * a_group = b_group = K whose weight operand is that expanded copy: only the activations are expanded per call,
 * into `workspace` (>= M * K bytes, 256-byte aligned, no initial contents; launches sharing it must not overlap).
 * Results are bit-identical to flh_b200_gemm_i4_dequant.  Neither has a counterpart in the reference, which
 * keeps int4 weights only: an engine with HBM to spare keeps both copies, the packed one for decode (where the
 * weight bytes are the cost) and this one for prefill (where the tensor cores are). */
int flh_b200_expand_i4(const uint8_t *packed, long rows, long K, uint8_t *out, void *stream);
int flh_b200_gemm_i8w_dequant(const uint8_t *A, const uint8_t *B8, const void *a_scale, const void *a_zero,
                              const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                              long M, long N, long K, int out_dtype, void *workspace,
                              size_t workspace_bytes, void *stream);

/* One column block of GPTQ's quantise-and-compensate sweep: the inner loop of FLHGPTQ.fasterquant
 * (flh/nn/gptq.py:198-232) for `count` <= 128 consecutive columns of all `rows` weight rows, in one launch.
 *   W     f32, rows x ldw   the block's columns as they stand before the sweep (read only)
 *   Hinv  f32, count x ldh  the block of the upper Cholesky factor of the inverse Hessian (its diagonal block)
 *   scale / zero  f32, rows x lds; column c of the block uses entry group_of_col[c] (zero may be NULL when sym)
 *   Q     f32, rows x ldq   the dequantised columns;  Err  f32, rows x count  the errors (w - q) / Hinv[c][c]
 * For each column c in order:  q = scale * clamp(rint(x / scale), -(maxq + 1), maxq)  (sym; x = w clamped to
 * +-scale * maxq * clip_ratio when clip_ratio < 1),  or  scale * (clamp(rint(x / scale + zero), 0, maxq) - zero),
 * err = (w - q) / Hinv[c][c],  and  w_j = w_j - err * Hinv[c][j]  for the columns j > c of the block; binary32
 * throughout, each product and difference rounded as the reference's torch code rounds them.  The caller applies
 * W[:, after the block] -= Err @ Hinv[block rows, after the block]  (a plain GEMM) before the next block. */
int flh_b200_gptq_block(const float *W, long ldw, const float *Hinv, long ldh, const float *scale, const float *zero,
                        long lds, const int *group_of_col, long rows, int count, int maxq, int sym, float clip_ratio,
                        float *Q, long ldq, float *Err, void *stream);

/* Which algorithm FLH_B200_GEMM_AUTO resolves to for this shape (one of FLH_B200_GEMM_*). */
int flh_b200_gemm_pick_algo(long M, long N, long K, long a_group, long b_group);

/* Decode GEMM (M <= 64) for callers that must not allocate.  Same arguments and results as
 * flh_b200_gemm_i4_dequant with algo = FLH_B200_GEMM_STREAM_SPLITK, but the split-K scratch is not a
 * caller buffer: it is a 4 KiB + 2 MiB array built into the library's device image, so a serving loop
 * that runs inside a fixed memory budget, a plugin host that owns every cudaMalloc, or code running
 * where allocation is forbidden (between two graph launches, inside a real-time section) can still use
 * the split-K kernel.  This entry point calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - Limit: shapes whose split-K scratch exceeds the built-in array (for example M = 32, N = 9216) are
 *     rejected with FLH_B200_EINVAL and a message naming the size; use the workspace form for those.
 *     Shapes that need no split (many output columns) run the plain streaming kernel, scratch untouched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call outside any stream capture.  Every GPU that loads the library carries the array
 *     until the process exits.  The looked-up address is kept in a plain per-device table: two host threads
 *     making the first call on one device at the same moment both look it up and store the same value.
 *   - All calls on a device share the one array and it keeps the previous call's contents; each call
 *     re-zeroes the counters on `stream` before the kernel.  Two calls whose kernels could overlap on the
 *     GPU (different streams, no ordering between them) race on it: order them or use the workspace form.
 * No counterpart in FLH (its GEMM takes no scratch). */
int flh_b200_gemm_i4_dequant_decode_noalloc(const uint8_t *A, const uint8_t *B, const void *a_scale,
                                            const void *a_zero, const void *b_scale, const int32_t *b_rowsum,
                                            const void *bias, void *D, long M, long N, long K, long a_group,
                                            long b_group, int out_dtype, void *stream);

/* Reads (and clears) the device status words of the tcgen05 GEMM: out[0] = 0, or the code of the
 * first bounded wait that ran out (1 TMA producer, 2/3 MMA issuer, 4/5 converters, 6/7 epilogue),
 * out[1] = the CTA that reported it.  SYNCHRONISES the device; for tests and post-mortems only.
 * out: 4 ints in HOST memory.  No counterpart in FLH. */
int flh_b200_gemm_status(int *out);

/* Diagnostic: nanoseconds the roles of the tcgen05 GEMM spent waiting on each other since the last call
 * (summed over CTAs; out[1] TMA producer on a free packed slot, out[2] MMA thread on a free accumulator,
 * out[3] MMA thread on converted operands, out[4] converters on TMA data, out[5] converters on a free
 * int8 slot, out[6] epilogue on a finished accumulator).  Reads and clears; SYNCHRONISES the device.
 * out: 8 x unsigned long long in HOST memory.  No counterpart in FLH. */
int flh_b200_gemm_wait_profile(unsigned long long *out);

/* Diagnostic of the tensor-core token quantiser (quant_token_tc_kernel), same conventions: nanoseconds summed over CTAs
 * since the last call — out[0] CTA lifetime, out[1] TMA thread on a free shared-memory stage, out[2] MMA thread on TMA
 * data, out[3] MMA thread on a free accumulator slot, out[4] the 16 epilogue warps on a finished accumulator (summed
 * over warps), out[5] set-up.  Reads and clears; SYNCHRONISES the device.  out: 8 x unsigned long long in HOST memory. */
int flh_b200_quant_token_wait_profile(unsigned long long *out);

/* One-shot all-reduce (sum) of small f16 / bf16 messages between the GPUs of one node: the partial outputs of a
 * row-parallel linear in tensor-parallel decode, where an all-reduce costs latency, not bandwidth.  No counterpart in FLH
 * (it has no multi-GPU code).  One process per GPU (or one process for several), at most 8 ranks.
 *   flh_b200_ar_create    allocates this rank's buffer on the current device: a control block, arrival flags and two
 *                         sets of `world` receive slots of max_bytes each (max_bytes a multiple of 16, <= 64 MiB).
 *   flh_b200_ar_export    writes the 64-byte CUDA IPC handle of that buffer; send it to the other processes.
 *   flh_b200_ar_import    maps rank `peer`'s buffer from its IPC handle (another process);
 *   flh_b200_ar_attach    the same for a rank that lives in this process (enables peer access if it is on another device).
 *   flh_b200_allreduce    out = sum over ranks of x, n elements (a multiple of 8, n * 2 <= max_bytes), x and out 16-byte
 *                         aligned, out may be x.  One kernel launch on `stream`, no other CUDA call: every rank pushes
 *                         its message into every peer's slot with plain stores, raises a flag there, waits for the
 *                         peers' flags and sums the slots in rank order in binary32 — all ranks get the same bits.
 *                         Every rank must make the same sequence of calls (same n).  May be recorded into a CUDA graph.
 *                         A wait that lasts 2 s ends with the status word set; the launch still completes.
 *   flh_b200_allreduce_ranks  all `world` ranks in ONE cooperative launch, for ranks whose buffers live on one device
 *                         (tests on a single GPU: launches that wait on one another must not share a GPU).
 *   flh_b200_ar_status    out4 (HOST) = {0 or 1 = a wait ran out, the peer waited for, the CTA, the call number}; synchronises.
 *   flh_b200_ar_destroy   unmaps the peers and frees the buffer (after all ranks are done with it). */
typedef struct flh_b200_ar flh_b200_ar;
int flh_b200_ar_create(int world, int rank, size_t max_bytes, flh_b200_ar **out);
int flh_b200_ar_export(flh_b200_ar *h, void *ipc64);
int flh_b200_ar_import(flh_b200_ar *h, int peer, const void *ipc64);
int flh_b200_ar_attach(flh_b200_ar *h, int peer, flh_b200_ar *other);
int flh_b200_allreduce(flh_b200_ar *h, const void *x, void *out, long n, int dtype, void *stream);
int flh_b200_allreduce_ranks(flh_b200_ar *const *hs, int world, const void *const *xs, void *const *outs, long n,
                             int dtype, void *stream);
/* The same all-reduce FUSED with what follows a row-parallel linear in the decoder (o_proj / down_proj -> residual add ->
 * RMS-norm -> the per-token asymmetric int4 quantiser in front of the next linear; modeling_llama.py decoder layer), one launch,
 * one CTA per token row (M <= 128, K = 4096 or 8192, M * K * 2 <= max_bytes):
 *   residual <- round16(residual + round16(sum over ranks of y))          y, residual: [M, K] f16 / bf16, contiguous
 *   q, scale, zero <- flh_b200_rmsnorm_quant_token_asym_i4(residual, eps, hadamard = 0, clip)      (norm weight 1)
 * Bit for bit what flh_b200_allreduce, an f16 add and flh_b200_rmsnorm_quant_token_asym_i4 give as three launches.
 * _ranks: all ranks in one cooperative launch on one device (M * world <= 148), for tests on a single GPU. */
int flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4(flh_b200_ar *h, const void *y, void *residual, long M, long K, int dtype,
                                                       float eps, float clip, uint8_t *q, void *scale, void *zero, void *stream);
int flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4_ranks(flh_b200_ar *const *hs, int world, const void *const *ys,
                                                             void *const *residuals, long M, long K, int dtype, float eps,
                                                             float clip, uint8_t *const *qs, void *const *scales,
                                                             void *const *zeros, void *stream);
int flh_b200_ar_status(flh_b200_ar *h, int *out4);
int flh_b200_ar_destroy(flh_b200_ar *h);

/* The reference's one true C symbol, same signature and meaning
 * (flh/kernels/gemm_and_dequant_i4.cu:471-480): group-128 symmetric scales, f16 output,
 * legacy default stream, no status (errors are kept for flh_b200_last_error). */
void flhDenseLayerGEMM_i4_o16(const uint8_t *A, const uint8_t *B, const void *A_scale,
                              const void *B_scale, void *D, size_t M, size_t N, size_t K);

#ifdef __cplusplus
}
#endif
#endif /* FLH_B200_H */
