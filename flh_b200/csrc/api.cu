// C ABI of libflh_b200.so: argument validation, error strings, algorithm choice.
// Every entry point only enqueues work on the caller's stream.
#include "common.cuh"
#include <string.h>

namespace flh {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_status(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return 0;
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return -(int)e;
}

// kernels (other translation units)
int launch_quant_group_sym(const void *, long, int, int, uint8_t *, void *, cudaStream_t);
int launch_fht_inplace(void *, long, int, cudaStream_t);
int launch_quant_token_asym(const void *, int, long, long, long, int, int, const uint32_t *, float,
                            uint8_t *, void *, void *, cudaStream_t);
int launch_quant_token_warp(const void *, int, long, long, long, int, float, float, uint8_t *, void *, void *, cudaStream_t);
int launch_rmsnorm_quant_group(const void *, long, int, float, uint8_t *, void *, cudaStream_t);
int launch_weight_rowsum(const uint8_t *, long, long, long, int32_t *, cudaStream_t);
int launch_gemm_mma_tile(const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                         const int32_t *, const void *, void *, long, long, long, long, long, int,
                         cudaStream_t);
int launch_gemm_mma_tile_gs(const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                            const int32_t *, const void *, void *, long, long, long, long, long, int, int,
                            cudaStream_t);
int launch_gemm_stream(const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                       const int32_t *, const void *, void *, long, long, long, long, long, int,
                       int, void *, cudaStream_t);
int launch_gemm_stream_static(const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                              const int32_t *, const void *, void *, long, long, long, long, long, int, cudaStream_t);
int stream_splits(long M, long N, long K);
size_t stream_scratch_bytes(long M, long N, int splits);
int launch_gemm_tcgen05(const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                        const int32_t *, const void *, void *, long, long, long, long, long, int, int,
                        cudaStream_t);

size_t gemm_i8_workspace_bytes(long M, long N, long K);
int launch_gemm_i8(const uint8_t *, const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                   const int32_t *, const void *, void *, long, long, long, int, int, void *, cudaStream_t);
int launch_expand_i4(const uint8_t *, long, long, uint8_t *, cudaStream_t);
int gemm_i8_status(int *);
int quant_token_factor_status(int *);
int quant_token_factor_status_clear();
const char *quant_token_kernel_name(long, long, int, int);
int launch_silu_mul(const void *, int, long, long, long, void *, cudaStream_t);
int launch_silu_mul_quant_token_tc(const void *, int, long, long, long, int, const uint32_t *, float, uint8_t *, void *, void *, cudaStream_t);
int launch_rope_kv(const void *, const float *, const float *, void *, void *, void *, int, int, int, int, int, int, int, cudaStream_t);
int quant_token_tc_status(int *);
int launch_gptq_block(const float *, long, const float *, long, const float *, const float *, long, const int *, long, int, int, int,
                      float, float *, long, float *, cudaStream_t);

int quant_token_tc_wait_profile(unsigned long long *);
int quant_token_tc_status_clear();
int gemm_i8_wait_profile(unsigned long long *);
int gemm_i8_status_clear();

size_t gemm_decode_tc_workspace_bytes(long M, long N, long K);
bool gemm_decode_tc_supported(long M, long N, long K, long a_group);
int launch_gemm_decode_tc(const uint8_t *, const uint8_t *, const void *, const void *, const void *,
                          const int32_t *, const void *, void *, long, long, long, long, long, int, void *, cudaStream_t);
int gemm_decode_tc_status(int *);
int gemm_decode_tc_status_clear();
int gemm_decode_tc_wait_profile(unsigned long long *);

int gemm_tcgen05_status(int *);
int gemm_tcgen05_wait_profile(unsigned long long *);
int gemm_tcgen05_status_clear();

static bool is_pow2(long v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace flh

using namespace flh;

extern "C" {

int flh_b200_version(void) { return 100; }

const char *flh_b200_last_error(void) { return g_err; }

int flh_b200_device_check(void) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
    int major = 0, minor = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    FLH_REQUIRE(major == 10, FLH_B200_EUNSUPPORTED,
                "flh_b200 is built for sm_100a only; device %d is sm_%d%d", dev, major, minor);
    return 0;
}

int flh_b200_quant_group_sym_i4(const void *x, long rows, int gs, int hadamard, uint8_t *q,
                                void *scales, void *stream) {
    FLH_REQUIRE(rows >= 0, FLH_B200_EINVAL, "rows must be >= 0 (got %ld)", rows);
    FLH_REQUIRE(gs == 32 || gs == 64 || gs == 128, FLH_B200_EINVAL, "group size must be 32, 64 or 128 (got %d)", gs);
    if (rows == 0) return 0;
    FLH_REQUIRE(x && q && scales, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(x), FLH_B200_EALIGN, "x must be 16-byte aligned");
    FLH_REQUIRE((reinterpret_cast<uintptr_t>(q) & 3) == 0, FLH_B200_EALIGN, "q must be 4-byte aligned");
    return launch_quant_group_sym(x, rows, gs, hadamard != 0, q, scales, static_cast<cudaStream_t>(stream));
}

int flh_b200_hadamard_f16_inplace(void *x, long rows, int n, void *stream) {
    FLH_REQUIRE(rows >= 0, FLH_B200_EINVAL, "rows must be >= 0 (got %ld)", rows);
    FLH_REQUIRE(n == 32 || n == 64 || n == 128, FLH_B200_EINVAL, "row length must be 32, 64 or 128 (got %d)", n);
    if (rows == 0) return 0;
    FLH_REQUIRE(x, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(x), FLH_B200_EALIGN, "x must be 16-byte aligned");
    return launch_fht_inplace(x, rows, n, static_cast<cudaStream_t>(stream));
}

int flh_b200_quant_token_asym_i4(const void *x, int in_dtype, long M, long K, long ld, int hadamard,
                                 int kfac, const uint32_t *sign_bits, float clip, uint8_t *q,
                                 void *scale, void *zero, void *stream) {
    FLH_REQUIRE(M >= 0 && K > 0, FLH_B200_EINVAL, "bad shape M=%ld K=%ld", M, K);
    FLH_REQUIRE(in_dtype == FLH_B200_F16 || in_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "in_dtype must be F16 or BF16");
    FLH_REQUIRE(K % 64 == 0 && K <= 32768, FLH_B200_EINVAL, "K must be a multiple of 64 and <= 32768 (got %ld)", K);
    FLH_REQUIRE(hadamard >= 0 && hadamard <= 2, FLH_B200_EINVAL, "hadamard must be 0, 1 or 2 (got %d)", hadamard);
    FLH_REQUIRE(ld >= K && ld % 8 == 0, FLH_B200_EALIGN, "row stride must be >= K and a multiple of 8 elements (got %ld)", ld);
    FLH_REQUIRE(clip > 0.0f && clip <= 1.0f, FLH_B200_EINVAL, "clip ratio must be in (0, 1]");
    if (hadamard) {
        FLH_REQUIRE(kfac >= 1 && K % kfac == 0, FLH_B200_EINVAL, "kfac=%d does not divide K=%ld", kfac, K);
        const long p = K / kfac;
        FLH_REQUIRE(is_pow2(p) && p >= 64, FLH_B200_EINVAL, "K / kfac must be a power of two >= 64 (got %ld)", p);
        FLH_REQUIRE(kfac == 1 || (kfac % 4 == 0 && kfac <= 172 && sign_bits), FLH_B200_EINVAL,
                    "kfac must be 1 or a Hadamard order <= 172 with its sign bits");
    } else {
        kfac = 1;
    }
    if (M == 0) return 0;
    FLH_REQUIRE(x && q && scale && zero, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(x), FLH_B200_EALIGN, "x must be 16-byte aligned");
    FLH_REQUIRE((reinterpret_cast<uintptr_t>(q) & 7) == 0, FLH_B200_EALIGN, "q must be 8-byte aligned");
    FLH_REQUIRE(kfac == 1 || aligned16(sign_bits), FLH_B200_EALIGN, "the factor table must be 16-byte aligned");
    return launch_quant_token_asym(x, in_dtype, M, K, ld, hadamard, kfac, sign_bits, clip, q, scale,
                                   zero, static_cast<cudaStream_t>(stream));
}

int flh_b200_rmsnorm_quant_group_sym_i4(const void *x, long M, long K, float eps, int hadamard, uint8_t *q, void *scales,
                                        void *stream) {
    FLH_REQUIRE(M >= 0, FLH_B200_EINVAL, "bad row count %ld", M);
    FLH_REQUIRE(K == 4096, FLH_B200_EUNSUPPORTED, "the fused RMS-norm group quantiser serves K = 4096 (got %ld)", K);
    FLH_REQUIRE(eps >= 0.0f, FLH_B200_EINVAL, "eps must be >= 0");
    FLH_REQUIRE(hadamard == 0 || hadamard == 1, FLH_B200_EINVAL, "hadamard must be 0 or 1 (got %d)", hadamard);
    if (M == 0) return 0;
    FLH_REQUIRE(x && q && scales, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(x) && aligned16(q), FLH_B200_EALIGN, "x and q must be 16-byte aligned");
    return launch_rmsnorm_quant_group(x, M, hadamard, eps, q, scales, static_cast<cudaStream_t>(stream));
}

int flh_b200_rmsnorm_quant_token_asym_i4(const void *x, int in_dtype, long M, long K, long ld, float eps, int hadamard,
                                         float clip, uint8_t *q, void *scale, void *zero, void *stream) {
    FLH_REQUIRE(M >= 0 && K > 0, FLH_B200_EINVAL, "bad shape M=%ld K=%ld", M, K);
    FLH_REQUIRE(in_dtype == FLH_B200_F16 || in_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "in_dtype must be F16 or BF16");
    FLH_REQUIRE(K == 4096 || K == 8192, FLH_B200_EUNSUPPORTED, "the fused RMS-norm quantiser serves K = 4096 and 8192 (got %ld)", K);
    FLH_REQUIRE(eps >= 0.0f, FLH_B200_EINVAL, "eps must be >= 0");
    FLH_REQUIRE(hadamard == 0 || hadamard == 1, FLH_B200_EINVAL, "hadamard must be 0 or 1 (got %d)", hadamard);
    FLH_REQUIRE(ld >= K && ld % 8 == 0, FLH_B200_EALIGN, "row stride must be >= K and a multiple of 8 elements (got %ld)", ld);
    FLH_REQUIRE(clip > 0.0f && clip <= 1.0f, FLH_B200_EINVAL, "clip ratio must be in (0, 1]");
    if (M == 0) return 0;
    FLH_REQUIRE(x && q && scale && zero, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(x), FLH_B200_EALIGN, "x must be 16-byte aligned");
    FLH_REQUIRE(aligned16(q), FLH_B200_EALIGN, "q must be 16-byte aligned");
    return launch_quant_token_warp(x, in_dtype, M, K, ld, hadamard, eps, clip, q, scale, zero, static_cast<cudaStream_t>(stream));
}

int flh_b200_silu_mul(const void *gu, int in_dtype, long M, long F, long ld, void *out, void *stream) {
    FLH_REQUIRE(M >= 0 && F > 0 && F % 8 == 0, FLH_B200_EINVAL, "bad shape M=%ld F=%ld (F must be a multiple of 8)", M, F);
    FLH_REQUIRE(in_dtype == FLH_B200_F16 || in_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "in_dtype must be F16 or BF16");
    FLH_REQUIRE(ld >= 2 * F && ld % 8 == 0, FLH_B200_EALIGN, "row stride %ld must be >= 2F and a multiple of 8", ld);
    if (M == 0) return 0;
    FLH_REQUIRE(gu && out, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(gu) && aligned16(out), FLH_B200_EALIGN, "gu and out must be 16-byte aligned");
    return launch_silu_mul(gu, in_dtype, M, F, ld, out, static_cast<cudaStream_t>(stream));
}

int flh_b200_silu_mul_quant_token_asym_i4(const void *gu, int in_dtype, long M, long F, long ld, int hadamard, int kfac,
                                          const uint32_t *sign_bits, float clip, uint8_t *q, void *scale, void *zero,
                                          void *stream) {
    FLH_REQUIRE(M >= 0 && F > 0 && F % 64 == 0, FLH_B200_EINVAL, "bad shape M=%ld F=%ld (F must be a multiple of 64)", M, F);
    FLH_REQUIRE(in_dtype == FLH_B200_F16 || in_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "in_dtype must be F16 or BF16");
    FLH_REQUIRE(ld >= 2 * F && ld % 8 == 0, FLH_B200_EALIGN, "row stride %ld must be >= 2F and a multiple of 8", ld);
    FLH_REQUIRE(clip > 0.0f && clip <= 1.0f, FLH_B200_EINVAL, "clip must be in (0, 1]");
    FLH_REQUIRE(kfac >= 1 && F % kfac == 0 && (kfac == 1 || sign_bits), FLH_B200_EINVAL, "kfac=%d must divide F=%ld and come with its sign bits", kfac, F);
    if (hadamard != 1) return fail(FLH_B200_EUNSUPPORTED, "the fused form exists for hadamard = 1 only; run flh_b200_silu_mul and the quantiser separately");
    if (M == 0) return 0;
    FLH_REQUIRE(gu && q && scale && zero, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(gu) && aligned16(q), FLH_B200_EALIGN, "gu and q must be 16-byte aligned");
    const int rc = launch_silu_mul_quant_token_tc(gu, in_dtype, M, F, ld, kfac, sign_bits, clip, q, scale, zero, static_cast<cudaStream_t>(stream));
    if (rc == -1000) return fail(FLH_B200_EUNSUPPORTED, "F=%ld is not a width the fused form takes (F = P * 64, P <= 256); run the two steps separately", F);
    return rc;
}

int flh_b200_rope_kv_f16(const void *qkv, const float *cos, const float *sin, void *q_out, void *k_cache, void *v_cache,
                         int B, int S, int nh, int nkv, int D, int T, int cur, void *stream) {
    FLH_REQUIRE(B >= 0 && S >= 0 && nh > 0 && nkv > 0 && D > 0 && D % 8 == 0, FLH_B200_EINVAL, "bad shape B=%d S=%d nh=%d nkv=%d D=%d", B, S, nh, nkv, D);
    FLH_REQUIRE(cur >= 0 && cur + S <= T, FLH_B200_EINVAL, "positions %d .. %d do not fit a cache of %d", cur, cur + S - 1, T);
    if (B == 0 || S == 0) return 0;
    FLH_REQUIRE(qkv && cos && sin && q_out && k_cache && v_cache, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(qkv) && aligned16(cos) && aligned16(sin) && aligned16(q_out) && aligned16(k_cache) && aligned16(v_cache),
                FLH_B200_EALIGN, "pointers must be 16-byte aligned");
    return launch_rope_kv(qkv, cos, sin, q_out, k_cache, v_cache, B, S, nh, nkv, D, T, cur, static_cast<cudaStream_t>(stream));
}

const char *flh_b200_quant_token_kernel(long M, long K, int hadamard, int kfac) {
    return quant_token_kernel_name(M, K, hadamard, kfac);
}

size_t flh_b200_sign_table_bytes(int kfac) {
    if (kfac <= 0) return 0;
    const size_t bits_bytes = ((size_t)kfac * ((kfac + 31) / 32) * 4 + 15) / 16 * 16;
    const size_t kp = (size_t)(kfac + 15) / 16 * 16;
    return bits_bytes + kp * kp * 2;
}

int flh_b200_pack_signs(const int8_t *signs, int kfac, uint32_t *out) {
    FLH_REQUIRE(signs && out && kfac > 0, FLH_B200_EINVAL, "bad arguments");
    const int words = (kfac + 31) / 32;
    memset(out, 0, flh_b200_sign_table_bytes(kfac));
    for (int k = 0; k < kfac; ++k)
        for (int j = 0; j < kfac; ++j)
            if (signs[k * kfac + j] < 0) out[k * words + (j >> 5)] |= 1u << (j & 31);
    // the same matrix as bfloat16 +-1 (0x3F80 / 0xBF80), padded with zeros to a multiple of 16
    const size_t bits_bytes = ((size_t)kfac * words * 4 + 15) / 16 * 16;
    uint16_t *mat = reinterpret_cast<uint16_t *>(reinterpret_cast<uint8_t *>(out) + bits_bytes);
    const int kp = (kfac + 15) / 16 * 16;
    for (int k = 0; k < kfac; ++k)
        for (int j = 0; j < kfac; ++j) mat[(size_t)k * kp + j] = signs[k * kfac + j] < 0 ? 0xBF80u : 0x3F80u;
    return 0;
}

int flh_b200_weight_rowsum(const uint8_t *B, long N, long K, long group, int32_t *rowsum, void *stream) {
    FLH_REQUIRE(N >= 0 && K > 0 && group > 0, FLH_B200_EINVAL, "bad shape");
    FLH_REQUIRE(K % group == 0 && group % 32 == 0, FLH_B200_EINVAL, "group must divide K and be a multiple of 32");
    if (N == 0) return 0;
    FLH_REQUIRE(B && rowsum, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE((reinterpret_cast<uintptr_t>(B) & 3) == 0, FLH_B200_EALIGN, "B must be 4-byte aligned");
    return launch_weight_rowsum(B, N, K, group, rowsum, static_cast<cudaStream_t>(stream));
}

// Decode shapes where the tensor-core kernel beats the mma.sync streaming kernel (measured on B200): its set-up and
// the hand-over of shared tiles cost ~9 us, its streaming rate is higher and does not drop with the token count.
static bool decode_tc_pays(long M, long N, long K, long a_group) {
    const double mib = (double)N * (double)K / 2.0 / (1 << 20);            // packed weight bytes
    const double need = M > 32 ? 12.0 : (M > 16 ? 32.0 : 64.0);
    return mib >= need && gemm_decode_tc_supported(M, N, K, a_group);
}
static int pick_stream(long M, long N, long K) {
    return stream_splits(M, N, K) > 1 ? FLH_B200_GEMM_STREAM_SPLITK : FLH_B200_GEMM_STREAM;
}

int flh_b200_gemm_pick_algo(long M, long N, long K, long a_group, long b_group) {
    if ((a_group < b_group ? a_group : b_group) < 128) return FLH_B200_GEMM_MMA_SYNC;    // K-groups of 32 / 64
    if (M <= 64) return decode_tc_pays(M, N, K, a_group) ? FLH_B200_GEMM_DECODE_TC : pick_stream(M, N, K);
    // large batches without group scales: expanding both operands to int8 first pays for itself — from 1,536 rows, or from
    // 1,024 when the output is wide enough to fill the GPU with 256 x 256 tiles (measured crossovers on B200)
    if (a_group == K && b_group == K && (M >= 1536 || (M >= 1024 && N >= 8192)))
        return N % 256 == 0 ? FLH_B200_GEMM_TCGEN05_I8_PAIR : FLH_B200_GEMM_TCGEN05_I8;
    return FLH_B200_GEMM_TCGEN05;
}

size_t flh_b200_gemm_workspace_bytes(long M, long N, long K, long a_group, long b_group, int algo) {
    if (algo == FLH_B200_GEMM_AUTO) algo = flh_b200_gemm_pick_algo(M, N, K, a_group, b_group);
    if (algo == FLH_B200_GEMM_TCGEN05_I8 || algo == FLH_B200_GEMM_TCGEN05_I8_PAIR) return gemm_i8_workspace_bytes(M, N, K);
    if (algo == FLH_B200_GEMM_DECODE_TC) return M <= 64 ? gemm_decode_tc_workspace_bytes(M, N, K) : 0;
    if (algo != FLH_B200_GEMM_STREAM_SPLITK || M > 64) return 0;
    return stream_scratch_bytes(M, N, stream_splits(M, N, K));
}

int flh_b200_gemm_i4_dequant(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                             const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                             long M, long N, long K, long a_group, long b_group, int out_dtype, int algo,
                             void *workspace, size_t workspace_bytes, void *stream) {
    FLH_REQUIRE(M >= 0 && N >= 0 && K > 0, FLH_B200_EINVAL, "bad shape M=%ld N=%ld K=%ld", M, N, K);
    FLH_REQUIRE(K % 128 == 0 && K <= 65536, FLH_B200_EINVAL, "K must be a multiple of 128 and <= 65536 (got %ld)", K);
    FLH_REQUIRE(N % 128 == 0, FLH_B200_EINVAL, "N must be a multiple of 128 (got %ld)", N);
    const long gmin = a_group < b_group ? a_group : b_group;       // the K-group the integer sums are cut into
    FLH_REQUIRE(gmin == 32 || gmin == 64 || gmin == 128 || gmin == K, FLH_B200_EINVAL,
                "the smaller of a_group and b_group must be 32, 64, 128 or K (got %ld, %ld)", a_group, b_group);
    FLH_REQUIRE(a_group == gmin || a_group == K, FLH_B200_EINVAL, "a_group must be %ld or K (got %ld)", gmin, a_group);
    FLH_REQUIRE(b_group == gmin || b_group == K, FLH_B200_EINVAL, "b_group must be %ld or K (got %ld)", gmin, b_group);
    FLH_REQUIRE(out_dtype == FLH_B200_F16 || out_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "out_dtype must be F16 or BF16");
    if (M == 0 || N == 0) return 0;
    FLH_REQUIRE(A && B && a_scale && b_scale && D, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(!a_zero || b_rowsum, FLH_B200_EINVAL, "a_zero needs b_rowsum");
    FLH_REQUIRE(aligned16(A) && aligned16(B), FLH_B200_EALIGN, "A and B must be 16-byte aligned");
    FLH_REQUIRE((reinterpret_cast<uintptr_t>(D) & 15) == 0, FLH_B200_EALIGN, "D must be 16-byte aligned");
    if (gmin == 32 || gmin == 64) {
        // groups narrower than the 128-K stage: the mma.sync tile kernel that folds every group's sum with its own scales
        FLH_REQUIRE(algo == FLH_B200_GEMM_AUTO || algo == FLH_B200_GEMM_MMA_SYNC, FLH_B200_EUNSUPPORTED,
                    "K-groups of %ld are served by the mma.sync tile kernel only (algo AUTO or MMA_SYNC)", gmin);
        return launch_gemm_mma_tile_gs(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, (int)gmin,
                                       out_dtype, static_cast<cudaStream_t>(stream));
    }
    if (algo == FLH_B200_GEMM_AUTO) {
        algo = flh_b200_gemm_pick_algo(M, N, K, a_group, b_group);
        // without (enough) scratch the tensor-core decode kernel gives way to the streaming kernels
        if (algo == FLH_B200_GEMM_DECODE_TC &&
            (!workspace || workspace_bytes < gemm_decode_tc_workspace_bytes(M, N, K) || (reinterpret_cast<uintptr_t>(workspace) & 255)))
            algo = pick_stream(M, N, K);
        // without (enough) scratch the split-K form quietly gives way to the plain streaming kernel
        if (algo == FLH_B200_GEMM_STREAM_SPLITK &&
            (!workspace || workspace_bytes < stream_scratch_bytes(M, N, stream_splits(M, N, K))))
            algo = FLH_B200_GEMM_STREAM;
        // likewise the int8-operand kernels give way to the converting kernel
        if ((algo == FLH_B200_GEMM_TCGEN05_I8 || algo == FLH_B200_GEMM_TCGEN05_I8_PAIR) &&
            (!workspace || workspace_bytes < gemm_i8_workspace_bytes(M, N, K) || (reinterpret_cast<uintptr_t>(workspace) & 255)))
            algo = FLH_B200_GEMM_TCGEN05;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (algo) {
        case FLH_B200_GEMM_STREAM:
            FLH_REQUIRE(M <= 64, FLH_B200_EINVAL, "the streaming kernel serves M <= 64 (got %ld)", M);
            return launch_gemm_stream(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, 1, nullptr, s);
        case FLH_B200_GEMM_STREAM_SPLITK: {
            FLH_REQUIRE(M <= 64, FLH_B200_EINVAL, "the streaming kernel serves M <= 64 (got %ld)", M);
            const int splits = stream_splits(M, N, K);
            if (splits <= 1)
                return launch_gemm_stream(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, 1, nullptr, s);
            const size_t need = stream_scratch_bytes(M, N, splits);
            FLH_REQUIRE(workspace && workspace_bytes >= need, FLH_B200_EINVAL,
                        "split-K needs %zu bytes of zero-initialised workspace (got %zu)", need, workspace_bytes);
            FLH_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, FLH_B200_EALIGN, "workspace must be 256-byte aligned");
            return launch_gemm_stream(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, splits, workspace, s);
        }
        case FLH_B200_GEMM_DECODE_TC: {
            FLH_REQUIRE(M <= 64, FLH_B200_EINVAL, "the decode kernel serves M <= 64 (got %ld)", M);
            FLH_REQUIRE(gemm_decode_tc_supported(M, N, K, a_group), FLH_B200_EUNSUPPORTED,
                        "the decode kernel does not serve N=%ld K=%ld with this scale layout (too many tiles or token scales)", N, K);
            const size_t need = gemm_decode_tc_workspace_bytes(M, N, K);
            FLH_REQUIRE(workspace && workspace_bytes >= need, FLH_B200_EINVAL,
                        "the decode kernel needs %zu bytes of zero-initialised workspace (got %zu)", need, workspace_bytes);
            FLH_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, FLH_B200_EALIGN, "workspace must be 256-byte aligned");
            return launch_gemm_decode_tc(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, workspace, s);
        }
        case FLH_B200_GEMM_MMA_SYNC:
            return launch_gemm_mma_tile(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, s);
        case FLH_B200_GEMM_TCGEN05:
            return launch_gemm_tcgen05(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, 0, s);
        case FLH_B200_GEMM_TCGEN05_I8:
        case FLH_B200_GEMM_TCGEN05_I8_PAIR: {
            FLH_REQUIRE(a_group == K && b_group == K, FLH_B200_EINVAL, "the int8-operand kernels take per-token / per-channel scales only");
            const size_t need = gemm_i8_workspace_bytes(M, N, K);
            FLH_REQUIRE(workspace && workspace_bytes >= need, FLH_B200_EINVAL,
                        "the int8-operand kernels need %zu bytes of workspace (got %zu)", need, workspace_bytes);
            FLH_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, FLH_B200_EALIGN, "workspace must be 256-byte aligned");
            FLH_REQUIRE(algo == FLH_B200_GEMM_TCGEN05_I8 || N % 256 == 0, FLH_B200_EINVAL, "the two-CTA kernel needs N %% 256 == 0 (got %ld)", N);
            return launch_gemm_i8(A, B, nullptr, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, out_dtype,
                                  algo == FLH_B200_GEMM_TCGEN05_I8_PAIR, workspace, s);
        }
        case FLH_B200_GEMM_TCGEN05_DIRECT:
            return launch_gemm_tcgen05(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, 1, s);
        default:
            return fail(FLH_B200_EINVAL, "unknown algo %d", algo);
    }
}

int flh_b200_gemm_i4_dequant_decode_noalloc(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                                            const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                                            long M, long N, long K, long a_group, long b_group, int out_dtype,
                                            void *stream) {
    FLH_REQUIRE(M >= 0 && N >= 0 && K > 0, FLH_B200_EINVAL, "bad shape M=%ld N=%ld K=%ld", M, N, K);
    FLH_REQUIRE(M <= 64, FLH_B200_EINVAL, "the decode entry point serves M <= 64 (got %ld)", M);
    FLH_REQUIRE(K % 128 == 0 && K <= 65536, FLH_B200_EINVAL, "K must be a multiple of 128 and <= 65536 (got %ld)", K);
    FLH_REQUIRE(N % 128 == 0, FLH_B200_EINVAL, "N must be a multiple of 128 (got %ld)", N);
    FLH_REQUIRE(a_group == 128 || a_group == K, FLH_B200_EINVAL, "a_group must be 128 or K (got %ld)", a_group);
    FLH_REQUIRE(b_group == 128 || b_group == K, FLH_B200_EINVAL, "b_group must be 128 or K (got %ld)", b_group);
    FLH_REQUIRE(out_dtype == FLH_B200_F16 || out_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "out_dtype must be F16 or BF16");
    if (M == 0 || N == 0) return 0;
    FLH_REQUIRE(A && B && a_scale && b_scale && D, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(!a_zero || b_rowsum, FLH_B200_EINVAL, "a_zero needs b_rowsum");
    FLH_REQUIRE(aligned16(A) && aligned16(B), FLH_B200_EALIGN, "A and B must be 16-byte aligned");
    return launch_gemm_stream_static(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group,
                                     out_dtype, static_cast<cudaStream_t>(stream));
}

int flh_b200_expand_i4(const uint8_t *packed, long rows, long K, uint8_t *out, void *stream) {
    FLH_REQUIRE(rows >= 0 && K > 0 && K % 128 == 0, FLH_B200_EINVAL, "bad shape rows=%ld K=%ld (K must be a multiple of 128)", rows, K);
    if (rows == 0) return 0;
    FLH_REQUIRE(packed && out, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(packed) && (reinterpret_cast<uintptr_t>(out) & 127) == 0, FLH_B200_EALIGN,
                "packed must be 16-byte aligned and out 128-byte aligned");
    return launch_expand_i4(packed, rows, K, out, static_cast<cudaStream_t>(stream));
}

int flh_b200_gemm_i8w_dequant(const uint8_t *A, const uint8_t *B8, const void *a_scale, const void *a_zero,
                              const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D, long M, long N,
                              long K, int out_dtype, void *workspace, size_t workspace_bytes, void *stream) {
    FLH_REQUIRE(M >= 0 && N >= 0 && K > 0, FLH_B200_EINVAL, "bad shape M=%ld N=%ld K=%ld", M, N, K);
    FLH_REQUIRE(K % 128 == 0 && K <= 65536, FLH_B200_EINVAL, "K must be a multiple of 128 and <= 65536 (got %ld)", K);
    FLH_REQUIRE(N % 128 == 0, FLH_B200_EINVAL, "N must be a multiple of 128 (got %ld)", N);
    FLH_REQUIRE(out_dtype == FLH_B200_F16 || out_dtype == FLH_B200_BF16, FLH_B200_EINVAL, "out_dtype must be F16 or BF16");
    if (M == 0 || N == 0) return 0;
    FLH_REQUIRE(A && B8 && a_scale && b_scale && D, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(!a_zero || b_rowsum, FLH_B200_EINVAL, "a_zero needs b_rowsum");
    FLH_REQUIRE(aligned16(A) && (reinterpret_cast<uintptr_t>(B8) & 127) == 0, FLH_B200_EALIGN,
                "A must be 16-byte aligned and the expanded weights 128-byte aligned");
    FLH_REQUIRE((reinterpret_cast<uintptr_t>(D) & 15) == 0, FLH_B200_EALIGN, "D must be 16-byte aligned");
    FLH_REQUIRE(workspace && workspace_bytes >= (size_t)M * K, FLH_B200_EINVAL,
                "needs M * K = %zu bytes of workspace for the expanded activations (got %zu)", (size_t)M * K, workspace_bytes);
    FLH_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, FLH_B200_EALIGN, "workspace must be 256-byte aligned");
    return launch_gemm_i8(A, nullptr, B8, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, out_dtype,
                          N % 256 == 0, workspace, static_cast<cudaStream_t>(stream));
}

int flh_b200_gptq_block(const float *W, long ldw, const float *Hinv, long ldh, const float *scale, const float *zero,
                        long lds, const int *group_of_col, long rows, int count, int maxq, int sym, float clip_ratio,
                        float *Q, long ldq, float *Err, void *stream) {
    FLH_REQUIRE(rows >= 0 && count >= 1 && count <= 128, FLH_B200_EINVAL, "bad shape rows=%ld count=%d (count must be 1..128)", rows, count);
    FLH_REQUIRE(ldw >= count && ldh >= count && ldq >= count && lds >= 1, FLH_B200_EINVAL, "leading dimensions must cover the block");
    FLH_REQUIRE(maxq >= 1 && maxq <= 255, FLH_B200_EINVAL, "maxq must be 1..255 (got %d)", maxq);
    FLH_REQUIRE(clip_ratio > 0.0f, FLH_B200_EINVAL, "clip_ratio must be positive");
    if (rows == 0) return 0;
    FLH_REQUIRE(W && Hinv && scale && group_of_col && Q && Err, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(sym || zero, FLH_B200_EINVAL, "asymmetric quantisation needs zero-points");
    return launch_gptq_block(W, ldw, Hinv, ldh, scale, zero, lds, group_of_col, rows, count, maxq, sym != 0, clip_ratio, Q, ldq, Err,
                             static_cast<cudaStream_t>(stream));
}

int flh_b200_gemm_status(int *out) {
    FLH_REQUIRE(out, FLH_B200_EINVAL, "null pointer");
    int rc = gemm_tcgen05_status(out);
    if (rc) return rc;
    if (out[0]) return gemm_tcgen05_status_clear();
    rc = gemm_i8_status(out);
    if (rc) return rc;
    if (out[0]) return gemm_i8_status_clear();
    rc = quant_token_factor_status(out);
    if (rc) return rc;
    if (out[0]) return quant_token_factor_status_clear();
    rc = quant_token_tc_status(out);
    if (rc) return rc;
    if (out[0]) return quant_token_tc_status_clear();
    rc = gemm_decode_tc_status(out);
    if (rc) return rc;
    return out[0] ? gemm_decode_tc_status_clear() : 0;
}

int flh_b200_quant_token_wait_profile(unsigned long long *out) {
    FLH_REQUIRE(out, FLH_B200_EINVAL, "null pointer");
    return quant_token_tc_wait_profile(out);
}

int flh_b200_gemm_wait_profile(unsigned long long *out) {
    FLH_REQUIRE(out, FLH_B200_EINVAL, "null pointer");
    int rc = gemm_tcgen05_wait_profile(out);
    if (rc) return rc;
    bool any = false;
    for (int i = 0; i < 8; ++i) any = any || out[i] != 0;
    if (any) return 0;
    rc = gemm_i8_wait_profile(out);                    // nothing from the converting kernels: the int8-operand ones,
    if (rc) return rc;
    for (int i = 0; i < 8; ++i) any = any || out[i] != 0;
    return any ? 0 : gemm_decode_tc_wait_profile(out); // then the decode kernel
}

void flhDenseLayerGEMM_i4_o16(const uint8_t *A, const uint8_t *B, const void *A_scale, const void *B_scale,
                              void *D, size_t M, size_t N, size_t K) {
    (void)flh_b200_gemm_i4_dequant(A, B, A_scale, nullptr, B_scale, nullptr, nullptr, D, (long)M, (long)N,
                                   (long)K, 128, 128, FLH_B200_F16, FLH_B200_GEMM_AUTO, nullptr, 0, nullptr);
}

}  // extern "C"
