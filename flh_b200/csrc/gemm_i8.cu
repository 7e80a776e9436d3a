// int4 x int4 GEMM for large token batches, per-token / per-channel scales: the nibbles of both operands
// are first expanded to int8 (16 * q, no sign extension needed) into a caller-provided workspace, then a
// persistent tcgen05 kernel multiplies the int8 tiles that TMA lays straight into the 128-byte-swizzled
// layout the tensor core reads.  Shared memory then carries every operand byte exactly twice (TMA write,
// tensor-core read) instead of three and a half times when the expansion happens inside the GEMM.
//
//   expand_i4_kernel   packed [rows, K/2] -> int8 [rows, K]; every 16 packed bytes give 16 even then 16 odd
//                      elements (the same order for both operands, so products still pair up); exact
//   gemm_i8_kernel     warp 0 TMA producer, warp 1 MMA issuer (tcgen05.mma kind::i8, int32 accumulators,
//                      two TMEM buffers), warps 4-7 epilogue (tcgen05.ld, zero-point term, scales, bias,
//                      f16/bf16 rows).  PAIR = true runs two CTAs of a cluster on one 256 x 256 tile
//                      (tcgen05 cta_group::2): each CTA loads 128 rows of A and 128 rows of B, the leader
//                      issues the MMAs for both, commits are multicast to both CTAs' barriers, the peer's TMA
//                      loads complete on the leader's barrier, and the peer reports its drained accumulators
//                      with remote mbarrier arrives.
// The int32 dot product is 256 * sum(qa qw); the factor is folded back exactly in the epilogue.
// Every wait is bounded (two seconds) and reports through the same status word as the other GEMM kernels.
#include "tc_common.cuh"
#include <cooperative_groups.h>

namespace flh {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;

__device__ int g_status_i8[4];
// Nanoseconds inside bounded waits, summed over CTAs: [1] producer on empty, [2] MMA on acc_empty, [3] MMA on full,
// [6] epilogue on acc_full, [7] MMA issuers (CTAs, or clusters).  Diagnostic only.
__device__ unsigned long long g_wait_ns_i8[8];

__device__ __forceinline__ bool wait_i8(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code,
                                        unsigned long long *waited = nullptr) {
    return mbar_wait_status(g_status_i8, bar, parity, abort_flag, code, waited);
}

// ---- cluster helpers (PAIR) -------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(bar), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(raddr) : "memory");
}
// TMA tile load of a CTA of a pair whose completion is counted on the barrier at the same offset in CTA 0
__device__ __forceinline__ void tma_load_2d_to_leader(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    uint32_t rbar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(rbar) : "r"(bar));
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(rbar) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tc_mma_i8_plain(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    if (PAIR)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}

// ---- expansion --------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) expand_i4_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, long n16) {
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint4 w = ldg_nc_v4(in + i);
        uint4 e, o;
        e.x = (w.x << 4) & 0xF0F0F0F0u; e.y = (w.y << 4) & 0xF0F0F0F0u;
        e.z = (w.z << 4) & 0xF0F0F0F0u; e.w = (w.w << 4) & 0xF0F0F0F0u;
        o.x = w.x & 0xF0F0F0F0u; o.y = w.y & 0xF0F0F0F0u; o.z = w.z & 0xF0F0F0F0u; o.w = w.w & 0xF0F0F0F0u;
        out[2 * i] = e;
        out[2 * i + 1] = o;
    }
}

struct I8Params {
    const __half *a_scale, *a_zero, *b_scale, *bias;
    const int32_t *b_rowsum;
    void *D;
    int M, N, K;
    int out_bf16;
    int num_tiles, m_blocks;        // tiles of (PAIR ? 256 : 128) x BN, row blocks fastest
};

// BN = columns of an output tile; BNL = rows of B this CTA loads per stage (BN, or BN / 2 in a pair)
template <int BN, bool PAIR>
struct I8Plan {
    static constexpr int BNL = PAIR ? BN / 2 : BN;
    static constexpr int kStageBytes = (BM + BNL) * BK;
    static constexpr int kStages = kStageBytes == 48 * 1024 ? 4 : 6;
    static constexpr int kAuxOff = kStages * kStageBytes;            // weight scales f32 [BN], row sums s32 [BN], bias f32 [BN]
    static constexpr int kBarOff = kAuxOff + 3 * BN * 4;
    static constexpr int kBytes = kBarOff + 512 + 1024;              // barriers, then slack to align the base to 1024
    static constexpr int kThreads = 256;
};

template <int BN, bool A_UNSIGNED, bool PAIR>
__global__ void __launch_bounds__(256, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const I8Params p) {
    using Plan = I8Plan<BN, PAIR>;
    constexpr int S = Plan::kStages;
    constexpr int kTmemCols = 2 * BN;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;        // the same offset in both CTAs of a pair
    uint8_t *sm = smem_dyn + (base - raw);

    const uint32_t bars = base + Plan::kBarOff;
    auto full = [&](int s) { return bars + 8u * s; };                 // the tiles of stage s have landed (a pair: both CTAs', counted by the leader)
    auto empty = [&](int s) { return bars + 8u * (16 + s); };        // the tensor core has read stage s
    auto acc_full = [&](int b) { return bars + 8u * (24 + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (26 + b); };    // leader only in a pair
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + Plan::kBarOff + 8 * 28);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Plan::kBarOff + 8 * 28 + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = p.K / BK;
    const uint32_t rank = PAIR ? cluster_rank() : 0u;
    const int first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), PAIR ? 256 : 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();            // both CTAs' barriers exist before anyone signals across
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (own halves)
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            unsigned long long w1 = 0;
            for (int tile = first; tile < p.num_tiles && ok; tile += step) {
                const int m0 = (tile % p.m_blocks) * (PAIR ? 2 * BM : BM) + (int)rank * BM;
                const int n0 = (tile / p.m_blocks) * BN + (int)rank * Plan::BNL;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    if (!wait_i8(empty(s), ((it / S) & 1) ^ 1, abort_flag, 11, &w1)) { ok = false; break; }
                    const uint32_t dst = base + s * Plan::kStageBytes;
                    if (PAIR && rank == 1) {
                        // the leader's barrier counts these bytes too (it has expected them, or will: a transaction
                        // count may run negative for a while, and the phase cannot end before the leader's arrive)
                        tma_load_2d_to_leader(dst, &map_a, kb * BK, m0, full(s));
                        tma_load_2d_to_leader(dst + BM * BK, &map_b, kb * BK, n0, full(s));
                    } else {
                        mbar_expect_tx(full(s), (PAIR ? 2 : 1) * Plan::kStageBytes);
                        tma_load_2d(dst, &map_a, kb * BK, m0, full(s));
                        tma_load_2d(dst + BM * BK, &map_b, kb * BK, n0, full(s));
                    }
                }
            }
            if (rank == 0) atomicAdd(&g_wait_ns_i8[1], w1);
            if (*abort_flag && rank == 0) {  // let the copies already issued land before the CTA leaves
                for (int j = it > S ? it - S : 0; j < it; ++j) {
                    const uint64_t t0 = gtimer();
                    while (!mbar_try(full(j % S), (j / S) & 1) && gtimer() - t0 < 100000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (the leader's, in a pair)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (2u << 4) | ((A_UNSIGNED ? 0u : 1u) << 7) | (1u << 10) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((PAIR ? 2 * BM : BM) >> 4) << 24);
            int it = 0, u = 0;
            bool ok = true;
            unsigned long long w2 = 0, w3 = 0, w4 = 0;
            // The outcome of the wait is made warp-uniform by a vote, and a warp that gave up keeps walking the tile loop
        // (no waits, no TMEM reads, no stores): the four warps meet at named barriers and at warp-wide tcgen05.ld, so
        // none of them may leave alone.
        for (int tile = first; tile < p.num_tiles; tile += step, ++u) {
                const int buf = u & 1;
                if (u >= 2 && !wait_i8(acc_empty(buf), ((u >> 1) & 1) ^ 1, abort_flag, 12, &w2)) { ok = false; break; }
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    if (!wait_i8(full(s), (it / S) & 1, abort_flag, 13, &w3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * Plan::kStageBytes;
                    const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + BM * BK);
#pragma unroll
                    for (int k4 = 0; k4 < BK / 32; ++k4)
                        tc_mma_i8_plain<PAIR>(tmem + buf * BN, adesc + 2 * k4, bdesc + 2 * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
                    if (PAIR) tc_commit_pair(empty(s)); else tc_commit(empty(s));
                }
                if (ok) { if (PAIR) tc_commit_pair(acc_full(buf)); else tc_commit(acc_full(buf)); }
            }
            atomicAdd(&g_wait_ns_i8[2], w2); atomicAdd(&g_wait_ns_i8[3], w3); atomicAdd(&g_wait_ns_i8[4], w4);
            atomicAdd(&g_wait_ns_i8[7], 1ull);
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ epilogue
        const int et = tid - 128;                        // 0..127
        const int wq = warp & 3;                         // TMEM lane quarter this warp may read
        float *sbuf = reinterpret_cast<float *>(sm + Plan::kAuxOff);
        int *rbuf = reinterpret_cast<int *>(sm + Plan::kAuxOff + BN * 4);
        float *bbuf = reinterpret_cast<float *>(sm + Plan::kAuxOff + 2 * BN * 4);
        const uint32_t tlane = tmem + ((uint32_t)(wq * 32) << 16);
        int u = 0;
        bool ok = true;
        // The outcome of the wait is made warp-uniform by a vote, and a warp that gave up keeps walking the tile loop
        // (no waits, no TMEM reads, no stores): the four warps meet at named barriers and at warp-wide tcgen05.ld, so
        // none of them may leave alone.
        for (int tile = first; tile < p.num_tiles; tile += step, ++u) {
            const int m0 = (tile % p.m_blocks) * (PAIR ? 2 * BM : BM) + (int)rank * BM;
            const int n0 = (tile / p.m_blocks) * BN;
            const int row = m0 + wq * 32 + lane;
            const int rowc = row < p.M ? row : p.M - 1;
            for (int c = et; c < BN; c += 128) {
                sbuf[c] = __half2float(p.b_scale[n0 + c]);
                rbuf[c] = A_UNSIGNED ? p.b_rowsum[n0 + c] : 0;
                bbuf[c] = p.bias ? __half2float(p.bias[n0 + c]) : 0.0f;
            }
            bar_sync_named(1, 128);
            const float sa = __half2float(p.a_scale[rowc]) * (1.0f / 256.0f);
            const int za = A_UNSIGNED ? (int)__half2float(p.a_zero[rowc]) : 0;
            const int buf = u & 1;
            ok = __all_sync(0xffffffffu, ok && wait_i8(acc_full(buf), (u >> 1) & 1, abort_flag, 16));
            tc_fence_after();
#pragma unroll 1
            for (int cc = 0; cc < BN / 32 && ok; ++cc) {
                uint32_t v[32];
                tc_ld32(tlane + buf * BN + cc * 32, v);
                tc_wait_ld();
                float o[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = cc * 32 + j;
                    const int I = (int)v[j] - ((za * rbuf[col]) << 8);
                    float r = __fmaf_rn((float)I, __fmul_rn(sa, sbuf[col]), 0.0f);
                    if (p.bias) r = __fadd_rn(r, bbuf[col]);
                    o[j] = r;
                }
                if (row < p.M) store_row_chunk(p.D, p.out_bf16, (long)row * p.N + n0 + cc * 32, o);
            }
            tc_fence_before();
            if (PAIR && rank == 1) mbar_arrive_remote(acc_empty(buf), 0); else mbar_arrive(acc_empty(buf));
            bar_sync_named(1, 128);                      // the staging arrays are rewritten for the next tile
        }
    }

    __syncthreads();
    if (PAIR) cluster_sync_all();            // nobody signals the peer's barriers or reads its tiles after this
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// rows x K bytes, row-major; box = box_rows x 128 bytes written with the 128-byte swizzle; rows past the end read as 0.
int make_map_i8(CUtensorMap *map, const uint8_t *ptr, long rows, long K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(FLH_B200_EUNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FLH_B200_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

int device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = kNumSMs;
    }
    return sms;
}

template <int BN, bool U, bool PAIR>
int launch_i8(const CUtensorMap &ma, const CUtensorMap &mb, const I8Params &p, cudaStream_t stream) {
    using Plan = I8Plan<BN, PAIR>;
    auto kern = gemm_i8_kernel<BN, U, PAIR>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kBytes);
    if (e != cudaSuccess) return cuda_status(e, "gemm_i8 attribute");
    I8Params q = p;
    const int tile_m = PAIR ? 2 * BM : BM;
    q.m_blocks = (p.M + tile_m - 1) / tile_m;
    q.num_tiles = q.m_blocks * (p.N / BN);
    const int sms = device_sms();
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.blockDim = dim3(Plan::kThreads);
    cfg.dynamicSmemBytes = Plan::kBytes;
    cfg.stream = stream;
    if (PAIR) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        // the kernel is persistent: launch no more clusters than can be resident at once
        static int max_pairs = 0;
        if (max_pairs == 0) {
            cfg.gridDim = dim3(sms / 2 * 2);
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) n = sms / 2;
            max_pairs = n;
        }
        int pairs = max_pairs;
        if (q.num_tiles < pairs) pairs = q.num_tiles;
        cfg.gridDim = dim3(2 * pairs);
    } else {
        cfg.gridDim = dim3(q.num_tiles < sms ? q.num_tiles : sms);
    }
    e = cudaLaunchKernelEx(&cfg, kern, ma, mb, q);
    return cuda_status(e, "gemm_i8 launch");
}

}  // namespace

size_t gemm_i8_workspace_bytes(long M, long N, long K) {
    const size_t a = ((size_t)M * K + 255) & ~(size_t)255;
    return a + (size_t)N * K;
}

int launch_expand_i4(const uint8_t *packed, long rows, long K, uint8_t *out, cudaStream_t stream) {
    const long n16 = rows * K / 32;                            // 16-byte packed chunks
    if (n16 == 0) return 0;
    long grid = (n16 + 255) / 256;
    const long cap = 8L * device_sms();
    if (grid > cap) grid = cap;
    expand_i4_kernel<<<(unsigned)grid, 256, 0, stream>>>(reinterpret_cast<const uint4 *>(packed), reinterpret_cast<uint4 *>(out), n16);
    return cuda_status(cudaGetLastError(), "expand_i4 launch");
}

// pair = 0: one CTA per 128 x BN tile; pair = 1: two-CTA clusters on 256 x 256 tiles (needs N % 256 == 0).
// B8 != nullptr: the weights are already expanded (launch_expand_i4), only A goes through the workspace.
int launch_gemm_i8(const uint8_t *A, const uint8_t *B, const uint8_t *B8, const void *a_scale, const void *a_zero,
                   const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D, long M, long N, long K,
                   int out_dtype, int pair, void *workspace, cudaStream_t stream) {
    uint8_t *ea = static_cast<uint8_t *>(workspace);
    const uint8_t *eb = B8;
    int rc = launch_expand_i4(A, M, K, ea, stream);
    if (rc) return rc;
    if (!eb) {
        uint8_t *dst = ea + (((size_t)M * K + 255) & ~(size_t)255);
        rc = launch_expand_i4(B, N, K, dst, stream);
        if (rc) return rc;
        eb = dst;
    }
    I8Params p;
    p.a_scale = static_cast<const __half *>(a_scale);
    p.a_zero = static_cast<const __half *>(a_zero);
    p.b_scale = static_cast<const __half *>(b_scale);
    p.bias = static_cast<const __half *>(bias);
    p.b_rowsum = b_rowsum; p.D = D;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.out_bf16 = out_dtype == FLH_B200_BF16;
    const bool u = a_zero != nullptr;
    CUtensorMap ma, mb;
    rc = make_map_i8(&ma, ea, M, K, BM);
    if (rc) return rc;
    if (pair) {
        if (N % 256 != 0) return fail(FLH_B200_EINVAL, "the two-CTA kernel needs N %% 256 == 0 (got %ld)", N);
        rc = make_map_i8(&mb, eb, N, K, 128);
        if (rc) return rc;
        return u ? launch_i8<256, true, true>(ma, mb, p, stream) : launch_i8<256, false, true>(ma, mb, p, stream);
    }
    const int bn = (N % 256 == 0) ? 256 : 128;
    rc = make_map_i8(&mb, eb, N, K, bn);
    if (rc) return rc;
    if (bn == 256) return u ? launch_i8<256, true, false>(ma, mb, p, stream) : launch_i8<256, false, false>(ma, mb, p, stream);
    return u ? launch_i8<128, true, false>(ma, mb, p, stream) : launch_i8<128, false, false>(ma, mb, p, stream);
}

int gemm_i8_wait_profile(unsigned long long *out8) {
    cudaError_t e = cudaMemcpyFromSymbol(out8, g_wait_ns_i8, sizeof(unsigned long long) * 8);
    if (e != cudaSuccess) return cuda_status(e, "wait profile read");
    unsigned long long z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_wait_ns_i8, z, sizeof(z)), "wait profile clear");
}

int gemm_i8_status(int *out4) {
    return cuda_status(cudaMemcpyFromSymbol(out4, g_status_i8, sizeof(int) * 4), "status read");
}
int gemm_i8_status_clear() {
    int z[4] = {0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_status_i8, z, sizeof(z)), "status clear");
}

}  // namespace flh
