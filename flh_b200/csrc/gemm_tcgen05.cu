// int4 x int4 GEMM with fused dequantisation on the 5th-generation tensor cores.
//
//   TMA (cp.async.bulk.tensor.2d)  packed int4 tiles of A [128 x 64 B] and B [BN x 64 B] -> smem ring
//   6 converter warps              nibbles -> int8 (x16, see below) written in the K-major
//                                  128-byte-swizzled layout tcgen05 reads, fence.proxy.async
//   1 elected thread               tcgen05.mma.cta_group::1.kind::i8, int32 accumulators in TMEM
//   1-2 epilogue warpgroups        tcgen05.ld, dequantise (per 128-K group or once), f16/bf16 store
// The kernel is persistent (one CTA per SM walks the tile list) and the accumulator is double-buffered
// in TMEM, so the epilogue of one tile or K-group overlaps the tensor-core work of the next;
// setmaxnreg moves registers from the producer/converter warps to the epilogue warps.
//
// There is no int4 MMA kind on sm_100, so the expansion to int8 happens in shared memory.  It is
// exact and needs no sign extension: (w << 4) & 0xF0F0F0F0 and w & 0xF0F0F0F0 leave each nibble in
// the high half of a byte, i.e. the int8 value 16 * q.  Both operands are expanded by the same rule
// (even elements of a packed word first, then the odd ones), so products pair up correctly and the
// int32 dot product is 256 * sum(qa * qw) — shifted back (or folded into the scale) exactly.
//
// Group-128 scales: the accumulator of every 128-K block goes to one of two TMEM buffers; the
// epilogue warps drain buffer g while the MMA thread fills buffer g+1, and keep one binary32
// accumulator per output column in registers:  acc = fmaf(float(I_g), sa * sb, acc), g ascending.
//
// Every wait on an mbarrier is bounded (two seconds); a wait that runs out records where in a
// device status word, and the CTA drains its copies, frees its TMEM and returns.
#include "tc_common.cuh"

namespace flh {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;                 // int8 elements per stage = one 128-byte swizzle row

__device__ int g_status[4];             // [0] = first error code, [1] = block, [2] = kb
// Nanoseconds spent inside bounded waits, summed over CTAs, one representative thread per role:
// [1] producer on pk_empty, [2] MMA on acc_empty, [3] MMA on ex_full, [4] converter on pk_full,
// [5] converter on ex_empty, [6]/[7] epilogue on acc_full.  Diagnostic only (flh_b200_gemm_wait_profile).
__device__ unsigned long long g_wait_ns[8];

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code,
                                          unsigned long long *waited = nullptr) {
    return mbar_wait_status(g_status, bar, parity, abort_flag, code, waited);
}

struct TcParams {
    const __half *a_scale, *a_zero, *b_scale, *bias;
    const int32_t *b_rowsum;
    void *D;
    const uint8_t *A, *B;       // packed operands (direct-load variant)
    int M, N, K;
    int ga_cols, gb_cols;
    int out_bf16;
    int num_tiles, m_blocks;
};

// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM owner), then the converter warps, then
// the epilogue warps.  With group scales the epilogue is the heavy role: 6 converter warps and one epilogue
// warpgroup per 128 output columns (which also receive registers through setmaxnreg).  Without them the
// converters are: 12 converter warps and a single epilogue warpgroup that walks all columns of a tile while
// the next tile is already being multiplied.
constexpr int kConvTid0 = 64;
template <bool GROUPED> struct Roles {
    static constexpr int kConvWarps = GROUPED ? 6 : 12;
    static constexpr int kConvThreads = 32 * kConvWarps;
    static constexpr int kNonEpi = kConvTid0 + kConvThreads;          // 256 or 448
    static constexpr int epi_threads(int bn) { return GROUPED ? bn : 128; }
};

template <int BN>
struct SmemPlan {
    static constexpr int kStages = BN == 256 ? 3 : 4;
    static constexpr int kExpStage = (BM + BN) * BK;          // int8 bytes
    static constexpr int kPkStage = (BM + BN) * (BK / 2);     // packed bytes
    static constexpr int kExpOff = 0;
    static constexpr int kPkOff = kStages * kExpStage;
    static constexpr int kAuxOff = kPkOff + kStages * kPkStage;   // weight scales [2][BN] f32, row sums [2][BN] s32, bias [BN] f32
    static constexpr int kBarOff = kAuxOff + 5 * BN * 4;
    static constexpr int kBytes = kBarOff + 256 + 1024;           // + slack to align the base to 1024
    // registers per thread after setmaxnreg: the 256 producer/converter threads drop to kLowRegs, the BN
    // epilogue threads rise to kEpiRegs; 256 * kLowRegs + BN * kEpiRegs must fit the 64 K register file
    static constexpr int kLowRegs(bool direct) { return direct ? 80 : 64; }
    static constexpr int kEpiRegs(bool direct) { return BN == 256 ? (direct ? 176 : 192) : 232; }
};
static_assert(256 * SmemPlan<256>::kLowRegs(true) + 256 * SmemPlan<256>::kEpiRegs(true) <= 65536, "register budget");
static_assert(256 * SmemPlan<256>::kLowRegs(false) + 256 * SmemPlan<256>::kEpiRegs(false) <= 65536, "register budget");
static_assert(256 * SmemPlan<128>::kLowRegs(true) + 128 * SmemPlan<128>::kEpiRegs(true) <= 384 * 168, "register budget");

// Persistent: CTA b works on output tiles b, b + gridDim.x, ... (row blocks fastest, so the CTAs that
// run together share the same weight columns).  Barrier phases and the TMEM accumulator buffer are
// driven by running counters: `it` counts 128-K stages, `u` counts accumulator uses (one per K-block
// with group scales, one per tile otherwise); buffer u & 1 is filled while buffer (u - 1) & 1 drains.
// DIRECT: the converter warps fetch the packed operands from global memory (L2) straight into registers,
// one stage ahead, instead of reading tiles that TMA staged in shared memory.  Shared memory then carries
// only the int8 tiles (written once, read once by the tensor core), which is what bounds this kernel:
// per 128x256x128 stage 96 KB cross the shared-memory port instead of 144 KB.  Warp 0 turns into an L2
// prefetcher that runs a few stages ahead.
template <int BN, bool GROUPED, bool A_UNSIGNED, bool DIRECT>
__global__ void __launch_bounds__(Roles<GROUPED>::kNonEpi + Roles<GROUPED>::epi_threads(BN), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const TcParams p) {
    using Plan = SmemPlan<BN>;
    using R = Roles<GROUPED>;
    constexpr int S = Plan::kStages;
    constexpr int kTmemCols = 2 * BN;
    constexpr int kConvThreads = R::kConvThreads, kNonEpiThreads = R::kNonEpi, kEpiThreads = R::epi_threads(BN);
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_dyn + (base - raw);

    const uint32_t bars = base + Plan::kBarOff;
    auto pk_full = [&](int s) { return bars + 8u * s; };
    auto pk_empty = [&](int s) { return bars + 8u * (4 + s); };
    auto ex_full = [&](int s) { return bars + 8u * (8 + s); };
    auto ex_empty = [&](int s) { return bars + 8u * (12 + s); };
    auto acc_full = [&](int b) { return bars + 8u * (16 + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (18 + b); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + Plan::kBarOff + 8 * 20);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Plan::kBarOff + 8 * 20 + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = p.K / BK;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), kConvThreads);
            mbar_init(ex_full(s), kConvThreads);
            mbar_init(ex_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), kEpiThreads); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (tid < kNonEpiThreads) {
        if (GROUPED) {
            if (DIRECT) asm volatile("setmaxnreg.dec.sync.aligned.u32 80;" ::);
            else asm volatile("setmaxnreg.dec.sync.aligned.u32 64;" ::);
        }
        if (warp == 0 && DIRECT) {
            // -------------------------------------------------------- L2 prefetcher (direct-load variant)
            constexpr int kAhead = 6;                      // stages ahead of the converters
            const long ldk = p.K / 2;
            int it = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                const int m0 = (tile % p.m_blocks) * BM, n0 = (tile / p.m_blocks) * BN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    // stay at most kAhead stages ahead: the converters publish progress through ex_full
                    if (it >= kAhead) {
                        const int j = it - kAhead, sj = j % S;
                        if (!mbar_wait(ex_full(sj), (j / S) & 1, abort_flag, 8)) goto prefetch_done;
                    }
                    for (int r = lane; r < BM + BN; r += 32) {
                        const uint8_t *src = r < BM ? p.A + (long)min(m0 + r, p.M - 1) * ldk
                                                    : p.B + (long)(n0 + r - BM) * ldk;
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(src + kb * 64));
                    }
                }
            }
        prefetch_done:;
        } else if (warp == 0) {
            // -------------------------------------------------------- TMA producer
            if (lane == 0) {
                int it = 0;
                bool ok = true;
                unsigned long long w1 = 0;
                for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                    const int m0 = (tile % p.m_blocks) * BM, n0 = (tile / p.m_blocks) * BN;
                    for (int kb = 0; kb < KB; ++kb, ++it) {
                        const int s = it % S;
                        if (!mbar_wait(pk_empty(s), ((it / S) & 1) ^ 1, abort_flag, 1, &w1)) { ok = false; break; }
                        mbar_expect_tx(pk_full(s), Plan::kPkStage);
                        const uint32_t dst = base + Plan::kPkOff + s * Plan::kPkStage;
                        tma_load_2d(dst, &map_a, kb * (BK / 2), m0, pk_full(s));
                        tma_load_2d(dst + BM * (BK / 2), &map_b, kb * (BK / 2), n0, pk_full(s));
                    }
                }
                atomicAdd(&g_wait_ns[1], w1);
                if (*abort_flag) {
                    // let the copies already issued land before the CTA leaves
                    for (int j = it > S ? it - S : 0; j < it; ++j) {
                        const uint64_t t0 = gtimer();
                        while (!mbar_try(pk_full(j % S), (j / S) & 1) && gtimer() - t0 < 100000000ull) {}
                    }
                }
            }
        } else if (warp == 1) {
            // -------------------------------------------------------- MMA issuer
            if (lane == 0) {
                const uint32_t idesc = (2u << 4) | ((A_UNSIGNED ? 0u : 1u) << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                int it = 0, u = 0;
                bool ok = true;
                unsigned long long w2 = 0, w3 = 0;
                for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                    for (int kb = 0; kb < KB; ++kb, ++it) {
                        const int s = it % S;
                        const int buf = u & 1;
                        if ((GROUPED || kb == 0) && u >= 2) {
                            if (!mbar_wait(acc_empty(buf), ((u >> 1) & 1) ^ 1, abort_flag, 2, &w2)) { ok = false; break; }
                        }
                        if (!mbar_wait(ex_full(s), (it / S) & 1, abort_flag, 3, &w3)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_addr = base + Plan::kExpOff + s * Plan::kExpStage;
                        const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + BM * BK);
#pragma unroll
                        for (int k4 = 0; k4 < BK / 32; ++k4) {
                            const uint32_t accum = GROUPED ? (k4 > 0) : (kb > 0 || k4 > 0);
                            tc_mma_i8(tmem + buf * BN, adesc + 2 * k4, bdesc + 2 * k4, idesc, accum);
                        }
                        tc_commit(ex_empty(s));
                        if (GROUPED || kb == KB - 1) { tc_commit(acc_full(buf)); ++u; }
                    }
                }
                atomicAdd(&g_wait_ns[2], w2);
                atomicAdd(&g_wait_ns[3], w3);
            }
        } else {
            // -------------------------------------------------------- int4 -> int8 converters
            const int ct = tid - kConvTid0;                 // 0..191
            constexpr int kChunks = (BM + BN) * 4;          // 16-byte packed chunks per stage
            auto expand_store = [&](uint8_t *ex, int ch, const uint4 &w) {
                const int row = ch >> 2, c = ch & 3;        // rows of A, then rows of B
                uint4 e, o;
                e.x = (w.x << 4) & 0xF0F0F0F0u; e.y = (w.y << 4) & 0xF0F0F0F0u;
                e.z = (w.z << 4) & 0xF0F0F0F0u; e.w = (w.w << 4) & 0xF0F0F0F0u;
                o.x = w.x & 0xF0F0F0F0u; o.y = w.y & 0xF0F0F0F0u; o.z = w.z & 0xF0F0F0F0u; o.w = w.w & 0xF0F0F0F0u;
                uint8_t *dst = ex + row * 128;
                const int sw = row & 7;
                *reinterpret_cast<uint4 *>(dst + (((2 * c) ^ sw) << 4)) = e;
                *reinterpret_cast<uint4 *>(dst + (((2 * c + 1) ^ sw) << 4)) = o;
            };
            int it = 0;
            bool ok = true;
            unsigned long long w4 = 0, w5 = 0;
            if (DIRECT) {
                // Register pipeline, kDepth stages deep: slot d holds the packed chunks of stage it + d; a slot is
                // refilled with stage it + kDepth as soon as it has been expanded, so kDepth - 1 stages of global
                // loads are always in flight per thread.
                constexpr int kPer = (kChunks + kConvThreads - 1) / kConvThreads;   // chunks per thread per stage
                constexpr int kDepth = GROUPED ? 1 : 3;
                const long ldk = p.K / 2;
                uint4 w[kDepth][kPer];
                const uint8_t *src[kPer];
                int ex_off[kPer];
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    const int ch = ct + j * kConvThreads, row = ch >> 2, c = ch & 3;
                    ex_off[j] = ch < kChunks ? row * 128 + (((2 * c) ^ (row & 7)) << 4) : -1;
                }
                int f_tile = blockIdx.x, f_kb = 0;          // fetch cursor
                auto set_tile = [&](int tile) {
                    const int m0 = (tile % p.m_blocks) * BM, n0 = (tile / p.m_blocks) * BN;
#pragma unroll
                    for (int j = 0; j < kPer; ++j) {
                        const int ch = ct + j * kConvThreads;
                        const int row = ch >> 2, c = ch & 3;
                        if (ch >= kChunks) src[j] = nullptr;
                        else if (row < BM) src[j] = (m0 + row < p.M) ? p.A + (long)(m0 + row) * ldk + c * 16 : nullptr;
                        else src[j] = p.B + (long)(n0 + row - BM) * ldk + c * 16;
                    }
                };
                auto fetch_next = [&](uint4 (&dst)[kPer]) {
                    if (f_tile >= p.num_tiles) return;
#pragma unroll
                    for (int j = 0; j < kPer; ++j)
                        dst[j] = src[j] ? ldg_nc_v4(src[j] + f_kb * 64) : make_uint4(0, 0, 0, 0);
                    if (++f_kb == KB) {
                        f_kb = 0;
                        f_tile += gridDim.x;
                        if (f_tile < p.num_tiles) set_tile(f_tile);
                    }
                };
                if (f_tile < p.num_tiles) set_tile(f_tile);
#pragma unroll
                for (int d = 0; d < kDepth; ++d) fetch_next(w[d]);
                int my_tiles = 0;
                for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) ++my_tiles;
                const int total = my_tiles * KB;
                while (it < total && ok) {
#pragma unroll
                    for (int d = 0; d < kDepth; ++d) {
                        if (it >= total || !ok) break;
                        const int s = it % S;
                        if (!mbar_wait(ex_empty(s), ((it / S) & 1) ^ 1, abort_flag, 5, &w5)) { ok = false; break; }
                        uint8_t *ex = sm + Plan::kExpOff + s * Plan::kExpStage;
#pragma unroll
                        for (int j = 0; j < kPer; ++j) {
                            if (ex_off[j] >= 0) {
                                const uint4 v = w[d][j];
                                uint4 e, o;
                                e.x = (v.x << 4) & 0xF0F0F0F0u; e.y = (v.y << 4) & 0xF0F0F0F0u;
                                e.z = (v.z << 4) & 0xF0F0F0F0u; e.w = (v.w << 4) & 0xF0F0F0F0u;
                                o.x = v.x & 0xF0F0F0F0u; o.y = v.y & 0xF0F0F0F0u; o.z = v.z & 0xF0F0F0F0u; o.w = v.w & 0xF0F0F0F0u;
                                *reinterpret_cast<uint4 *>(ex + ex_off[j]) = e;
                                *reinterpret_cast<uint4 *>(ex + (ex_off[j] ^ 16)) = o;
                            }
                        }
                        fetch_next(w[d]);
                        fence_proxy_async();
                        mbar_arrive(ex_full(s));
                        ++it;
                    }
                }
            } else {
                // this thread's chunks are the same in every stage: their offsets are computed once
                constexpr int kPerT = (kChunks + kConvThreads - 1) / kConvThreads;
                constexpr int kBatch = GROUPED ? 4 : kPerT;
                int pk_off[kPerT], ex_off[kPerT];
#pragma unroll
                for (int j = 0; j < kPerT; ++j) {
                    const int ch = ct + j * kConvThreads;
                    const int row = ch >> 2, c = ch & 3;      // rows of A, then rows of B
                    pk_off[j] = ch < kChunks ? row * 64 + c * 16 : -1;
                    ex_off[j] = row * 128 + (((2 * c) ^ (row & 7)) << 4);
                }
                for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                    for (int kb = 0; kb < KB; ++kb, ++it) {
                        const int s = it % S;
                        if (!mbar_wait(pk_full(s), (it / S) & 1, abort_flag, 4, &w4)) { ok = false; break; }
                        if (!mbar_wait(ex_empty(s), ((it / S) & 1) ^ 1, abort_flag, 5, &w5)) { ok = false; break; }
                        const uint8_t *pk = sm + Plan::kPkOff + s * Plan::kPkStage;
                        uint8_t *ex = sm + Plan::kExpOff + s * Plan::kExpStage;
                        // the packed chunks are fetched in batches (independent shared loads in flight) and then
                        // expanded; with group scales the epilogue owns the registers, so the batches are smaller
#pragma unroll
                        for (int j0 = 0; j0 < kPerT; j0 += kBatch) {
                            uint4 wv[kBatch];
#pragma unroll
                            for (int j = 0; j < kBatch; ++j)
                                if (j0 + j < kPerT && pk_off[j0 + j] >= 0) wv[j] = *reinterpret_cast<const uint4 *>(pk + pk_off[j0 + j]);
#pragma unroll
                            for (int j = 0; j < kBatch; ++j) {
                                if (j0 + j < kPerT && pk_off[j0 + j] >= 0) {
                                    const uint4 w = wv[j];
                                    uint4 e, o;
                                    e.x = (w.x << 4) & 0xF0F0F0F0u; e.y = (w.y << 4) & 0xF0F0F0F0u;
                                    e.z = (w.z << 4) & 0xF0F0F0F0u; e.w = (w.w << 4) & 0xF0F0F0F0u;
                                    o.x = w.x & 0xF0F0F0F0u; o.y = w.y & 0xF0F0F0F0u; o.z = w.z & 0xF0F0F0F0u; o.w = w.w & 0xF0F0F0F0u;
                                    *reinterpret_cast<uint4 *>(ex + ex_off[j0 + j]) = e;          // 16-byte chunk 2c   ^ (row & 7)
                                    *reinterpret_cast<uint4 *>(ex + (ex_off[j0 + j] ^ 16)) = o;   // 16-byte chunk 2c+1 ^ (row & 7)
                                }
                            }
                        }
                        fence_proxy_async();
                        mbar_arrive(ex_full(s));
                        mbar_arrive(pk_empty(s));
                    }
                }
            }
            if (ct == 0) { atomicAdd(&g_wait_ns[4], w4); atomicAdd(&g_wait_ns[5], w5); }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        if (GROUPED) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Plan::kEpiRegs(DIRECT)));
        const int wg = (tid - kNonEpiThreads) >> 7;      // warpgroup index: which 128 columns (group scales); 0 otherwise
        const int et = (tid - kNonEpiThreads) & 127;     // 0..127 within the warpgroup
        const int wq = warp & 3;                         // TMEM lane quarter this warp may read
        float *sbuf = reinterpret_cast<float *>(sm + Plan::kAuxOff);               // [2][BN] weight scales
        int *rbuf = reinterpret_cast<int *>(sm + Plan::kAuxOff + 2 * BN * 4);      // [2][BN] weight row sums
        float *bbuf = reinterpret_cast<float *>(sm + Plan::kAuxOff + 4 * BN * 4);  // [BN] bias
        const uint32_t tlane = tmem + ((uint32_t)(wq * 32) << 16) + wg * 128;
        const int cbase = wg * 128;                      // first tile column of this warpgroup
        int u = 0;
        bool ok = true;
        unsigned long long w6 = 0;

        // A wait that runs out must not split the warpgroup: its threads meet at named barriers and at warp-wide
        // tcgen05.ld.  So the outcome of every wait is made warp-uniform by a vote, and a warp that gave up keeps
        // walking the loops (no waits, no TMEM reads, no stores) and still reaches every named barrier.
        for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
            const int m0 = (tile % p.m_blocks) * BM, n0 = (tile / p.m_blocks) * BN;
            const int row = m0 + wq * 32 + lane;
            const int rowc = row < p.M ? row : p.M - 1;
            const int gcol = n0 + cbase + et;            // the column this thread stages
            if (GROUPED) {
                const int G = KB;
                const int gbs = p.gb_cols == 1 ? 0 : 1, gas = p.ga_cols == 1 ? 0 : 1;
                uint64_t acc[64];
#pragma unroll
                for (int i = 0; i < 64; ++i) acc[i] = 0ull;
                sbuf[cbase + et] = __half2float(p.b_scale[(long)gcol * p.gb_cols]);
                if (A_UNSIGNED) rbuf[cbase + et] = p.b_rowsum[(long)gcol * G];
                bar_sync_named(1 + wg, 128);
                for (int kb = 0; kb < KB; ++kb, ++u) {
                    const int buf = u & 1, slot = kb & 1;
                    float nsb = 0.f; int nrs = 0;
                    if (kb + 1 < KB) {                   // next group's column data, fetched early
                        nsb = __half2float(p.b_scale[(long)gcol * p.gb_cols + gbs * (kb + 1)]);
                        if (A_UNSIGNED) nrs = p.b_rowsum[(long)gcol * G + kb + 1];
                    }
                    // 256 * sum arrives from the tensor core; without zero-points the 1/256 rides in the scale
                    float sa = __half2float(p.a_scale[(long)rowc * p.ga_cols + gas * kb]);
                    if (!A_UNSIGNED) sa *= (1.0f / 256.0f);
                    const int za = A_UNSIGNED ? (int)__half2float(p.a_zero[(long)rowc * p.ga_cols + gas * kb]) : 0;
                    const uint64_t sa2 = pack2(sa, sa);
                    ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full(buf), (u >> 1) & 1, abort_flag, 6, &w6));
                    tc_fence_after();
                    const float *sb = sbuf + slot * BN + cbase;
                    const int *rs = rbuf + slot * BN + cbase;
                    // the next 32-column chunk is in flight from TMEM while this one is folded into the accumulators
                    uint32_t vv[2][32];
                    if (ok) tc_ld32(tlane + buf * BN, vv[0]);
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        if (!ok) break;
                        tc_wait_ld();
                        if (cc + 1 < 4) tc_ld32(tlane + buf * BN + (cc + 1) * 32, vv[(cc + 1) & 1]);
                        const uint32_t (&v)[32] = vv[cc & 1];
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const int col = cc * 32 + j;
                            const float2 sbp = *reinterpret_cast<const float2 *>(sb + col);
                            int i0 = (int)v[j], i1 = (int)v[j + 1];
                            if (A_UNSIGNED) { i0 = (i0 >> 8) - za * rs[col]; i1 = (i1 >> 8) - za * rs[col + 1]; }
                            const uint64_t p2 = mul2(sa2, pack2(sbp.x, sbp.y));
                            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[col >> 1]) : "l"(pack2((float)i0, (float)i1)), "l"(p2));
                        }
                    }
                    tc_fence_before();
                    mbar_arrive(acc_empty(buf));
                    if (kb + 1 < KB) { sbuf[(slot ^ 1) * BN + cbase + et] = nsb; if (A_UNSIGNED) rbuf[(slot ^ 1) * BN + cbase + et] = nrs; }
                    bar_sync_named(1 + wg, 128);
                }
                if (ok && row < p.M) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        float o[32];
#pragma unroll
                        for (int j = 0; j < 16; ++j) unpack2(acc[cc * 16 + j], o[2 * j], o[2 * j + 1]);
                        if (p.bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) o[j] = __fadd_rn(o[j], __half2float(p.bias[n0 + cbase + cc * 32 + j]));
                        }
                        store_row_chunk(p.D, p.out_bf16, (long)row * p.N + n0 + cbase + cc * 32, o);
                    }
                }
            } else {
                // one warpgroup serves the whole tile: stage scale, row sum and bias of all BN columns
                for (int c = et; c < BN; c += 128) {
                    sbuf[c] = __half2float(p.b_scale[n0 + c]);
                    rbuf[c] = A_UNSIGNED ? p.b_rowsum[n0 + c] : 0;
                    bbuf[c] = p.bias ? __half2float(p.bias[n0 + c]) : 0.0f;
                }
                bar_sync_named(1, 128);
                const float sa = __half2float(p.a_scale[rowc]) * (1.0f / 256.0f);
                const int za = A_UNSIGNED ? (int)__half2float(p.a_zero[rowc]) : 0;
                const int buf = u & 1;
                ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full(buf), (u >> 1) & 1, abort_flag, 7, &w6));
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
                mbar_arrive(acc_empty(buf));
                ++u;
                bar_sync_named(1, 128);                  // the staging arrays are rewritten for the next tile
            }
        }
        if (et == 0 && wg == 0) atomicAdd(&g_wait_ns[6], w6);
    }

    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
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

// rows x (K/2) bytes, row-major; box = box_rows x 64 bytes, no swizzle, out-of-range rows read as 0.
int make_map(CUtensorMap *map, const uint8_t *ptr, long rows, long K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(FLH_B200_EUNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FLH_B200_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

template <int BN, bool GROUPED, bool U, bool DIRECT>
int launch_t(const CUtensorMap &ma, const CUtensorMap &mb, const TcParams &p, cudaStream_t stream) {
    auto kern = gemm_tcgen05_kernel<BN, GROUPED, U, DIRECT>;
    const int smem = SmemPlan<BN>::kBytes;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "gemm_tcgen05 attribute");
    TcParams q = p;
    q.m_blocks = (p.M + BM - 1) / BM;
    q.num_tiles = q.m_blocks * (p.N / BN);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = kNumSMs;
    }
    const int grid = q.num_tiles < sms ? q.num_tiles : sms;        // one persistent CTA per SM
    kern<<<grid, Roles<GROUPED>::kNonEpi + Roles<GROUPED>::epi_threads(BN), smem, stream>>>(ma, mb, q);
    return cuda_status(cudaGetLastError(), "gemm_tcgen05 launch");
}

}  // namespace

int launch_gemm_tcgen05(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                        const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D, long M,
                        long N, long K, long a_group, long b_group, int out_dtype, int direct, cudaStream_t stream) {
    TcParams p;
    p.A = A; p.B = B;
    p.a_scale = static_cast<const __half *>(a_scale);
    p.a_zero = static_cast<const __half *>(a_zero);
    p.b_scale = static_cast<const __half *>(b_scale);
    p.bias = static_cast<const __half *>(bias);
    p.b_rowsum = b_rowsum; p.D = D;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.ga_cols = (int)(K / a_group); p.gb_cols = (int)(K / b_group);
    p.out_bf16 = out_dtype == FLH_B200_BF16;
    const bool grouped = a_group < K || b_group < K;
    const int bn = (N % 256 == 0) ? 256 : 128;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, M, K, BM);
    if (rc) return rc;
    rc = make_map(&mb, B, N, K, bn);
    if (rc) return rc;
    const bool u = a_zero != nullptr;
#define FLH_TC(BN_, G_) \
    (direct ? (u ? launch_t<BN_, G_, true, true>(ma, mb, p, stream) : launch_t<BN_, G_, false, true>(ma, mb, p, stream)) \
            : (u ? launch_t<BN_, G_, true, false>(ma, mb, p, stream) : launch_t<BN_, G_, false, false>(ma, mb, p, stream)))
    if (grouped && bn == 256) return FLH_TC(256, true);
    if (grouped) return FLH_TC(128, true);
    if (bn == 256) return FLH_TC(256, false);
    return FLH_TC(128, false);
#undef FLH_TC
}

// Host-side read of the device status word the bounded waits write (synchronises the device).
int gemm_tcgen05_status(int *out4) {
    cudaError_t e = cudaMemcpyFromSymbol(out4, g_status, sizeof(int) * 4);
    return cuda_status(e, "status read");
}
// Reads and clears the wait-time counters (8 x unsigned long long, nanoseconds summed over CTAs).
int gemm_tcgen05_wait_profile(unsigned long long *out8) {
    cudaError_t e = cudaMemcpyFromSymbol(out8, g_wait_ns, sizeof(unsigned long long) * 8);
    if (e != cudaSuccess) return cuda_status(e, "wait profile read");
    unsigned long long z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_wait_ns, z, sizeof(z)), "wait profile clear");
}
int gemm_tcgen05_status_clear() {
    int z[4] = {0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_status, z, sizeof(z)), "status clear");
}

}  // namespace flh
