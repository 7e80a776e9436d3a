// Decode GEMM (M <= 64 tokens) on the 5th-generation tensor cores, operands swapped: the 128 output channels of a
// weight tile are the M side of tcgen05.mma kind::i8 (one TMEM lane each), the tokens the N side (16, 32 or 64
// columns), so the kernel streams the packed weights once and spends no CUDA-core multiply on them.
//
//   warp 0 (one thread)   TMA: 128 x 64 B of packed weights + TOK x 64 B of packed tokens per 128-K block -> smem ring
//   warps 2-5             nibbles -> int8 (x16) in the K-major 128-byte-swizzled layout tcgen05 reads
//   warp 1 (one thread)   four tcgen05.mma (K = 32 each) per block; D[channel][token] int32 in TMEM
//   warps 6-9 (6-13 for 64 tokens: two groups, 32 token columns each)
//                         thread = output channel: tcgen05.ld of its token sums of a block, dequantise
//                         (acc = fmaf(float(I_g), sa * sb, acc) per 128-K group, or once per channel), store D^T
//
// Work split ("stream-K"): the (tile, K-block) pairs are laid out in one line, tile-major, and cut into equal
// contiguous ranges, one per CTA, so that every CTA streams the same number of bytes whatever N is.  A range
// that covers only part of a tile's K leaves a partial sum (int32 without group scales — exact; a binary32
// chain with them) in the workspace; the last CTA to arrive at a tile (a counter per tile, no waiting) adds the
// parts in K order and writes the outputs.  With group scales a tile whose K is shared by several CTAs is
// therefore within rounding of the single-chain result (the same bits on every run); without them the result
// does not depend on the split.
//
// Every mbarrier wait is bounded (two seconds) and reports through a status word; a CTA that gives up drains
// its copies, frees its TMEM and returns.
#include "tc_common.cuh"

namespace flh {
namespace {

constexpr int BR = 128;                 // output channels per tile = MMA M
constexpr int BK = 128;                 // K per stage = one 128-byte swizzle row of int8
// One arrival counter per tile and epilogue group, in the first 4 KB of the workspace: the same 4 KB the split-K
// streaming kernel keeps its slab counters in (both leave them zero, and everything after is scratch for both),
// so one workspace can serve whichever of the two AUTO picks for a shape.
constexpr int kMaxTiles = 512;          // N <= 65536
constexpr int kCounterBytes = 2 * kMaxTiles * 4;

__device__ int g_status[4];

// Nanoseconds spent inside bounded waits, summed over CTAs, one representative thread per role: [1] producer on
// pk_empty, [2] MMA on acc_empty, [3] MMA on ex_full, [4] converter on pk_full, [5] converter on ex_empty,
// [6] epilogue on acc_full, [7] epilogue in the arrival protocol of shared tiles.  Diagnostic only.
__device__ unsigned long long g_wait_ns[8];

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code,
                                          unsigned long long *waited = nullptr) {
    // the first try may already sleep in hardware, so the whole call is timed
    const uint64_t t0 = waited ? gtimer() : 0;
    const bool ok = mbar_wait_status(g_status, bar, parity, abort_flag, code);
    if (waited) *waited += gtimer() - t0;
    return ok;
}

struct DecParams {
    const __half *a_scale, *a_zero, *b_scale, *bias;
    const int32_t *b_rowsum;
    void *D;
    int M, N, K, KB;
    int ga_cols, gb_cols, out_bf16;
    int per, total;                     // K-blocks per CTA; tiles * KB
    int *counters;
    float *partials;                    // [2 * grid][TOK][128]
};

template <int TOK, bool GROUPED>
struct DecPlan {
    static constexpr bool kTwo = TOK <= 32;                 // two CTAs per SM
    static constexpr int SP = TOK == 16 ? 7 : (TOK == 32 ? 6 : 10);  // packed stages in flight (TMA)
    static constexpr int SE = kTwo ? 2 : 3;                 // expanded stages
    static constexpr int NBUF = GROUPED ? 4 : 2;            // TMEM accumulators
    static constexpr int EG = TOK == 64 ? 2 : 1;            // epilogue groups of four warps, TOK / EG token columns each
    static constexpr int kThreads = 192 + 128 * EG;
    static constexpr int kTmemCols = NBUF * TOK < 32 ? 32 : NBUF * TOK;
    static constexpr int kPkStage = (BR + TOK) * (BK / 2);
    static constexpr int kExStage = (BR + TOK) * BK;
    static constexpr int kExOff = 0;
    static constexpr int kPkOff = SE * kExStage;
    static constexpr int kBarOff = kPkOff + SP * kPkStage;
    static constexpr int kAuxOff = kBarOff + 512;           // token scales f32, then token zero-points s32
    static constexpr int kSlack = 1024;                     // to align the base
};

template <int TOK>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[TOK]) {
    if constexpr (TOK == 16) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                       "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                     : "r"(taddr) : "memory");
    } else {
#pragma unroll
        for (int c = 0; c < TOK / 32; ++c) tc_ld32(taddr + 32 * c, *reinterpret_cast<uint32_t (*)[32]>(&v[32 * c]));
    }
}

template <int TOK, bool GROUPED, bool A_UNSIGNED>
__global__ void __launch_bounds__((DecPlan<TOK, GROUPED>::kThreads), TOK <= 32 ? 2 : 1)
gemm_decode_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const DecParams p) {
    using Plan = DecPlan<TOK, GROUPED>;
    constexpr int SP = Plan::SP, SE = Plan::SE, NBUF = Plan::NBUF, EG = Plan::EG, TE = TOK / EG;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_dyn + (base - raw);

    const uint32_t bars = base + Plan::kBarOff;
    auto pk_full = [&](int s) { return bars + 8u * s; };
    auto pk_empty = [&](int s) { return bars + 8u * (SP + s); };
    auto ex_full = [&](int s) { return bars + 8u * (2 * SP + s); };
    auto ex_empty = [&](int s) { return bars + 8u * (2 * SP + SE + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * SP + 2 * SE + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * SP + 2 * SE + NBUF + b); };
    static_assert(8 * (2 * SP + 2 * SE + 2 * NBUF) <= 320, "barrier area");
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + Plan::kBarOff + 320);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Plan::kBarOff + 328);
    volatile int *s_last = reinterpret_cast<volatile int *>(sm + Plan::kBarOff + 336);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = p.KB;
    const int lin_begin = blockIdx.x * p.per;
    const int lin_end = min(p.total, lin_begin + p.per);
    const int count = lin_end - lin_begin;          // K-blocks this CTA streams (> 0 by the choice of the grid)

    // token scales (and zero-points) of the whole K: [group][token] with group scales on the token side, [token]
    // otherwise; tokens past M read as zero.  The epilogue warps stage them while the first tiles are in flight.
    const int sa_n = p.ga_cols > 1 ? KB * TOK : TOK;
    float *sa_s = reinterpret_cast<float *>(sm + Plan::kAuxOff);
    int *za_s = reinterpret_cast<int *>(sa_s + sa_n);

    if (tid == 0) {
        for (int s = 0; s < SP; ++s) { mbar_init(pk_full(s), 1); mbar_init(pk_empty(s), 128); }
        for (int s = 0; s < SE; ++s) { mbar_init(ex_full(s), 128); mbar_init(ex_empty(s), 1); }
        for (int b = 0; b < NBUF; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 128 * EG); }
        *abort_flag = 0;
        s_last[0] = 0; s_last[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Plan::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int tile = lin_begin / KB, kb = lin_begin - tile * KB;
            int it = 0;
            unsigned long long w1 = 0;
            for (; it < count; ++it) {
                const int s = it % SP;
                if (!mbar_wait(pk_empty(s), ((it / SP) & 1) ^ 1, abort_flag, 1, &w1)) break;
                mbar_expect_tx(pk_full(s), Plan::kPkStage);
                const uint32_t dst = base + Plan::kPkOff + s * Plan::kPkStage;
                tma_load_2d(dst, &map_w, kb * (BK / 2), tile * BR, pk_full(s));
                tma_load_2d(dst + BR * (BK / 2), &map_x, kb * (BK / 2), 0, pk_full(s));
                if (++kb == KB) { kb = 0; ++tile; }
            }
            atomicAdd(&g_wait_ns[1], w1);
            if (*abort_flag) {
                // let the copies already issued land before the CTA leaves
                for (int j = it > SP ? it - SP : 0; j < it; ++j) {
                    const uint64_t t0 = gtimer();
                    while (!mbar_try(pk_full(j % SP), (j / SP) & 1) && gtimer() - t0 < 100000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // D s32; A = weights (signed), B = tokens (unsigned codes with zero-points, else signed); N = TOK, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | ((A_UNSIGNED ? 0u : 1u) << 10) |
                                   ((uint32_t)(TOK >> 3) << 17) | ((uint32_t)(BR >> 4) << 24);
            int kb = lin_begin % KB;
            int u = 0;
            unsigned long long w2 = 0, w3 = 0;
            for (int it = 0; it < count; ++it) {
                const int s = it % SE;
                const int buf = u % NBUF;
                const bool seg_first = it == 0 || kb == 0;
                const bool seg_last = it == count - 1 || kb == KB - 1;
                if ((GROUPED || seg_first) && u >= NBUF) {
                    if (!mbar_wait(acc_empty(buf), ((u / NBUF) & 1) ^ 1, abort_flag, 2, &w2)) break;
                }
                if (!mbar_wait(ex_full(s), (it / SE) & 1, abort_flag, 3, &w3)) break;
                tc_fence_after();
                const uint32_t a_addr = base + Plan::kExOff + s * Plan::kExStage;
                const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + BR * BK);
#pragma unroll
                for (int k4 = 0; k4 < BK / 32; ++k4) {
                    const uint32_t accum = GROUPED ? (k4 > 0) : (!seg_first || k4 > 0);
                    tc_mma_i8(tmem + buf * TOK, adesc + 2 * k4, bdesc + 2 * k4, idesc, accum);
                }
                tc_commit(ex_empty(s));
                if (GROUPED || seg_last) { tc_commit(acc_full(buf)); ++u; }
                if (++kb == KB) kb = 0;
            }
            atomicAdd(&g_wait_ns[2], w2);
            atomicAdd(&g_wait_ns[3], w3);
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ int4 -> int8 converters
        const int ct = tid - 64;                          // 0..127
        constexpr int kChunks = (BR + TOK) * 4;           // 16-byte packed chunks per stage: weight rows, then token rows
        constexpr int kPerT = (kChunks + 127) / 128;
        int pk_off[kPerT], ex_off[kPerT];
#pragma unroll
        for (int j = 0; j < kPerT; ++j) {
            const int ch = ct + j * 128;
            const int row = ch >> 2, c = ch & 3;
            pk_off[j] = ch < kChunks ? ch * 16 : -1;
            ex_off[j] = row * 128 + (((2 * c) ^ (row & 7)) << 4);
        }
        unsigned long long w4 = 0, w5 = 0;
        for (int it = 0; it < count; ++it) {
            const int sp = it % SP, se = it % SE;
            if (!mbar_wait(pk_full(sp), (it / SP) & 1, abort_flag, 4, &w4)) break;
            if (!mbar_wait(ex_empty(se), ((it / SE) & 1) ^ 1, abort_flag, 5, &w5)) break;
            const uint8_t *pk = sm + Plan::kPkOff + sp * Plan::kPkStage;
            uint8_t *ex = sm + Plan::kExOff + se * Plan::kExStage;
            uint4 wv[kPerT];
#pragma unroll
            for (int j = 0; j < kPerT; ++j)
                if (pk_off[j] >= 0) wv[j] = *reinterpret_cast<const uint4 *>(pk + pk_off[j]);
#pragma unroll
            for (int j = 0; j < kPerT; ++j) {
                if (pk_off[j] >= 0) {
                    const uint4 w = wv[j];
                    uint4 e, o;
                    e.x = (w.x << 4) & 0xF0F0F0F0u; e.y = (w.y << 4) & 0xF0F0F0F0u;
                    e.z = (w.z << 4) & 0xF0F0F0F0u; e.w = (w.w << 4) & 0xF0F0F0F0u;
                    o.x = w.x & 0xF0F0F0F0u; o.y = w.y & 0xF0F0F0F0u; o.z = w.z & 0xF0F0F0F0u; o.w = w.w & 0xF0F0F0F0u;
                    *reinterpret_cast<uint4 *>(ex + ex_off[j]) = e;            // 16-byte chunk 2c   ^ (row & 7)
                    *reinterpret_cast<uint4 *>(ex + (ex_off[j] ^ 16)) = o;     // 16-byte chunk 2c+1 ^ (row & 7)
                }
            }
            fence_proxy_async();
            mbar_arrive(ex_full(se));
            mbar_arrive(pk_empty(sp));
        }
        if (ct == 0) { atomicAdd(&g_wait_ns[4], w4); atomicAdd(&g_wait_ns[5], w5); }
    } else {
        // ------------------------------------------------------------ epilogue: thread = output channel
        // 64 token columns are shared by two groups of four warps (32 columns each): the per-group work of a K-block
        // is what bounds this role
        const int eg = (tid - 192) >> 7;                 // epilogue group
        const int et = (tid - 192) & 127;                // 0..127 within the group
        const int j0 = eg * TE;                          // first token column of this group
        const int wq = warp & 3;                         // the TMEM lane quarter this warp may read
        const int r = wq * 32 + lane;                    // channel within the tile = TMEM lane
        const uint32_t tlane = tmem + ((uint32_t)(wq * 32) << 16);
        const int gbs = p.gb_cols > 1 ? 1 : 0, gas = p.ga_cols > 1 ? TOK : 0;
        if (p.ga_cols > 1) {
            // only the K-groups this CTA multiplies; consecutive threads read consecutive groups of one token
            const int ng = min(count, KB);
            for (int i = tid - 192; i < ng * TOK; i += 128 * EG) {
                const int j = i / ng, kb = (lin_begin + (i - j * ng)) % KB;
                sa_s[kb * TOK + j] = j < p.M ? __half2float(p.a_scale[(long)j * KB + kb]) : 0.0f;
                if (A_UNSIGNED) za_s[kb * TOK + j] = j < p.M ? (int)__half2float(p.a_zero[(long)j * KB + kb]) : 0;
            }
        } else {
            for (int j = tid - 192; j < TOK; j += 128 * EG) {
                sa_s[j] = j < p.M ? __half2float(p.a_scale[j]) : 0.0f;
                if (A_UNSIGNED) za_s[j] = j < p.M ? (int)__half2float(p.a_zero[j]) : 0;
            }
        }
        bar_sync_named(1, 128 * EG);
        int u = 0;
        bool ok = true;
        unsigned long long w6 = 0, w7 = 0;
        // A wait that runs out must not split the four warps: they meet at named barriers.  The outcome of every
        // wait is made warp-uniform by a vote, and a warp that gave up keeps walking (no waits, no TMEM reads, no
        // stores) and still reaches every barrier and the arrival counters.
        int lin = lin_begin;
        while (lin < lin_end) {
            const int tile = lin / KB, kb0 = lin - tile * KB;
            const int kb1 = min(KB, kb0 + (lin_end - lin));
            const int n = tile * BR + r;
            const bool whole = kb0 == 0 && kb1 == KB;
            uint64_t accf[TE / 2];                       // binary32 chains, two tokens per register pair
            int acci[TE];                                // int32 sums (x256) without group scales
#pragma unroll
            for (int j = 0; j < TE / 2; ++j) accf[j] = 0ull;

            if (GROUPED) {
                // 256 * sum arrives from the tensor core; without zero-points the 1/256 rides in the weight scale
                const float unit = A_UNSIGNED ? 1.0f : (1.0f / 256.0f);
                float sbv = __half2float(p.b_scale[(long)n * p.gb_cols + gbs * kb0]) * unit;
                int rsv = A_UNSIGNED ? p.b_rowsum[(long)n * KB + kb0] : 0;
                for (int kb = kb0; kb < kb1; ++kb, ++u) {
                    float nsb = sbv;
                    int nrs = rsv;
                    if (kb + 1 < kb1) {                  // the next group's channel data, fetched early
                        if (gbs) nsb = __half2float(p.b_scale[(long)n * p.gb_cols + kb + 1]) * unit;
                        if (A_UNSIGNED) nrs = p.b_rowsum[(long)n * KB + kb + 1];
                    }
                    const int buf = u % NBUF;
                    ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full(buf), (u / NBUF) & 1, abort_flag, 6, &w6));
                    tc_fence_after();
                    uint32_t v[TE];
                    if (ok) { tmem_ld_cols<TE>(tlane + buf * TOK + j0, v); tc_wait_ld(); }
                    tc_fence_before();
                    mbar_arrive(acc_empty(buf));
                    if (ok) {
                        const float *sa = sa_s + gas * kb + j0;
                        const int *za = za_s + gas * kb + j0;
                        const uint64_t sb2 = pack2(sbv, sbv);
#pragma unroll
                        for (int j = 0; j < TE; j += 2) {
                            const float2 sap = *reinterpret_cast<const float2 *>(sa + j);
                            int i0 = (int)v[j], i1 = (int)v[j + 1];
                            if (A_UNSIGNED) { i0 = (i0 >> 8) - za[j] * rsv; i1 = (i1 >> 8) - za[j + 1] * rsv; }
                            const uint64_t p2 = mul2(pack2(sap.x, sap.y), sb2);
                            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(accf[j >> 1]) : "l"(pack2((float)i0, (float)i1)), "l"(p2));
                        }
                    }
                    sbv = nsb; rsv = nrs;
                }
            } else {
                const int buf = u % NBUF;
                ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full(buf), (u / NBUF) & 1, abort_flag, 7, &w6));
                tc_fence_after();
                uint32_t v[TE];
                if (ok) { tmem_ld_cols<TE>(tlane + buf * TOK + j0, v); tc_wait_ld(); }
                tc_fence_before();
                mbar_arrive(acc_empty(buf));
                ++u;
#pragma unroll
                for (int j = 0; j < TE; ++j) acci[j] = ok ? (int)v[j] : 0;
            }

            bool finish = whole;
            if (!whole) {
                // this CTA holds only part of the tile's K: leave the partial sums, count the arrival
                const int first_cta = (tile * KB) / p.per, last_cta = (tile * KB + KB - 1) / p.per;
                const int slot = 2 * blockIdx.x + (lin_begin / KB == tile ? 0 : 1);
                float *dst = p.partials + ((size_t)slot * TOK + j0) * BR + r;
                if (ok) {
#pragma unroll
                    for (int j = 0; j < TE; ++j) {
                        float lo, hi;
                        unpack2(accf[j >> 1], lo, hi);
                        dst[j * BR] = GROUPED ? ((j & 1) ? hi : lo) : __int_as_float(acci[j]);
                    }
                }
                const uint64_t t7 = gtimer();
                __threadfence();
                bar_sync_named(2 + eg, 128);
                if (et == 0) s_last[eg] = atomicAdd(&p.counters[tile + eg * kMaxTiles], 1) == last_cta - first_cta;
                bar_sync_named(2 + eg, 128);
                finish = s_last[eg] != 0;
                if (finish) {
                    __threadfence();
#pragma unroll
                    for (int j = 0; j < TE / 2; ++j) accf[j] = 0ull;
#pragma unroll
                    for (int j = 0; j < TE; ++j) acci[j] = 0;
                    constexpr int PF = TE == 16 ? 4 : 2;     // parts whose loads are in flight together
                    for (int c0 = first_cta; c0 <= last_cta; c0 += PF) {
                        float w[PF][TE];
#pragma unroll
                        for (int q = 0; q < PF; ++q) {
                            const int c = min(c0 + q, last_cta);
                            const int sl = 2 * c + ((c * p.per) / KB == tile ? 0 : 1);
                            const float *src = p.partials + ((size_t)sl * TOK + j0) * BR + r;
#pragma unroll
                            for (int j = 0; j < TE; ++j) w[q][j] = __ldcg(src + j * BR);
                        }
#pragma unroll
                        for (int q = 0; q < PF; ++q) {
                            if (c0 + q > last_cta) break;
#pragma unroll
                            for (int j = 0; j < TE; j += 2) {
                                if (GROUPED) accf[j >> 1] = (c0 + q == first_cta) ? pack2(w[q][j], w[q][j + 1]) : add2(accf[j >> 1], pack2(w[q][j], w[q][j + 1]));
                                else { acci[j] += __float_as_int(w[q][j]); acci[j + 1] += __float_as_int(w[q][j + 1]); }
                            }
                        }
                    }
                    if (et == 0) p.counters[tile + eg * kMaxTiles] = 0;     // ready for the next launch
                }
                w7 += gtimer() - t7;
            }

            if (finish && ok) {
                const float bias = p.bias ? __half2float(p.bias[n]) : 0.0f;
                float sbc = 0.0f;
                int rsc = 0;
                if (!GROUPED) {
                    sbc = __half2float(p.b_scale[n]) * (1.0f / 256.0f);
                    rsc = A_UNSIGNED ? p.b_rowsum[n] : 0;
                }
#pragma unroll
                for (int j = 0; j < TE; ++j) {
                    float lo, hi;
                    unpack2(accf[j >> 1], lo, hi);
                    float o = (j & 1) ? hi : lo;
                    const int tok = j0 + j;
                    if (!GROUPED) {
                        const int I = A_UNSIGNED ? acci[j] - ((za_s[tok] * rsc) << 8) : acci[j];
                        o = __fmaf_rn((float)I, __fmul_rn(sa_s[tok], sbc), 0.0f);
                    }
                    if (p.bias) o = __fadd_rn(o, bias);
                    if (tok < p.M) {
                        if (p.out_bf16) static_cast<__nv_bfloat16 *>(p.D)[(long)tok * p.N + n] = __float2bfloat16_rn(o);
                        else static_cast<__half *>(p.D)[(long)tok * p.N + n] = __float2half_rn(o);
                    }
                }
            }
            lin += kb1 - kb0;
        }
        if (et == 0 && eg == 0) { atomicAdd(&g_wait_ns[6], w6); atomicAdd(&g_wait_ns[7], w7); }
    }

    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Plan::kTmemCols) : "memory");
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

// rows x (K/2) bytes, row-major; box = box_rows x 64 bytes, no swizzle, rows past the end read as 0.  The last few
// maps are remembered per host thread: a decode step multiplies the same weights again and again.
struct MapKey { const void *ptr; long rows, K; int box; };
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
struct MapCache { MapSlot slots[16]; int next; };
thread_local MapCache g_maps_w, g_maps_x;           // weights and tokens apart: fresh token buffers do not evict the weights

int get_map(MapCache &cache, const CUtensorMap **out, const uint8_t *ptr, long rows, long K, int box_rows) {
    for (int i = 0; i < 16; ++i) {
        const MapSlot &s = cache.slots[i];
        if (s.used && s.key.ptr == ptr && s.key.rows == rows && s.key.K == K && s.key.box == box_rows) { *out = &s.map; return 0; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(FLH_B200_EUNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    MapSlot &s = cache.slots[cache.next];
    cache.next = (cache.next + 1) % 16;
    s.used = false;
    cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(&s.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FLH_B200_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    s.key = MapKey{ptr, rows, K, box_rows};
    s.used = true;
    *out = &s.map;
    return 0;
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = kNumSMs;
    }
    return sms;
}

struct DecodeSplit { int tok, grid, per; };

// Token columns, CTAs and K-blocks per CTA for a shape: as many CTAs as can be resident (two per SM up to 32
// tokens, one above), never fewer than four K-blocks each unless the whole problem is smaller than that.
DecodeSplit decode_split(long M, long N, long K) {
    DecodeSplit d;
    d.tok = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const long total = (N / BR) * (K / BK);
    const long slots = (long)sm_count() * (d.tok <= 32 ? 2 : 1);
    long per = (total + slots - 1) / slots;
    if (per < 4) per = total < 4 ? total : 4;
    d.per = (int)per;
    d.grid = (int)((total + per - 1) / per);
    return d;
}

template <int TOK, bool G, bool U>
int launch_t(const CUtensorMap &mw, const CUtensorMap &mx, const DecParams &p, int grid, int aux_bytes, cudaStream_t stream) {
    using Plan = DecPlan<TOK, G>;
    auto kern = gemm_decode_tc_kernel<TOK, G, U>;
    const int smem = Plan::kAuxOff + aux_bytes + Plan::kSlack;
    if (smem > 227 * 1024) return fail(FLH_B200_EUNSUPPORTED, "K = %d needs %d bytes of shared memory for the token scales", p.K, smem);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "gemm_decode_tc attribute");
    kern<<<grid, Plan::kThreads, smem, stream>>>(mw, mx, p);
    return cuda_status(cudaGetLastError(), "gemm_decode_tc launch");
}

template <int TOK>
int launch_tok(const CUtensorMap &mw, const CUtensorMap &mx, const DecParams &p, bool grouped, bool u, int grid, int aux, cudaStream_t s) {
    if (grouped) return u ? launch_t<TOK, true, true>(mw, mx, p, grid, aux, s) : launch_t<TOK, true, false>(mw, mx, p, grid, aux, s);
    return u ? launch_t<TOK, false, true>(mw, mx, p, grid, aux, s) : launch_t<TOK, false, false>(mw, mx, p, grid, aux, s);
}

}  // namespace

// Shapes the kernel serves: M <= 64, at most 512 tiles of 128 channels, and token scales of the whole K that fit
// beside the stage rings in shared memory (group scales on the token side are the large case).
bool gemm_decode_tc_supported(long M, long N, long K, long a_group) {
    if (M < 1 || M > 64 || N % BR || K % BK || N / BR > kMaxTiles) return false;
    const int tok = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const long aux = (a_group < K ? (K / BK) * tok : tok) * 8;      // with zero-points
    const long fixed = tok == 16 ? DecPlan<16, true>::kAuxOff : (tok == 32 ? DecPlan<32, true>::kAuxOff : DecPlan<64, true>::kAuxOff);
    return fixed + aux + 1024 <= 227 * 1024;
}

// Zero-initialised scratch the kernel needs: arrival counters (left at zero again) and two partial-sum slots per CTA.
size_t gemm_decode_tc_workspace_bytes(long M, long N, long K) {
    const DecodeSplit d = decode_split(M, N, K);
    return kCounterBytes + (size_t)2 * d.grid * d.tok * BR * sizeof(float);
}

int launch_gemm_decode_tc(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                          const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D, long M,
                          long N, long K, long a_group, long b_group, int out_dtype, void *workspace,
                          cudaStream_t stream) {
    if (N / BR > kMaxTiles) return fail(FLH_B200_EUNSUPPORTED, "N = %ld is more than the %d tiles the counters cover", N, kMaxTiles);
    DecParams p;
    p.a_scale = static_cast<const __half *>(a_scale);
    p.a_zero = static_cast<const __half *>(a_zero);
    p.b_scale = static_cast<const __half *>(b_scale);
    p.bias = static_cast<const __half *>(bias);
    p.b_rowsum = b_rowsum; p.D = D;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KB = (int)(K / BK);
    p.ga_cols = (int)(K / a_group); p.gb_cols = (int)(K / b_group);
    p.out_bf16 = out_dtype == FLH_B200_BF16;
    const DecodeSplit d = decode_split(M, N, K);
    p.per = d.per;
    p.total = (int)((N / BR) * (K / BK));
    p.counters = static_cast<int *>(workspace);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + kCounterBytes);
    const bool grouped = a_group < K || b_group < K;
    const bool u = a_zero != nullptr;
    const int aux = (p.ga_cols > 1 ? p.KB * d.tok : d.tok) * (u ? 8 : 4);
    const CUtensorMap *mw = nullptr, *mx = nullptr;
    int rc = get_map(g_maps_w, &mw, B, N, K, BR);
    if (rc) return rc;
    rc = get_map(g_maps_x, &mx, A, M, K, d.tok);
    if (rc) return rc;
    if (d.tok == 16) return launch_tok<16>(*mw, *mx, p, grouped, u, d.grid, aux, stream);
    if (d.tok == 32) return launch_tok<32>(*mw, *mx, p, grouped, u, d.grid, aux, stream);
    return launch_tok<64>(*mw, *mx, p, grouped, u, d.grid, aux, stream);
}

int gemm_decode_tc_status(int *out4) {
    return cuda_status(cudaMemcpyFromSymbol(out4, g_status, sizeof(int) * 4), "status read");
}
// Reads and clears the wait-time counters (8 x unsigned long long, nanoseconds summed over CTAs).
int gemm_decode_tc_wait_profile(unsigned long long *out8) {
    cudaError_t e = cudaMemcpyFromSymbol(out8, g_wait_ns, sizeof(unsigned long long) * 8);
    if (e != cudaSuccess) return cuda_status(e, "wait profile read");
    unsigned long long z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_wait_ns, z, sizeof(z)), "wait profile clear");
}
int gemm_decode_tc_status_clear() {
    int z[4] = {0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_status, z, sizeof(z)), "status clear");
}

}  // namespace flh
