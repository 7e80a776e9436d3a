// Per-token quantiser with the HIGH part of the full-width Hadamard transform on the 5th-generation tensor cores.
//
// A row of K = P * 64 values is a P x 64 matrix X[p][j] (j contiguous).  The transform of matmul_hadU
// (flh/functional/hadamard.py:92-113), (hadK (x) H_{2^a} (x) H_64) x, factors into two commuting steps:
//   1. over p:  T[p'][j] = sum_p G[p'][p] X[p][j],  G = hadK (x) H_{2^a}  (a P x P matrix of +-1, P = kfac * 2^a)
//   2. over j:  six butterfly bits on the 64 values of each p'.
// Step 1 runs FIRST, on the raw 16-bit inputs: every product with +-1 is exact, so tcgen05.mma (kind::f16) with
// binary32 accumulation in TMEM needs no operand splitting — A = G (K-major, built once per CTA in shared memory
// from the sign bits), B = the row itself exactly as it lies in global memory (TMA with the 128-byte swizzle, read as
// an N-major operand: j is the contiguous N dimension, p the contraction), D[p'][j] in TMEM with one p' per lane.
// Step 2 then needs no data movement at all: a thread reads its lane's 64 columns with one tcgen05.ld and runs the six
// bits in registers (packed binary32 pairs), takes part in the row's min/max, and turns its 64 consecutive outputs
// into 32 bytes of codes.  The CUDA cores do 6 of the 12+ butterfly bits instead of all of them.
//
// The sums of step 1 are accumulated by the tensor core in its own order, so the result is not bit-identical to the
// sequential butterflies (that order is hadamard = 2): same values up to binary32 rounding of the accumulation.  The
// order does not depend on the batch: every M takes this kernel.
//
// Shapes: P <= 64: two rows per MMA (A = diag(G, G), 128 x 128); 64 < P <= 128: one row per MMA (M = 128);
// 128 < P <= 256: one row on two MMAs (M = 256 as two tiles).  256 < P <= 512 (K = 28672, 32768): G = H_2 (x) G' with G' of
// order P / 2 <= 256; the row is read as its two halves X_0, X_1 of the top Sylvester bit (a 5-D TMA box picks every other
// block of chunks), and the accumulator tiles of out_0 = G' X_0 + G' X_1 and out_1 = G' X_0 - G' X_1 are filled by the same
// instructions with the negate-A bit of the instruction descriptor set for the one minus sign: four tiles per row, the
// operand in shared memory stays G'.  Roles of the persistent CTA: 16 epilogue warps (four
// groups of four, one group per 128-lane accumulator tile), one TMA thread, one MMA thread.  Rings: shared-memory stages
// (TMA -> MMA), 64-column TMEM slots (MMA -> epilogue).  All mbarrier waits are bounded; a wait that runs out sets a status word,
// the warps keep walking their loops without touching the tensor core so that every named barrier is still reached.
#include <string.h>
#include "tc_common.cuh"
#include "token_common.cuh"
#include "act_common.cuh"
#include "tc_quant_common.cuh"

namespace flh {
namespace {

constexpr int kEpiWarpsTc = 16;
constexpr int kThreadsTc = kEpiWarpsTc * 32 + 128;       // + one warpgroup: the TMA thread (warp 16) and up to three MMA issuer threads (warps 17-19)
constexpr int kSlots = 8;                                // 64-column accumulator slots in TMEM (512 columns)
constexpr int kMaxStages = 8;
__device__ int g_status_tc[4];
// Diagnostic (flh_b200_quant_token_wait_profile): nanoseconds summed over CTAs — [0] CTA lifetime, [1] TMA thread waiting for a free
// stage, [2] MMA thread waiting for TMA data, [3] MMA thread waiting for a free accumulator slot, [4] epilogue warps waiting
// for a finished accumulator (summed over the 16 warps), [5] set-up (A operand, barriers, TMEM allocation).
__device__ unsigned long long g_wait_tc[8];

struct TcQuantParams {
    long M;
    int K, P;                  // K = P * 64
    int kfac, B;               // P = kfac * B, B a power of two
    int words;                 // 32-bit words per row of the sign-bit table
    const uint32_t *sign_bits; // kfac rows of bits (1 = negative), or null for kfac = 1
    int R, T;                  // rows per 128-lane accumulator block (2 when P <= 64), tiles of G per row (2 when PG > 128)
    int H;                     // halves of the top Sylvester bit handled by signed accumulation (2 when P > 256, else 1)
    int PG, BG;                // order of the operand G (P / H) and its Sylvester part (B / H)
    int NB;                    // 64-column blocks per MMA: N = 64 * NB, i.e. R * NB rows per unit
    int CK, nchunks;           // a stage holds CK rows of the contraction (the K dimension of the MMAs) of every row of the unit;
                               // a unit is nchunks stages (1 when R = 2)
    int Kdim, Mtot;            // contraction length of the MMAs (multiple of 16), rows of A (128 or 256)
    int a_bytes, stage_bytes, stages;
    int bf16;
    int dbg;                   // PROFILE only: bit 0 = the epilogue only loads and releases its accumulators (how fast TMA + MMA run alone)
    const uint8_t *gu;         // FUSE: merged gate/up matrix [M][2K] (gate = the first K columns), row stride gu_ld_bytes
    long gu_ld_bytes;
    float clip, c;
    uint8_t *q;
    __half *scale, *zero;
};

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&v)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]),
          "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]),
          "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]),
          "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]),
          "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
        : "r"(taddr) : "memory");
}

// six butterfly bits over 64 values held as 32 packed pairs (pair k = elements 2k, 2k + 1); bit 0 inside the pairs
__device__ __forceinline__ void bfly6_pairs(uint64_t (&p)[32]) {
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        float a, b;
        unpack2(p[k], a, b);
        p[k] = pack2(__fadd_rn(a, b), __fsub_rn(a, b));
    }
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
}

// PROFILE: time every wait with %globaltimer and add the sums to g_wait_tc (flh_b200_quant_token_wait_profile).
// HALVES: the two-half form for 256 < P <= 512 (below).
// FUSE: the rows are not read by TMA but MADE by the epilogue warps — SiLU(gate) * up of the merged gate/up GEMM output
// (act_common.cuh), written into the stages in the layout TMA would have produced; the unit after the one whose
// accumulators are being turned into codes is made first, so the tensor core always has a unit to work on.
template <bool PROFILE, bool FUSE, bool HALVES>
__global__ void __launch_bounds__(kThreadsTc, 1) quant_token_tc_kernel(const __grid_constant__ CUtensorMap map_x, const TcQuantParams p) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_dyn + (base - raw);
    const int S = p.stages, T = p.T, R = p.R, NB = p.NB;
    constexpr int H = HALVES ? 2 : 1;                    // halves of the top Sylvester bit (HALVES: P > 256)
    const int TT = T * H;                                // accumulator tiles per row
    const int BPU = TT * NB;                             // 128-lane x 64-column accumulator blocks per unit (1, 2 or 4)
    const int NU = kSlots / BPU;                         // units whose accumulators fit TMEM
    const int NT = 4 / BPU;                              // epilogue teams (each takes every NT-th unit)
    const uint32_t a_base = base, st_base = base + p.a_bytes;
    const int aux = p.a_bytes + S * p.stage_bytes;
    uint32_t *red = reinterpret_cast<uint32_t *>(sm + aux);   // [2][8 rows in flight][8 warps of a row][|min| bits, max bits]
    const uint32_t bars = base + aux + 1024;
    auto stage_full = [&](int s) { return bars + 8u * s; };
    auto stage_empty = [&](int s) { return bars + 8u * (kMaxStages + s); };
    auto slot_full = [&](int u) { return bars + 8u * (2 * kMaxStages + u); };
    auto slot_empty = [&](int u) { return bars + 8u * (2 * kMaxStages + kSlots + u); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + aux + 1024 + 8 * (2 * kMaxStages + 2 * kSlots));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t t_start = PROFILE ? gtimer() : 0;

    // ---- one-time set-up: A = G (or diag(G, G)) as a K-major operand with the 128-byte swizzle ----
    build_sign_operand(sm, reinterpret_cast<uint32_t *>(sm + aux + 2048), p.sign_bits, p.kfac, p.words, p.PG, p.BG, R, p.Kdim, p.Mtot,
                       p.bf16 != 0, tid, kThreadsTc);
    if (tid == 0) {
        // every accumulator tile of a row has its own MMA issuer thread: all of them free a stage, all of them fill a slot
        for (int s = 0; s < kMaxStages; ++s) { mbar_init(stage_full(s), FUSE ? kEpiWarpsTc : 1); mbar_init(stage_empty(s), TT); }
        for (int u = 0; u < kSlots; ++u) { mbar_init(slot_full(u), TT); mbar_init(slot_empty(u), 4 * BPU); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    if (warp == kEpiWarpsTc + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const long n_units = (p.M + R * NB - 1) / (R * NB);
    if (PROFILE && tid == 0) atomicAdd(&g_wait_tc[5], gtimer() - t_start);
    // a bounded wait, timed as a whole when profiling (try_wait may itself block for a while before it returns)
    auto wait = [&](uint32_t bar, uint32_t parity, int code, unsigned long long &acc) {
        const uint64_t ta = PROFILE ? gtimer() : 0;
        const bool got = mbar_wait_status(g_status_tc, bar, parity, abort_flag, code);
        if (PROFILE) acc += gtimer() - ta;
        return got;
    };

    if (warp >= kEpiWarpsTc) {
        if constexpr (!HALVES) {
            if (!FUSE && warp == kEpiWarpsTc && lane == 0) {
                // ============================================================= TMA producer
                long it = 0;                                 // stages issued so far
                unsigned long long w1 = 0;
                bool ok = true;
                for (long unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                    for (int c = 0; c < p.nchunks; ++c, ++it) {
                        const int s = (int)(it % S);
                        if (!wait(stage_empty(s), (uint32_t)(((it / S) & 1) ^ 1), 31, w1)) { ok = false; break; }
                        mbar_expect_tx(stage_full(s), (uint32_t)p.stage_bytes);
                        tma_load_3d(st_base + s * p.stage_bytes, &map_x, 0, c * p.CK, (int)(unit * R * NB), stage_full(s));
                    }
                }
                if (PROFILE) atomicAdd(&g_wait_tc[1], w1);
            } else if (warp > kEpiWarpsTc && warp - kEpiWarpsTc - 1 < T && lane == 0) {
                // ============================================================= MMA issuers
                // One tcgen05.mma costs its issuing thread a few hundred cycles whatever its size, and for P > 128 that thread
                // is the kernel's limit: the two accumulator tiles of a row are independent, so each gets its own issuer.
                const int ti = warp - kEpiWarpsTc - 1;
                const uint32_t fmt = p.bf16 ? 1u : 0u;
                // D binary32, A / B format, B N-major (bit 16), N = 64 NB, M = 128
                const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)((64 * NB) >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                const uint32_t nblk = (uint32_t)p.stage_bytes / (uint32_t)NB;          // bytes between the 64-column blocks of B (one block = R rows)
                const int ksteps = (R == 2 ? p.Kdim : p.CK) >> 4;          // K steps of 16 per stage
                long it = 0, sc = 0;                                       // units, stages consumed so far
                unsigned long long w2 = 0, w3 = 0;
                bool ok = true;
                for (long unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ++it) {
                    const int u = (int)(it % NU);
                    if (!wait(slot_empty(u), (uint32_t)(((it / NU) & 1) ^ 1), 33, w3)) break;
                    for (int c = 0; c < p.nchunks; ++c, ++sc) {
                        const int s = (int)(sc % S);
                        if (!wait(stage_full(s), (uint32_t)((sc / S) & 1), 32, w2)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t bst = st_base + s * p.stage_bytes;
                        {
                            const int t = ti;
                            const uint32_t d = tmem + (uint32_t)((u * BPU + t * NB) * 64);
                            for (int ks = 0; ks < ksteps; ++ks) {
                                const int kg = c * ksteps + ks;            // K step within the whole contraction
                                // A: K-major, 8-row groups 1024 bytes apart; K step of 16 = 32 bytes inside the 128-byte row, next atom after 4
                                const uint64_t ad = umma_desc_tc(a_base + ((kg >> 2) * (p.Mtot >> 3) + t * 16) * 1024 + (kg & 3) * 32, 16, 1024);
                                // B: N-major (64 values of j = one 128-byte row per p), 8-row groups 1024 bytes apart (SBO), 16 rows per
                                // K step; the NB blocks of 64 columns (different token rows) lie nblk bytes apart (LBO)
                                const uint64_t bd = umma_desc_tc(bst + ks * 2048, nblk, 1024);
                                const uint32_t acc = kg ? 1u : 0u;
                                asm volatile("{\n\t.reg .pred pp;\n\tsetp.ne.b32 pp, %4, 0;\n\t"
                                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pp;\n\t}"
                                             ::"r"(d), "l"(ad), "l"(bd), "r"(idesc), "r"(acc) : "memory");
                            }
                        }
                        tc_commit(stage_empty(s));
                    }
                    if (ok) tc_commit(slot_full(u));
                }
                if (PROFILE && ti == 0) { atomicAdd(&g_wait_tc[2], w2); atomicAdd(&g_wait_tc[3], w3); }
            }
        } else {
            // One tcgen05.mma costs its issuing thread a few hundred cycles whatever its size, and for P > 128 that is the kernel's
            // limit: the accumulator tiles of a row are independent, so each has its own issuer thread — warps 17, 18, 19 for tiles
            // 0, 1, 2, and the TMA thread of warp 16 for a fourth tile (two halves x two tiles of G).
            const uint32_t fmt = p.bf16 ? 1u : 0u;
            // D binary32, A / B format, B N-major (bit 16), N = 64 NB, M = 128; bit 13 negates A (the minus sign of out_1 = G' X_0 - G' X_1)
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)((64 * NB) >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            const uint32_t nblk = (uint32_t)p.stage_bytes / (uint32_t)NB;          // bytes between the 64-column blocks of B (one block = R rows)
            const int ksteps = (R == 2 ? p.Kdim : p.CK) >> 4;          // K steps of 16 per stage
            const int SPU = H * p.nchunks;                             // stages per unit: the chunks of half 0, then of half 1
            // the K steps of stage s (chunk c of half h) into accumulator tile ti of TMEM slot u
            auto mma_stage = [&](int ti, int u, int h, int c, int s) {
                const int t = HALVES ? ti % T : ti, hp = HALVES ? ti / T : 0;                     // tile of G, half h' of the output
                const uint32_t bst = st_base + s * p.stage_bytes;
                const uint32_t d = tmem + (uint32_t)((u * BPU + ti * NB) * 64);
                const uint32_t idv = (hp == 1 && h == 1) ? (idesc | (1u << 13)) : idesc;
                for (int ks = 0; ks < ksteps; ++ks) {
                    const int kg = c * ksteps + ks;                    // K step within the whole contraction
                    // A: K-major, 8-row groups 1024 bytes apart; K step of 16 = 32 bytes inside the 128-byte row, next atom after 4
                    const uint64_t ad = umma_desc_tc(a_base + ((kg >> 2) * (p.Mtot >> 3) + t * 16) * 1024 + (kg & 3) * 32, 16, 1024);
                    // B: N-major (64 values of j = one 128-byte row per p), 8-row groups 1024 bytes apart (SBO), 16 rows per
                    // K step; the NB blocks of 64 columns (different token rows) lie nblk bytes apart (LBO)
                    const uint64_t bd = umma_desc_tc(bst + ks * 2048, nblk, 1024);
                    const uint32_t acc = (kg | h) ? 1u : 0u;
                    asm volatile("{\n\t.reg .pred pp;\n\tsetp.ne.b32 pp, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pp;\n\t}"
                                 ::"r"(d), "l"(ad), "l"(bd), "r"(idv), "r"(acc) : "memory");
                }
            };
            // stage number `ld` of this CTA (unit ld / SPU of its list): the TMA load
            auto issue_load = [&](long ld) {
                const long iu = ld / SPU;
                const int hc = (int)(ld - iu * SPU), h = hc / p.nchunks, c = hc - h * p.nchunks;
                const long unit = blockIdx.x + iu * gridDim.x;
                const int s = (int)(ld % S);
                mbar_expect_tx(stage_full(s), (uint32_t)p.stage_bytes);
                if (H == 1) {
                    tma_load_3d(st_base + s * p.stage_bytes, &map_x, 0, c * p.CK, (int)(unit * R * NB), stage_full(s));
                } else {
                    // chunk rows [c CK, (c + 1) CK) of half h, in the order of G': (a, b') with b' < BG
                    const int r0 = c * p.CK;
                    tma_load_5d(st_base + s * p.stage_bytes, &map_x, 0, p.kfac > 1 ? 0 : r0, h, p.kfac > 1 ? r0 / p.BG : 0,
                                (int)(unit * R * NB), stage_full(s));
                }
            };
            const long my_units = (long)blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
            if (!FUSE && warp == kEpiWarpsTc && lane == 0 && TT < 4) {
                // ============================================================= TMA producer
                unsigned long long w1 = 0;
                for (long ld = 0; ld < my_units * SPU; ++ld) {
                    if (!wait(stage_empty((int)(ld % S)), (uint32_t)(((ld / S) & 1) ^ 1), 31, w1)) break;
                    issue_load(ld);
                }
                if (PROFILE) atomicAdd(&g_wait_tc[1], w1);
            } else if (!FUSE && warp == kEpiWarpsTc && lane == 0) {
                // ============================================================= TMA producer that also issues the fourth tile's MMAs:
                // before it waits for a stage it makes sure that stage is on its way, then issues as many further loads as free
                // stages allow without waiting
                unsigned long long w1 = 0, w2 = 0, w3 = 0;
                const long total = my_units * SPU;
                long loads = 0;
                bool ok = true;
                for (long it = 0; it < my_units && ok; ++it) {
                    const int u = (int)(it % NU);
                    if (!wait(slot_empty(u), (uint32_t)(((it / NU) & 1) ^ 1), 33, w3)) break;
                    for (int hc = 0; hc < SPU; ++hc) {
                        const long sc = it * SPU + hc;
                        while (loads <= sc && ok) {
                            ok = wait(stage_empty((int)(loads % S)), (uint32_t)(((loads / S) & 1) ^ 1), 31, w1);
                            if (ok) issue_load(loads++);
                        }
                        if (!ok) break;
                        while (loads < total && loads < sc + S && mbar_try(stage_empty((int)(loads % S)), (uint32_t)(((loads / S) & 1) ^ 1))) issue_load(loads++);
                        const int s = (int)(sc % S);
                        if (!wait(stage_full(s), (uint32_t)((sc / S) & 1), 32, w2)) { ok = false; break; }
                        tc_fence_after();
                        mma_stage(3, u, hc / p.nchunks, hc % p.nchunks, s);
                        tc_commit(stage_empty(s));
                    }
                    if (ok) tc_commit(slot_full(u));
                }
                if (PROFILE) atomicAdd(&g_wait_tc[1], w1);
            } else if (warp > kEpiWarpsTc && warp - kEpiWarpsTc - 1 < TT && lane == 0) {
                // ============================================================= MMA issuers
                const int ti = warp - kEpiWarpsTc - 1;
                unsigned long long w2 = 0, w3 = 0;
                bool ok = true;
                for (long it = 0; it < my_units && ok; ++it) {
                    const int u = (int)(it % NU);
                    if (!wait(slot_empty(u), (uint32_t)(((it / NU) & 1) ^ 1), 33, w3)) break;
                    for (int hc = 0; hc < SPU; ++hc) {
                        const long sc = it * SPU + hc;
                        const int s = (int)(sc % S);
                        if (!wait(stage_full(s), (uint32_t)((sc / S) & 1), 32, w2)) { ok = false; break; }
                        tc_fence_after();
                        mma_stage(ti, u, hc / p.nchunks, hc % p.nchunks, s);
                        tc_commit(stage_empty(s));
                    }
                    if (ok) tc_commit(slot_full(u));
                }
                if (PROFILE && ti == 0) { atomicAdd(&g_wait_tc[2], w2); atomicAdd(&g_wait_tc[3], w3); }
            }
        }
    } else {
        // ================================================================= epilogue
        const int g = warp >> 2, quarter = warp & 3;
        const int team = g / BPU, b = g - team * BPU;                // this group's block of the unit
        const int tile = b / NB, nb = b - tile * NB;                 // accumulator tile of the row (h' T + tile of G), 64-column block of the MMA
        const int wpr = R == 2 ? 2 : 4 * TT;                         // warps that share one row
        const int m = quarter * 32 + lane;                           // TMEM lane = row of the accumulator tile
        const int riu = R == 2 ? nb * 2 + (m >> 6) : nb;             // row of the unit
        const int pg = R == 2 ? (m & 63) : (HALVES ? tile % T : tile) * 128 + m;     // row of G this thread holds
        // its p' in the full transform: with two halves the top Sylvester bit h' sits between the factor index and the rest
        const int pp = !HALVES ? pg : (pg / p.BG) * (2 * p.BG) + (tile / T) * p.BG + (pg % p.BG);
        const int rslot = R == 2 ? (quarter & 1) : tile * 4 + quarter;   // this warp among the warps of its row
        const int rt = team * R * NB + riu;                          // row in flight: named barrier 1 + rt (at most 8)
        const bool live = pg < p.PG;
        const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * 64);
        uint8_t *qbase = p.q + pp * 32;
        const long qld = (long)(p.K >> 1);
        bool ok = true;
        int n = 0;
        unsigned long long w4 = 0;
        // FUSE (one team of all sixteen warps, NT = 1): make the stages of unit number `iu` of this CTA
        auto produce = [&](long iu) {
            const long unit = blockIdx.x + iu * gridDim.x;
            const int rows = R * NB, rowbytes_k = p.CK * 128;        // token rows of a stage, bytes of one token row in a stage
            const long F2 = (long)p.K * 2;                           // bytes from a gate element to its up element
            for (int c = 0; c < p.nchunks; ++c) {
                const long sc = iu * p.nchunks + c;
                const int s = (int)(sc % S);
                unsigned long long w0 = 0;
                ok = __all_sync(0xffffffffu, ok && wait(stage_empty(s), (uint32_t)(((sc / S) & 1) ^ 1), 35, w0));
                uint8_t *st = sm + p.a_bytes + s * p.stage_bytes;
                if (ok) {
                    for (int xr = 0; xr < rows; ++xr) {
                        const long row = unit * rows + xr;
                        const uint8_t *grow = p.gu + row * p.gu_ld_bytes;
                        // 16-byte pieces of this token row's part of the stage: piece j = (contraction row j / 8, chunk j % 8)
                        for (int j0 = tid; j0 < p.CK * 8; j0 += 4 * kEpiWarpsTc * 32) {
                            uint4 g[4], u[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int j = j0 + q * kEpiWarpsTc * 32;
                                const int pl = j >> 3, c16 = j & 7;
                                const int prow = (R == 2 ? 0 : c * p.CK) + pl;
                                g[q] = make_uint4(0u, 0u, 0u, 0u); u[q] = g[q];
                                if (j < p.CK * 8 && prow < p.P && row < p.M) {
                                    const uint8_t *src = grow + ((long)prow * 64 + c16 * 8) * 2;
                                    g[q] = ldg_nc_v4(src);
                                    u[q] = ldg_nc_v4(src + F2);
                                }
                            }
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int j = j0 + q * kEpiWarpsTc * 32;
                                if (j < p.CK * 8) {
                                    const int pl = j >> 3, c16 = j & 7;
                                    const int rs = xr * p.CK + pl;           // 128-byte row of the stage
                                    const uint4 a = p.bf16 ? silu_mul_8<true>(g[q], u[q]) : silu_mul_8<false>(g[q], u[q]);
                                    *reinterpret_cast<uint4 *>(st + (long)xr * rowbytes_k + pl * 128 + ((c16 ^ (rs & 7)) << 4)) = a;
                                }
                            }
                        }
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(stage_full(s));
            }
        };
        if (FUSE && (long)blockIdx.x < n_units) produce(0);
        const int nu_mask = NU - 1, nu_log = 31 - __clz(NU);          // NU is 8, 4 or 2
        const int units_i = (int)n_units, stride = (int)gridDim.x, rows_pu = R * NB;
        for (int it = team;; it += NT, ++n) {
            const int unit = (int)blockIdx.x + it * stride;
            if (unit >= units_i) break;
            if (FUSE && unit + stride < units_i) produce(it + 1);
            const int u = it & nu_mask;
            ok = __all_sync(0xffffffffu, ok && wait(slot_full(u), (uint32_t)((it >> nu_log) & 1), 34, w4));
            uint64_t v[32];
            if (PROFILE && (p.dbg & 2)) {                            // experiment: no TMEM load either
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(slot_empty(u));
                continue;
            }
            if (ok) {
                tc_fence_after();
                uint32_t rawv[64];
                tmem_ld64(tbase + (uint32_t)(u * BPU * 64), rawv);
                tc_wait_ld();
#pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = ((uint64_t)rawv[2 * k + 1] << 32) | rawv[2 * k];
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = 0ull;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_empty(u));               // the accumulator is in registers: the slot is free
            if (PROFILE && (p.dbg & 1)) {
                if (v[0] == 0x123456789abcdefull) p.q[0] = 1;         // keep the load alive
                continue;
            }
            bfly6_pairs(v);
            // ---- row minimum (<= 0) and maximum (>= 0): the bit pattern of a non-negative binary32 orders like an
            //      unsigned integer, so |min| and max go through one redux.sync each ----
            float mn0 = 0.0f, mn1 = 0.0f, mx0 = 0.0f, mx1 = 0.0f;
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
                float x0, x1, x2, x3;
                unpack2(v[k], x0, x1);
                unpack2(v[k + 1], x2, x3);
                mn0 = min3(mn0, x0, x1); mx0 = max3(mx0, x0, x1);
                mn1 = min3(mn1, x2, x3); mx1 = max3(mx1, x2, x3);
            }
            const uint32_t wmin = warp_max_u32(__float_as_uint(fminf(mn0, mn1)) & 0x7fffffffu);
            const uint32_t wmax = warp_max_u32(__float_as_uint(fmaxf(mx0, mx1)) & 0x7fffffffu);
            uint32_t *rd_ = red + (n & 1) * 128 + rt * (HALVES && wpr > 8 ? 32 : 16);    // sixteen warps per row only with one row in flight
            if (lane == 0) *reinterpret_cast<uint2 *>(rd_ + rslot * 2) = make_uint2(wmin, wmax);
            bar_sync_named(1 + rt, 32 * wpr);
            uint32_t umin, umax;
            {
                const uint4 e0 = *reinterpret_cast<const uint4 *>(rd_);
                umin = max(e0.x, e0.z); umax = max(e0.y, e0.w);
                if (wpr > 2) {
                    const uint4 e1 = *reinterpret_cast<const uint4 *>(rd_ + 4);
                    umin = max(umin, max(e1.x, e1.z)); umax = max(umax, max(e1.y, e1.w));
                }
                if (wpr > 4) {
                    const uint4 e2 = *reinterpret_cast<const uint4 *>(rd_ + 8), e3 = *reinterpret_cast<const uint4 *>(rd_ + 12);
                    umin = max(umin, max(max(e2.x, e2.z), max(e3.x, e3.z))); umax = max(umax, max(max(e2.y, e2.w), max(e3.y, e3.w)));
                }
                if (HALVES && wpr > 8) {
#pragma unroll
                    for (int e = 16; e < 32; e += 4) {
                        const uint4 ee = *reinterpret_cast<const uint4 *>(rd_ + e);
                        umin = max(umin, max(ee.x, ee.z)); umax = max(umax, max(ee.y, ee.w));
                    }
                }
            }
            const TokenRowParams rp = token_row_params(__uint_as_float(umin | 0x80000000u), __uint_as_float(umax), p.clip, p.c);
            const long row = (long)unit * rows_pu + riu;
            if (ok && row < p.M) {
                if (pp == 0) { p.scale[row] = rp.scale; p.zero[row] = __float2half_rn(rp.zero); }
                if (live) {
                    // y = fma(x, rd, M + zero) = M + code with M = 1.5 * 2^23 (the sum is rounded to an integer, ties to even on the
                    // code); the codes of four neighbours (c0, c1 | c2, c3 as two packed pairs) are joined in binary32, every value an
                    // exact integer: (c2, c3) = y23 - M;  u = (c2, c3) * 256 + y01 = M + (c0 + 256 c2, c1 + 256 c3);
                    // w = (u.hi - M) * 16 + u.lo = M + c0 + 16 c1 + 256 c2 + 4096 c3: the low 16 bits of w's pattern are the two bytes
                    const float Mf = 12582912.0f;
                    const float Mzf = __fadd_rn(Mf, rp.zero);
                    const uint64_t rd2 = pack2(rp.rd, rp.rd), Mz2 = pack2(Mzf, Mzf), nM2 = pack2(-Mf, -Mf), c256 = pack2(256.0f, 256.0f);
#pragma unroll
                    for (int k = 0; k < 32; ++k) v[k] = fma2(v[k], rd2, Mz2);
                    if (rp.clamp) {
#pragma unroll
                        for (int k = 0; k < 32; ++k) {
                            float x0, x1;
                            unpack2(v[k], x0, x1);
                            v[k] = pack2(fmaxf(fminf(x0, Mf + 15.0f), Mf), fmaxf(fminf(x1, Mf + 15.0f), Mf));
                        }
                    }
                    uint32_t o[8];
#pragma unroll
                    for (int wd = 0; wd < 8; ++wd) {
                        uint32_t hw[2];
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int k = wd * 4 + hh * 2;
                            float lo, hi;
                            unpack2(fma2(add2(v[k + 1], nM2), c256, v[k]), lo, hi);
                            hw[hh] = __float_as_uint(__fmaf_rn(__fsub_rn(hi, Mf), 16.0f, lo));
                        }
                        o[wd] = __byte_perm(hw[0], hw[1], 0x5410);
                    }
                    uint4 *dst = reinterpret_cast<uint4 *>(qbase + row * qld);
                    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
        }
        if (PROFILE && lane == 0) atomicAdd(&g_wait_tc[4], w4);
    }

    tc_fence_before();
    __syncthreads();
    if (PROFILE && tid == 0) atomicAdd(&g_wait_tc[0], gtimer() - t_start);
    if (warp == kEpiWarpsTc + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

typedef CUresult (*EncodeTiledFnTc)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

EncodeTiledFnTc encode_fn_tc() {
    static EncodeTiledFnTc fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFnTc>(ptr);
    }
    return fn;
}

// The tensor map of an input is a pure function of (pointer, M, P, row stride, box): the last few are remembered per
// host thread, so that a serving loop that re-uses its buffers encodes each map once.
struct MapKey {
    const void *x; long M, ld; int P, boxP, R;          // boxP: contraction rows per TMA box, R: token rows per box
    int H, BG, kfac;                                    // two-half mode: 5-D map over (j, b', h, a, row)
    bool operator==(const MapKey &o) const {
        return x == o.x && M == o.M && ld == o.ld && P == o.P && boxP == o.boxP && R == o.R && H == o.H && BG == o.BG && kfac == o.kfac;
    }
};
struct MapCache { MapKey key[8]; CUtensorMap map[8]; int used = 0, next = 0; };

int get_map(const MapKey &k, CUtensorMap *out) {
    static thread_local MapCache cache;
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == k) { *out = cache.map[i]; return 0; }
    EncodeTiledFnTc fn = encode_fn_tc();
    if (!fn) return fail(FLH_B200_EUNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    // x as [M][P][64] 16-bit values: dimension 0 = j (contiguous), 1 = p (128 bytes apart), 2 = row (ld * 2 bytes apart);
    // chunks past P and rows past M read as zero
    cuuint64_t dims[3] = {64u, (cuuint64_t)k.P, (cuuint64_t)k.M};
    cuuint64_t strides[2] = {128u, (cuuint64_t)k.ld * 2u};
    cuuint32_t box[3] = {64u, (cuuint32_t)k.boxP, (cuuint32_t)k.R};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUtensorMap m;
    CUresult r;
    if (k.H == 1) {
        r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(k.x), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        // chunk index p = a * (2 BG) + h * BG + b': dimension 1 = b' (128 bytes apart), 2 = h (BG chunks apart), 3 = a (2 BG chunks
        // apart), 4 = row; a box takes boxP chunks of one half in (a, b') order — whole a-blocks, or part of the only one
        cuuint64_t d5[5] = {64u, (cuuint64_t)k.BG, 2u, (cuuint64_t)k.kfac, (cuuint64_t)k.M};
        cuuint64_t s5[4] = {128u, (cuuint64_t)k.BG * 128u, (cuuint64_t)k.BG * 256u, (cuuint64_t)k.ld * 2u};
        cuuint32_t b5[5] = {64u, (cuuint32_t)(k.kfac > 1 ? k.BG : k.boxP), 1u, (cuuint32_t)(k.kfac > 1 ? k.boxP / k.BG : 1), (cuuint32_t)k.R};
        cuuint32_t e5[5] = {1u, 1u, 1u, 1u, 1u};
        r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, const_cast<void *>(k.x), d5, s5, b5, e5,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(FLH_B200_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    const int slot = cache.used < 8 ? cache.used++ : (cache.next++ & 7);
    cache.key[slot] = k;
    cache.map[slot] = m;
    *out = m;
    return 0;
}

}  // namespace

// Shapes this kernel takes: K = P * 64 with P = kfac * 2^a <= 512 (above 256 the Sylvester part must be at least 2: the top
// bit is then handled by signed accumulation of the two halves of the row).
bool quant_token_tc_takes(long K, int kfac) {
    if (K % 64 != 0 || kfac < 1) return false;
    const long P = K / 64;
    if (P > 512 || P % kfac != 0) return false;
    const long B = P / kfac;
    if ((B & (B - 1)) != 0) return false;
    return P <= 256 || (B >= 2 && kfac <= 256);
}

// Full-width transform + per-token asymmetric int4 for K = P * 64, P = kfac * 2^a <= 256.  x: the rows to quantise, or
// null with gu = the merged gate/up matrix [M][2K] whose SiLU(gate) * up is to be quantised (row stride ld either way).
// Returns -1000 when the shape (or an alignment) is not one this kernel takes; the caller then uses the CUDA-core kernels.
static int launch_tc(const void *x, const void *gu, int in_dtype, long M, long K, long ld, int kfac, const uint32_t *sign_bits,
                     float clip, uint8_t *q, void *scale, void *zero, cudaStream_t stream) {
    if (M < 1 || !quant_token_tc_takes(K, kfac)) return -1000;
    const int P = (int)(K / 64);
    const int B = P / kfac;
    const void *in = gu ? gu : x;
    if ((reinterpret_cast<uintptr_t>(q) & 15) != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || ld % 8 != 0) return -1000;
    if (M > 0x7fffffffL / 2) return -1000;                       // TMA coordinates are 32-bit
    TcQuantParams p;
    p.M = M; p.K = (int)K; p.P = P; p.kfac = kfac; p.B = B;
    p.words = (kfac + 31) / 32;
    p.sign_bits = kfac > 1 ? sign_bits : nullptr;
    p.H = P > 256 ? 2 : 1;
    if (p.H == 2 && gu) return -1000;                            // the fused form makes whole rows: not written for two halves
    p.PG = P / p.H; p.BG = B / p.H;
    p.R = p.PG <= 64 ? 2 : 1;
    p.T = p.PG > 128 ? 2 : 1;
    const int boxP = p.R == 2 ? 64 : (p.PG + 15) / 16 * 16;
    p.Kdim = p.R == 2 ? 128 : boxP;
    p.Mtot = 128 * p.T;
    p.a_bytes = ((p.Kdim + 63) / 64) * p.Mtot * 128;
    const int budget = 227 * 1024 - 7168 - 1024 - p.a_bytes;     // aux (reductions, barriers, sign words) + alignment slack
    // MMAs as wide as TMEM allows (N = 64 NB columns: NB rows, or row pairs, per instruction — an MMA costs about the same
    // for any N); small batches take narrower ones so that the rows spread over more SMs.  A stage holds CK of the Kdim
    // contraction rows of every row of the unit: the largest divisor of Kdim (in steps of 16) of which two stages fit
    // beside A (large stages keep more bytes in flight per barrier round trip than many small ones).
    int NB = 4 / (p.T * p.H);
    if (NB < 1) return -1000;
    while (!gu && NB > 1 && (M + (long)p.R * NB - 1) / ((long)p.R * NB) < kNumSMs) NB >>= 1;     // (the fused form works as one team)
    { const char *e = getenv("FLH_B200_TC_NB"); if (e && !gu) { const int v = atoi(e); if (v == 1 || v == 2 || v == 4) NB = v <= 4 / (p.T * p.H) ? v : NB; } }   // tuning aid
    int CK = p.R == 2 ? 64 : 16;
    if (p.R == 1) {
        for (int c = p.Kdim; c >= 16; c -= 16) {
            if (p.Kdim % c != 0 || 2 * NB * c * 128 > budget) continue;
            // two halves: a TMA box is whole blocks of BG chunks (or a part of the only block) and at most 256 of anything
            if (p.H == 2 && (kfac > 1 ? (c % p.BG != 0 || c / p.BG > 256) : (p.BG % c != 0 || c > 256))) continue;
            CK = c;
            break;
        }
        if (p.H == 2 && (kfac > 1 ? CK % p.BG != 0 : p.BG % CK != 0)) return -1000;
    }
    p.NB = NB;
    p.CK = CK;
    p.nchunks = p.R == 2 ? 1 : p.Kdim / CK;
    p.stage_bytes = p.R * NB * CK * 128;
    int stages = budget / p.stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return -1000;
    p.stages = stages;
    p.bf16 = in_dtype == FLH_B200_BF16;
    p.clip = clip;
    p.c = sqrtf((float)K);
    p.q = q;
    p.scale = static_cast<__half *>(scale);
    p.zero = static_cast<__half *>(zero);
    p.gu = static_cast<const uint8_t *>(gu);
    p.gu_ld_bytes = ld * 2;
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    if (!gu) {
        MapKey key{x, M, ld, P, CK, p.R * NB, p.H, p.BG, kfac};
        const int rc = get_map(key, &map);
        if (rc) return rc;
    }
    const int smem = p.a_bytes + stages * p.stage_bytes + 7168 + 1024;
    // FLH_B200_TC_PROFILE=1 (read once): the variant that times its waits for flh_b200_quant_token_wait_profile
    static int profile = -1;
    if (profile < 0) { const char *e = getenv("FLH_B200_TC_PROFILE"); profile = e ? atoi(e) : 0; }
    p.dbg = profile > 1 ? profile >> 1 : 0;                      // FLH_B200_TC_PROFILE=3: profile + accumulators loaded and dropped
    using Kern = void (*)(const CUtensorMap, const TcQuantParams);
    const bool fuse = gu != nullptr;
    const Kern kern = p.H == 2 ? (profile ? quant_token_tc_kernel<true, false, true> : quant_token_tc_kernel<false, false, true>)
                      : fuse   ? (profile ? quant_token_tc_kernel<true, true, false> : quant_token_tc_kernel<false, true, false>)
                               : (profile ? quant_token_tc_kernel<true, false, false> : quant_token_tc_kernel<false, false, false>);
    static bool attr_done[3][64] = {};
    const int variant = p.H == 2 ? 2 : fuse ? 1 : 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
    if (dev < 0 || !attr_done[variant][dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return cuda_status(e, "quant_token_tc smem attribute");
        if (dev >= 0) attr_done[variant][dev] = true;
    }
    const long n_units = (M + (long)p.R * NB - 1) / ((long)p.R * NB);
    const long grid = n_units < kNumSMs ? n_units : kNumSMs;
    kern<<<(unsigned)grid, kThreadsTc, smem, stream>>>(map, p);
    return cuda_status(cudaGetLastError(), "quant_token_tc launch");
}

int launch_quant_token_tc(const void *x, int in_dtype, long M, long K, long ld, int kfac, const uint32_t *sign_bits,
                          float clip, uint8_t *q, void *scale, void *zero, cudaStream_t stream) {
    return launch_tc(x, nullptr, in_dtype, M, K, ld, kfac, sign_bits, clip, q, scale, zero, stream);
}

// SiLU(gate) * up of gu [M][2K] (row stride ld elements) -> full-width transform -> per-token asymmetric int4, one kernel.
int launch_silu_mul_quant_token_tc(const void *gu, int in_dtype, long M, long K, long ld, int kfac, const uint32_t *sign_bits,
                                   float clip, uint8_t *q, void *scale, void *zero, cudaStream_t stream) {
    return launch_tc(nullptr, gu, in_dtype, M, K, ld, kfac, sign_bits, clip, q, scale, zero, stream);
}

int quant_token_tc_wait_profile(unsigned long long *out8) {
    cudaError_t e = cudaMemcpyFromSymbol(out8, g_wait_tc, sizeof(unsigned long long) * 8);
    if (e != cudaSuccess) return cuda_status(e, "wait profile read");
    unsigned long long z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_wait_tc, z, sizeof(z)), "wait profile clear");
}

int quant_token_tc_status(int *out4) {
    return cuda_status(cudaMemcpyFromSymbol(out4, g_status_tc, sizeof(int) * 4), "status read");
}
int quant_token_tc_status_clear() {
    int z[4] = {0, 0, 0, 0};
    return cuda_status(cudaMemcpyToSymbol(g_status_tc, z, sizeof(z)), "status clear");
}

}  // namespace flh
