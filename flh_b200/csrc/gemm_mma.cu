// int4 x int4 GEMM with fused dequantisation on the legacy warp-level tensor path
// (mma.sync.m16n8k32 s8), two kernels:
//   * gemm_tile_kernel    128x128x128 CTA tiles, cp.async ring; any M.  Bring-up cross-check for
//                         the tcgen05 kernel and the "legacy mma.sync" line of the benchmark.
//   * gemm_stream_kernel  decode shapes (M <= 64): every CTA streams a 32- or 64-row slab of packed
//                         weights through an 8-deep cp.async ring; HBM-bound on the weight bytes.
//
// Both feed the tensor cores without unpacking to natural order.  A packed 32-bit word holds eight
// nibbles; (w << 4) & 0xF0F0F0F0 and w & 0xF0F0F0F0 are the even and the odd elements as int8
// values multiplied by 16 (the nibble sits in the byte's high half, so the byte's sign bit is the
// nibble's).  A and B are expanded by the same rule, hence element k of A always meets element k
// of B; the dot product comes out multiplied by 256 and is shifted back exactly.
#include "common.cuh"

namespace flh {
namespace {

struct GemmParams {
    const uint8_t *A, *B;
    const __half *a_scale, *a_zero, *b_scale, *bias;
    const int32_t *b_rowsum;
    void *D;
    int M, N, K;
    int ga_cols, gb_cols;   // scale columns: K / a_group, K / b_group
    int grouped;            // 1: dequantise every 128-K block; 0: one integer sum over all of K
    int out_bf16;
    int splits;             // split-K (streaming kernel): CTAs along K per row slab; 1 = none
    int *counters;          // split-K scratch: one arrival counter per row slab (zero between launches)
    float *partials;        // split-K scratch: [splits][8 * NT][N] partial sums (raw 32-bit words)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

template <bool A_UNSIGNED>
__device__ __forceinline__ void mma_i8(int32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
    if (A_UNSIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t even16(uint32_t w) { return (w << 4) & 0xF0F0F0F0u; }
__device__ __forceinline__ uint32_t odd16(uint32_t w) { return w & 0xF0F0F0F0u; }

__device__ __forceinline__ void store_pair(void *D, bool bf16, long off, float v0, float v1) {
    if (bf16) {
        *reinterpret_cast<__nv_bfloat162 *>(static_cast<__nv_bfloat16 *>(D) + off) = __floats2bfloat162_rn(v0, v1);
    } else {
        *reinterpret_cast<__half2 *>(static_cast<__half *>(D) + off) = __floats2half2_rn(v0, v1);
    }
}

// Scales, zero-points and weight row sums one thread needs for a 16x8 fragment in K-group g:
// rows (r0, r0 + 8), columns (c0, c0 + 1).
struct RowQ { float sa[2]; int za[2]; };
struct ColQ { float sb[2]; int rs[2]; };

__device__ __forceinline__ RowQ load_rowq(const GemmParams &p, int r0, int g, bool has_zero) {
    RowQ q;
    const int ga = p.ga_cols == 1 ? 0 : g;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = min(r0 + 8 * h, p.M - 1);
        q.sa[h] = __half2float(p.a_scale[(long)r * p.ga_cols + ga]);
        q.za[h] = has_zero ? (int)__half2float(p.a_zero[(long)r * p.ga_cols + ga]) : 0;
    }
    return q;
}
__device__ __forceinline__ ColQ load_colq(const GemmParams &p, int c0, int g, bool has_zero) {
    ColQ q;
    const int gb = p.gb_cols == 1 ? 0 : g;
    const int G = p.grouped ? p.K / 128 : 1;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        q.sb[j] = __half2float(p.b_scale[(long)(c0 + j) * p.gb_cols + gb]);
        q.rs[j] = has_zero ? p.b_rowsum[(long)(c0 + j) * G + g] : 0;
    }
    return q;
}
// c holds 256 * integer sum of the group; acc = fmaf(float(I), sa * sb, acc).
__device__ __forceinline__ void dequant_frag(const int32_t (&c)[4], float (&acc)[4], const RowQ &rq, const ColQ &cq) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int32_t I = (c[2 * h + j] >> 8) - rq.za[h] * cq.rs[j];
            acc[2 * h + j] = __fmaf_rn((float)I, __fmul_rn(rq.sa[h], cq.sb[j]), acc[2 * h + j]);
        }
}

// --------------------------------------------------------------------------------------------
// Tile kernel: 8 warps as 2 (M) x 4 (N); warp tile 64 x 32 = 4 x 4 mma tiles.
constexpr int TBM = 128, TBN = 128, TSTAGES = 4;
constexpr int TSTAGE_BYTES = (TBM + TBN) * 64;      // 128-K block = 64 packed bytes per row

template <bool A_UNSIGNED>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(const GemmParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp >> 2, wn = warp & 3;
    const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;
    const int KB = p.K / 128;
    const long ldk = p.K / 2;

    auto load_stage = [&](int stage, int kb) {
        uint8_t *sA = smem + stage * TSTAGE_BYTES, *sB = sA + TBM * 64;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int ch = tid + i * 256, row = ch >> 2, c = ch & 3;
            const int gr = m0 + row;
            const uint8_t *src = p.A + (long)(gr < p.M ? gr : p.M - 1) * ldk + kb * 64 + c * 16;
            cp_async16(smem_u32(sA + row * 64 + c * 16), src, gr < p.M ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int ch = tid + i * 256, row = ch >> 2, c = ch & 3;
            cp_async16(smem_u32(sB + row * 64 + c * 16), p.B + (long)(n0 + row) * ldk + kb * 64 + c * 16, 16);
        }
    };

    int32_t c[4][4][4];
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) { c[i][j][k] = 0; acc[i][j][k] = 0.0f; }

#pragma unroll
    for (int s = 0; s < TSTAGES - 1; ++s) {
        if (s < KB) load_stage(s, s);
        cp_async_commit();
    }
    const bool has_zero = p.a_zero != nullptr;
    auto dequant_all = [&](int grp) {
        ColQ cq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) cq[j] = load_colq(p, n0 + wn * 32 + j * 8 + 2 * t, grp, has_zero);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const RowQ rq = load_rowq(p, m0 + wm * 64 + i * 16 + g, grp, has_zero);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dequant_frag(c[i][j], acc[i][j], rq, cq[j]);
#pragma unroll
                for (int k = 0; k < 4; ++k) c[i][j][k] = 0;
            }
        }
    };

    for (int kb = 0; kb < KB; ++kb) {
        cp_async_wait<TSTAGES - 2>();
        __syncthreads();
        if (kb + TSTAGES - 1 < KB) load_stage((kb + TSTAGES - 1) % TSTAGES, kb + TSTAGES - 1);
        cp_async_commit();

        const uint8_t *sA = smem + (kb % TSTAGES) * TSTAGE_BYTES, *sB = sA + TBM * 64;
        uint4 bw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            bw[j] = *reinterpret_cast<const uint4 *>(sB + (wn * 32 + j * 8 + g) * 64 + t * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 a_lo = *reinterpret_cast<const uint4 *>(sA + (wm * 64 + i * 16 + g) * 64 + t * 16);
            const uint4 a_hi = *reinterpret_cast<const uint4 *>(sA + (wm * 64 + i * 16 + g + 8) * 64 + t * 16);
            const uint32_t al[4] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w}, ah[4] = {a_hi.x, a_hi.y, a_hi.z, a_hi.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t b[4] = {bw[j].x, bw[j].y, bw[j].z, bw[j].w};
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    mma_i8<A_UNSIGNED>(c[i][j], even16(al[q]), even16(ah[q]), odd16(al[q]), odd16(ah[q]),
                                       even16(b[q]), odd16(b[q]));
            }
        }
        if (p.grouped) dequant_all(kb);
    }
    cp_async_wait<0>();
    if (!p.grouped) dequant_all(0);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + wn * 32 + j * 8 + 2 * t;
            float b0 = 0.f, b1 = 0.f;
            if (p.bias) { b0 = __half2float(p.bias[col]); b1 = __half2float(p.bias[col + 1]); }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = m0 + wm * 64 + i * 16 + g + 8 * h;
                if (r < p.M) {
                    float v0 = acc[i][j][2 * h], v1 = acc[i][j][2 * h + 1];
                    if (p.bias) { v0 = __fadd_rn(v0, b0); v1 = __fadd_rn(v1, b1); }
                    store_pair(p.D, p.out_bf16, (long)r * p.N + col, v0, v1);
                }
            }
        }
}

// --------------------------------------------------------------------------------------------
// Tile kernel for K-groups of GS = 32 or 64 (the *_gs entry points of the reference, which scale every 128-K block with
// the FIRST scale of the block whatever the group size; here every group of GS elements gets its own scales).  Same CTA tile and
// cp.async ring as above; the difference is the order in which a 128-K stage is fed to the tensor cores: one
// m16n8k32 per 32-element sub-block (thread t takes the t-th 32-bit word of the sub-block's 16 packed bytes), so that
// the int32 fragment after 1 (GS = 32) or 2 (GS = 64) instructions is the exact integer sum of one group and can be
// folded into the binary32 accumulator with that group's scales.
template <bool A_UNSIGNED, int GS>
__global__ void __launch_bounds__(256)
gemm_tile_gs_kernel(const GemmParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp >> 2, wn = warp & 3;
    const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;
    const int KB = p.K / 128;
    const long ldk = p.K / 2;
    const int G = p.K / GS;                                  // groups per row (row sums are [N][G])
    const bool has_zero = p.a_zero != nullptr;

    auto load_stage = [&](int stage, int kb) {
        uint8_t *sA = smem + stage * TSTAGE_BYTES, *sB = sA + TBM * 64;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int ch = tid + i * 256, row = ch >> 2, c = ch & 3;
            const int gr = m0 + row;
            const uint8_t *src = p.A + (long)(gr < p.M ? gr : p.M - 1) * ldk + kb * 64 + c * 16;
            cp_async16(smem_u32(sA + row * 64 + c * 16), src, gr < p.M ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int ch = tid + i * 256, row = ch >> 2, c = ch & 3;
            cp_async16(smem_u32(sB + row * 64 + c * 16), p.B + (long)(n0 + row) * ldk + kb * 64 + c * 16, 16);
        }
    };

    int32_t c[4][4][4];
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) { c[i][j][k] = 0; acc[i][j][k] = 0.0f; }
#pragma unroll
    for (int s = 0; s < TSTAGES - 1; ++s) {
        if (s < KB) load_stage(s, s);
        cp_async_commit();
    }
    // fold the integer sums of group grp into the accumulators
    auto dequant_all = [&](int grp) {
        const int ga = p.ga_cols == 1 ? 0 : grp, gb = p.gb_cols == 1 ? 0 : grp;
        float sb[4][2];
        int rs[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = n0 + wn * 32 + j * 8 + 2 * t + e;
                sb[j][e] = __half2float(p.b_scale[(long)col * p.gb_cols + gb]);
                rs[j][e] = has_zero ? p.b_rowsum[(long)col * G + grp] : 0;
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = min(m0 + wm * 64 + i * 16 + g + 8 * h, p.M - 1);
                const float sa = __half2float(p.a_scale[(long)r * p.ga_cols + ga]);
                const int za = has_zero ? (int)__half2float(p.a_zero[(long)r * p.ga_cols + ga]) : 0;
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int32_t I = (c[i][j][2 * h + e] >> 8) - za * rs[j][e];
                        acc[i][j][2 * h + e] = __fmaf_rn((float)I, __fmul_rn(sa, sb[j][e]), acc[i][j][2 * h + e]);
                        c[i][j][2 * h + e] = 0;
                    }
            }
        }
    };

    for (int kb = 0; kb < KB; ++kb) {
        cp_async_wait<TSTAGES - 2>();
        __syncthreads();
        if (kb + TSTAGES - 1 < KB) load_stage((kb + TSTAGES - 1) % TSTAGES, kb + TSTAGES - 1);
        cp_async_commit();
        const uint8_t *sA = smem + (kb % TSTAGES) * TSTAGE_BYTES, *sB = sA + TBM * 64;
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {                   // 32-element sub-block = 16 packed bytes = one word per thread t
            uint32_t bw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) bw[j] = *reinterpret_cast<const uint32_t *>(sB + (wn * 32 + j * 8 + g) * 64 + sub * 16 + t * 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t al = *reinterpret_cast<const uint32_t *>(sA + (wm * 64 + i * 16 + g) * 64 + sub * 16 + t * 4);
                const uint32_t ah = *reinterpret_cast<const uint32_t *>(sA + (wm * 64 + i * 16 + g + 8) * 64 + sub * 16 + t * 4);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mma_i8<A_UNSIGNED>(c[i][j], even16(al), even16(ah), odd16(al), odd16(ah), even16(bw[j]), odd16(bw[j]));
            }
            if (GS == 32) dequant_all(kb * 4 + sub);
            else if (sub & 1) dequant_all(kb * 2 + (sub >> 1));
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + wn * 32 + j * 8 + 2 * t;
            float b0 = 0.f, b1 = 0.f;
            if (p.bias) { b0 = __half2float(p.bias[col]); b1 = __half2float(p.bias[col + 1]); }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = m0 + wm * 64 + i * 16 + g + 8 * h;
                if (r < p.M) {
                    float v0 = acc[i][j][2 * h], v1 = acc[i][j][2 * h + 1];
                    if (p.bias) { v0 = __fadd_rn(v0, b0); v1 = __fadd_rn(v1, b1); }
                    store_pair(p.D, p.out_bf16, (long)r * p.N + col, v0, v1);
                }
            }
        }
}

// --------------------------------------------------------------------------------------------
// Streaming kernel for decode (M <= 64): HBM-bound on the packed weight bytes.
//
// The weights are the ROW operand of mma.m16n8k32 (16 output channels per warp), the tokens the
// column operand (8 per mma), so a warp spends 2 shared-memory loads, 24 logic ops and 4 mma per
// kilobyte of weights for up to 8 tokens.  CTA = WARPS warps = 16*WARPS weight rows; K advances in
// stages of 256 (128 packed bytes per row) through a 6-deep cp.async ring that also carries
// the token tile and, for group-128 scales, the two scale groups of the stage (4-byte copies), so
// the dequantisation never waits on global memory.  16-byte chunk c of row r sits at chunk
// c ^ ((r & 1) << 2): the eight lanes of a quarter warp (two rows x four chunks) cover all banks.
constexpr int SSTAGES = 6;

template <int WARPS, int NT>
struct StreamPlan {
    static constexpr int BN = 16 * WARPS, TOK = 8 * NT;
    static constexpr int TS = NT == 1 ? 1 : (NT == 2 ? 2 : 4);   // warps sharing one weight tile, each with NT / TS token tiles
    static constexpr int kB = 0;                              // weights  BN x 128 B
    static constexpr int kA = kB + BN * 128;                  // tokens   TOK x 128 B
    static constexpr int kSB = kA + TOK * 128;                // weight scales  [BN][2] half
    static constexpr int kRS = kSB + BN * 4;                  // weight row sums [BN][2] int32
    static constexpr int kSA = kRS + BN * 8;                  // token scales   [TOK][2] half
    static constexpr int kZA = kSA + TOK * 4;                 // token zeros    [TOK][2] half
    static constexpr int kStage = ((kZA + TOK * 4 + 127) / 128) * 128;
};

__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src));
}

template <bool B_UNSIGNED>
__device__ __forceinline__ void mma_w_by_tok(int32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    if (B_UNSIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// SPLIT: blockIdx.y selects a contiguous range of 256-K stages; every CTA of a row slab writes its partial
// sums (int32 without group scales — exact; binary32 chains with them) to scratch, and the last one to
// arrive (a counter per slab) adds them in split order, finishes the epilogue and re-zeroes the counter.
template <int WARPS, int NT, bool A_UNSIGNED, bool GROUPED, bool SPLIT>
__global__ void __launch_bounds__(WARPS * StreamPlan<WARPS, NT>::TS * 32)
gemm_stream_kernel(const GemmParams p) {
    using Plan = StreamPlan<WARPS, NT>;
    constexpr int BN = Plan::BN, TOK = Plan::TOK, TS = Plan::TS, NTW = NT / TS, NTHREADS = WARPS * TS * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31;
    // warp (wr, wt): 16 weight rows wr, token tiles [wt * NTW, (wt + 1) * NTW) — the warps of a token split
    // read the same weight tile from shared memory, so more warps hide latency at no extra HBM traffic
    const int warp = (tid >> 5) % WARPS, wt = (tid >> 5) / WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * BN;
    const int KB = p.K / 128, KB2 = (KB + 1) / 2;
    const long ldk = p.K / 2;
    const bool has_zero = A_UNSIGNED;
    int st_begin = 0, st_end = KB2;                    // this CTA's range of 256-K stages
    if (SPLIT) {
        const int per = (KB2 + p.splits - 1) / p.splits;
        st_begin = blockIdx.y * per;
        st_end = min(KB2, st_begin + per);
    }
    // 4-byte copies of two adjacent f16 scales need an even number of groups per row
    const bool pair_ok = (KB & 1) == 0;

    auto load_stage = [&](int stage, int kb2) {
        uint8_t *st = smem + stage * Plan::kStage;
        const int kbytes = (int)ldk - kb2 * 128;          // bytes left in a row from this stage on
        for (int ch = tid; ch < BN * 8; ch += NTHREADS) {
            const int row = ch >> 3, c = ch & 7;
            const bool ok = c * 16 < kbytes;
            cp_async16(smem_u32(st + Plan::kB + row * 128 + ((c ^ ((row & 1) << 2)) << 4)),
                       p.B + (long)(n0 + row) * ldk + kb2 * 128 + (ok ? c * 16 : 0), ok ? 16 : 0);
        }
        for (int ch = tid; ch < TOK * 8; ch += NTHREADS) {
            const int row = ch >> 3, c = ch & 7;
            const bool ok = row < p.M && c * 16 < kbytes;
            cp_async16(smem_u32(st + Plan::kA + row * 128 + ((c ^ ((row & 1) << 2)) << 4)),
                       p.A + (long)(row < p.M ? row : p.M - 1) * ldk + kb2 * 128 + (c * 16 < kbytes ? c * 16 : 0), ok ? 16 : 0);
        }
        if (GROUPED) {
            const int g0 = kb2 * 2;
            const bool two = g0 + 1 < KB;
            // weight side: BN rows; token side: TOK rows.  One thread per row and array.
            for (int r = tid; r < BN; r += NTHREADS) {
                if (p.gb_cols > 1) {
                    const __half *src = p.b_scale + (long)(n0 + r) * KB + g0;
                    __half *dst = reinterpret_cast<__half *>(st + Plan::kSB) + 2 * r;
                    if (pair_ok) cp_async4(smem_u32(dst), src);
                    else { dst[0] = src[0]; dst[1] = two ? src[1] : src[0]; }
                }
                if (has_zero) {
                    const int32_t *src = p.b_rowsum + (long)(n0 + r) * KB + g0;
                    int32_t *dst = reinterpret_cast<int32_t *>(st + Plan::kRS) + 2 * r;
                    if (pair_ok) cp_async8(smem_u32(dst), src);
                    else { dst[0] = src[0]; dst[1] = two ? src[1] : src[0]; }
                }
            }
            for (int r = tid; r < TOK; r += NTHREADS) {
                const int rr = r < p.M ? r : p.M - 1;
                if (p.ga_cols > 1) {
                    const __half *src = p.a_scale + (long)rr * KB + g0;
                    __half *dst = reinterpret_cast<__half *>(st + Plan::kSA) + 2 * r;
                    if (pair_ok) cp_async4(smem_u32(dst), src);
                    else { dst[0] = src[0]; dst[1] = two ? src[1] : src[0]; }
                    if (has_zero) {
                        const __half *zs = p.a_zero + (long)rr * KB + g0;
                        __half *zd = reinterpret_cast<__half *>(st + Plan::kZA) + 2 * r;
                        if (pair_ok) cp_async4(smem_u32(zd), zs);
                        else { zd[0] = zs[0]; zd[1] = two ? zs[1] : zs[0]; }
                    }
                }
            }
        }
    };

    int32_t c[NTW][4];
    float acc[NTW][4];
#pragma unroll
    for (int i = 0; i < NTW; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) { c[i][k] = 0; acc[i][k] = 0.0f; }

    // quantities that do not depend on the K-group
    float sb_c[2] = {0.f, 0.f}, sa_c[NTW][2];
    int za_c[NTW][2];
    const int ch0 = n0 + warp * 16 + g;                  // this thread's channels: ch0, ch0 + 8
#pragma unroll
    for (int ii = 0; ii < NTW; ++ii)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = wt * NTW + ii;
            const int tok = min(i * 8 + 2 * t + j, p.M - 1);
            sa_c[ii][j] = p.ga_cols == 1 ? __half2float(p.a_scale[tok]) : 0.f;
            za_c[ii][j] = (has_zero && p.ga_cols == 1) ? (int)__half2float(p.a_zero[tok]) : 0;
        }
    if (p.gb_cols == 1) { sb_c[0] = __half2float(p.b_scale[ch0]); sb_c[1] = __half2float(p.b_scale[ch0 + 8]); }

#pragma unroll
    for (int s = 0; s < SSTAGES - 1; ++s) {
        if (st_begin + s < st_end) load_stage(s, st_begin + s);
        cp_async_commit();
    }

    for (int kb2 = st_begin; kb2 < st_end; ++kb2) {
        const int rel = kb2 - st_begin;
        cp_async_wait<SSTAGES - 2>();
        __syncthreads();
        if (kb2 + SSTAGES - 1 < st_end) load_stage((rel + SSTAGES - 1) % SSTAGES, kb2 + SSTAGES - 1);
        cp_async_commit();

        const uint8_t *st = smem + (rel % SSTAGES) * Plan::kStage;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int kb = kb2 * 2 + half;
            if (kb >= KB) break;
            const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
            const int chunk = half * 4 + t;
            const uint4 w_lo = *reinterpret_cast<const uint4 *>(st + Plan::kB + r_lo * 128 + ((chunk ^ ((r_lo & 1) << 2)) << 4));
            const uint4 w_hi = *reinterpret_cast<const uint4 *>(st + Plan::kB + r_hi * 128 + ((chunk ^ ((r_hi & 1) << 2)) << 4));
            const uint32_t wl[4] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w}, wh[4] = {w_hi.x, w_hi.y, w_hi.z, w_hi.w};
            uint32_t a0[4], a1[4], a2[4], a3[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) { a0[q] = even16(wl[q]); a1[q] = even16(wh[q]); a2[q] = odd16(wl[q]); a3[q] = odd16(wh[q]); }
#pragma unroll
            for (int ii = 0; ii < NTW; ++ii) {
                const int i = wt * NTW + ii;
                const int tr = i * 8 + g;
                const uint4 xv = *reinterpret_cast<const uint4 *>(st + Plan::kA + tr * 128 + ((chunk ^ ((tr & 1) << 2)) << 4));
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                int32_t c2[4] = {0, 0, 0, 0};          // second chain: the four mma no longer depend on each other in a row
                mma_w_by_tok<A_UNSIGNED>(c[ii], a0[0], a1[0], a2[0], a3[0], even16(xw[0]), odd16(xw[0]));
                mma_w_by_tok<A_UNSIGNED>(c2, a0[1], a1[1], a2[1], a3[1], even16(xw[1]), odd16(xw[1]));
                mma_w_by_tok<A_UNSIGNED>(c[ii], a0[2], a1[2], a2[2], a3[2], even16(xw[2]), odd16(xw[2]));
                mma_w_by_tok<A_UNSIGNED>(c2, a0[3], a1[3], a2[3], a3[3], even16(xw[3]), odd16(xw[3]));
#pragma unroll
                for (int k = 0; k < 4; ++k) c[ii][k] += c2[k];
                if (GROUPED) {
                    // c[i][2h + j]: channel ch0 + 8h, token i*8 + 2t + j.  Scales of this K-group come from the
                    // stage in shared memory; without zero-points the x256 of the accumulator rides in the scale.
                    const int r0 = warp * 16 + g;
                    float sbv[2], sav[2];
                    int rsv[2] = {0, 0}, zav[2] = {0, 0};
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sbv[h] = p.gb_cols == 1 ? sb_c[h] : __half2float(reinterpret_cast<const __half *>(st + Plan::kSB)[2 * (r0 + 8 * h) + half]);
                        if (has_zero) rsv[h] = reinterpret_cast<const int32_t *>(st + Plan::kRS)[2 * (r0 + 8 * h) + half];
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int tk = i * 8 + 2 * t + j;
                        sav[j] = p.ga_cols == 1 ? sa_c[ii][j] : __half2float(reinterpret_cast<const __half *>(st + Plan::kSA)[2 * tk + half]);
                        if (has_zero) zav[j] = p.ga_cols == 1 ? za_c[ii][j] : (int)__half2float(reinterpret_cast<const __half *>(st + Plan::kZA)[2 * tk + half]);
                        if (!has_zero) sav[j] *= (1.0f / 256.0f);
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int32_t I = has_zero ? (c[ii][2 * h + j] >> 8) - zav[j] * rsv[h] : c[ii][2 * h + j];
                            acc[ii][2 * h + j] = __fmaf_rn((float)I, __fmul_rn(sav[j], sbv[h]), acc[ii][2 * h + j]);
                            c[ii][2 * h + j] = 0;
                        }
                }
            }
        }
    }
    cp_async_wait<0>();

    if (SPLIT) {
        __shared__ int s_last;
        constexpr int TOKP = 8 * NT;
        // raw 32-bit partials: int32 (x256) without group scales, binary32 chains with them
#pragma unroll
        for (int ii = 0; ii < NTW; ++ii)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = wt * NTW + ii;
                    const int tok = i * 8 + 2 * t + j;
                    const float w = GROUPED ? acc[ii][2 * h + j] : __int_as_float(c[ii][2 * h + j]);
                    p.partials[((long)blockIdx.y * TOKP + tok) * p.N + ch0 + 8 * h] = w;
                }
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(&p.counters[blockIdx.x], 1) == p.splits - 1;
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int ii = 0; ii < NTW; ++ii)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = wt * NTW + ii;
                    const int tok = i * 8 + 2 * t + j;
                    float fsum = 0.0f;
                    int isum = 0;
                    for (int sp = 0; sp < p.splits; ++sp) {
                        const float w = __ldcg(&p.partials[((long)sp * TOKP + tok) * p.N + ch0 + 8 * h]);
                        if (GROUPED) fsum = sp == 0 ? w : __fadd_rn(fsum, w);
                        else isum += __float_as_int(w);
                    }
                    acc[ii][2 * h + j] = fsum;
                    c[ii][2 * h + j] = isum;
                }
        if (tid == 0) p.counters[blockIdx.x] = 0;       // ready for the next launch
    }

#pragma unroll
    for (int ii = 0; ii < NTW; ++ii)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int i = wt * NTW + ii;
            const int ch = ch0 + 8 * h;
            const float bias = p.bias ? __half2float(p.bias[ch]) : 0.f;
            const int rs = (!GROUPED && has_zero) ? p.b_rowsum[ch] : 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int tok = i * 8 + 2 * t + j;
                float v = acc[ii][2 * h + j];
                if (!GROUPED) {
                    const int32_t I = (c[ii][2 * h + j] >> 8) - za_c[ii][j] * rs;
                    v = __fmaf_rn((float)I, __fmul_rn(sa_c[ii][j], sb_c[h]), 0.0f);
                }
                if (p.bias) v = __fadd_rn(v, bias);
                if (tok < p.M) {
                    if (p.out_bf16) static_cast<__nv_bfloat16 *>(p.D)[(long)tok * p.N + ch] = __float2bfloat16_rn(v);
                    else static_cast<__half *>(p.D)[(long)tok * p.N + ch] = __float2half_rn(v);
                }
            }
        }
}

GemmParams make_params(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                       const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                       long M, long N, long K, long a_group, long b_group, int out_dtype) {
    GemmParams p;
    p.A = A; p.B = B;
    p.a_scale = static_cast<const __half *>(a_scale);
    p.a_zero = static_cast<const __half *>(a_zero);
    p.b_scale = static_cast<const __half *>(b_scale);
    p.bias = static_cast<const __half *>(bias);
    p.b_rowsum = b_rowsum; p.D = D;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.ga_cols = (int)(K / a_group); p.gb_cols = (int)(K / b_group);
    p.grouped = (a_group < K || b_group < K) ? 1 : 0;
    p.out_bf16 = out_dtype == FLH_B200_BF16;
    p.splits = 1; p.counters = nullptr; p.partials = nullptr;
    return p;
}

}  // namespace

int launch_gemm_mma_tile(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                         const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                         long M, long N, long K, long a_group, long b_group, int out_dtype,
                         cudaStream_t stream) {
    const GemmParams p = make_params(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype);
    const int smem = TSTAGES * TSTAGE_BYTES;
    dim3 grid((unsigned)(N / TBN), (unsigned)((M + TBM - 1) / TBM));
    cudaError_t e;
    if (a_zero) {
        e = cudaFuncSetAttribute(gemm_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_status(e, "gemm_tile attribute");
        gemm_tile_kernel<true><<<grid, 256, smem, stream>>>(p);
    } else {
        e = cudaFuncSetAttribute(gemm_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_status(e, "gemm_tile attribute");
        gemm_tile_kernel<false><<<grid, 256, smem, stream>>>(p);
    }
    return cuda_status(cudaGetLastError(), "gemm_tile launch");
}

// K-groups of 32 or 64: a_group and b_group are each gs or K.
int launch_gemm_mma_tile_gs(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                            const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                            long M, long N, long K, long a_group, long b_group, int gs, int out_dtype,
                            cudaStream_t stream) {
    const GemmParams p = make_params(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype);
    const int smem = TSTAGES * TSTAGE_BYTES;
    dim3 grid((unsigned)(N / TBN), (unsigned)((M + TBM - 1) / TBM));
    using Kern = void (*)(const GemmParams);
    const Kern kern = a_zero ? (gs == 32 ? gemm_tile_gs_kernel<true, 32> : gemm_tile_gs_kernel<true, 64>)
                             : (gs == 32 ? gemm_tile_gs_kernel<false, 32> : gemm_tile_gs_kernel<false, 64>);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "gemm_tile_gs attribute");
    kern<<<grid, 256, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "gemm_tile_gs launch");
}

template <int WARPS, int NT, bool U, bool G, bool SPLIT>
static int launch_stream_t(const GemmParams &p, cudaStream_t stream) {
    const int smem = SSTAGES * StreamPlan<WARPS, NT>::kStage;
    auto kern = gemm_stream_kernel<WARPS, NT, U, G, SPLIT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "gemm_stream attribute");
    dim3 grid((unsigned)(p.N / (16 * WARPS)), (unsigned)(SPLIT ? p.splits : 1));
    kern<<<grid, WARPS * StreamPlan<WARPS, NT>::TS * 32, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "gemm_stream launch");
}

template <int WARPS, int NT>
static int launch_stream_w(const GemmParams &p, bool u, cudaStream_t stream) {
    if (p.splits > 1) {
        if (p.grouped) return u ? launch_stream_t<WARPS, NT, true, true, true>(p, stream) : launch_stream_t<WARPS, NT, false, true, true>(p, stream);
        return u ? launch_stream_t<WARPS, NT, true, false, true>(p, stream) : launch_stream_t<WARPS, NT, false, false, true>(p, stream);
    }
    if (p.grouped) return u ? launch_stream_t<WARPS, NT, true, true, false>(p, stream) : launch_stream_t<WARPS, NT, false, true, false>(p, stream);
    return u ? launch_stream_t<WARPS, NT, true, false, false>(p, stream) : launch_stream_t<WARPS, NT, false, false, false>(p, stream);
}

// Split-K plan of the streaming kernel: how many CTAs share a 32-row slab along K, and the scratch they need.
// The slabs alone fill the GPU when there are at least two per SM; otherwise K is cut so that about three
// CTAs per SM exist, keeping at least four 256-K stages per CTA.
int stream_splits(long M, long N, long K) {
    (void)M;
    const long slabs = N / 32;
    if (slabs >= 2 * kNumSMs) return 1;
    const long stages = (K / 128 + 1) / 2;
    long s = (3 * kNumSMs + slabs - 1) / slabs;
    if (s > stages / 4) s = stages / 4;
    if (s > 8) s = 8;
    return s < 2 ? 1 : (int)s;
}
size_t stream_scratch_bytes(long M, long N, int splits) {
    if (splits <= 1) return 0;
    const long tokp = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    return 4096 + (size_t)splits * tokp * N * 4;           // 4 KB of slab counters, then the partial sums
}

int launch_gemm_stream(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                       const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                       long M, long N, long K, long a_group, long b_group, int out_dtype,
                       int splits, void *scratch, cudaStream_t stream) {
    GemmParams p = make_params(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype);
    p.splits = splits > 1 ? splits : 1;
    p.counters = static_cast<int *>(scratch);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + 4096);
    const bool u = a_zero != nullptr;
    // 32-row CTAs unless that would be more than ~8 CTAs per SM; N is a multiple of 128
    const bool wide = splits <= 1 && N / 32 > 8 * kNumSMs;
    if (M <= 8) return wide ? launch_stream_w<4, 1>(p, u, stream) : launch_stream_w<2, 1>(p, u, stream);
    if (M <= 16) return wide ? launch_stream_w<4, 2>(p, u, stream) : launch_stream_w<2, 2>(p, u, stream);
    if (M <= 32) return wide ? launch_stream_w<4, 4>(p, u, stream) : launch_stream_w<2, 4>(p, u, stream);
    return launch_stream_w<2, 8>(p, u, stream);
}

// --------------------------------------------------------------------------------------------
// Split-K decode GEMM for callers that cannot allocate device memory: the scratch the kernel needs
// (slab counters + per-split partial sums) lives in this file-scope device array instead of a caller
// buffer.  Every GPU that loads the library holds the array until the process exits.
constexpr size_t kStaticScratchBytes = 4096 + (2u << 20);      // counters + 2 MiB of partial sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, never a device address: the address
// is asked for once per device, with that device current, and remembered.
static void *g_static_scratch_addr[64];

size_t stream_static_scratch_capacity() { return kStaticScratchBytes; }

int launch_gemm_stream_static(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                              const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                              long M, long N, long K, long a_group, long b_group, int out_dtype,
                              cudaStream_t stream) {
    const int splits = stream_splits(M, N, K);
    if (splits <= 1)        // this shape fills the GPU without cutting K: no scratch is involved at all
        return launch_gemm_stream(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, 1, nullptr, stream);
    const size_t need = stream_scratch_bytes(M, N, splits);
    if (need > kStaticScratchBytes)
        return fail(FLH_B200_EINVAL,
                    "M=%ld N=%ld K=%ld needs %zu bytes of split-K scratch, more than the %zu bytes built into the library; "
                    "use flh_b200_gemm_i4_dequant with a caller workspace", M, N, K, need, (size_t)kStaticScratchBytes);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FLH_B200_EUNSUPPORTED, "device ordinal %d is outside the table of 64", dev);
    void *ptr = g_static_scratch_addr[dev];
    if (!ptr) {             // first call on this device (do it before any stream capture)
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return cuda_status(e, "cudaGetSymbolAddress(static scratch)");
        g_static_scratch_addr[dev] = ptr;
    }
    // the array keeps whatever the previous call left: the arrival counters must start at zero
    e = cudaMemsetAsync(ptr, 0, 4096, stream);
    if (e != cudaSuccess) return cuda_status(e, "clearing the static scratch counters");
    return launch_gemm_stream(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype, splits, ptr, stream);
}

// rowsum[n, g] = sum of signed nibbles of row n over K-group g.  One warp per (row, group chunk).
__global__ void weight_rowsum_kernel(const uint8_t *__restrict__ B, int N, int K, int group,
                                     int32_t *__restrict__ rs) {
    const int G = K / group;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)N * G) return;
    const int lane = threadIdx.x & 31;
    const long n = item / G;
    const int gidx = (int)(item % G);
    const uint32_t *row = reinterpret_cast<const uint32_t *>(B + n * (K / 2) + (long)gidx * (group / 2));
    int32_t s = 0;
    for (int w = lane; w < group / 8; w += 32) {
        const uint32_t v = row[w];
        // sum of eight signed nibbles = sum of the int8 values (nibble << 4) >> 4
        const int32_t e = __dp4a((int)even16(v), 0x01010101, 0);
        const int32_t o = __dp4a((int)odd16(v), 0x01010101, 0);
        s += (e + o) >> 4;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) rs[item] = s;
}

int launch_weight_rowsum(const uint8_t *B, long N, long K, long group, int32_t *rowsum, cudaStream_t stream) {
    const long items = N * (K / group);
    const int wpb = 8;
    weight_rowsum_kernel<<<(unsigned)((items + wpb - 1) / wpb), wpb * 32, 0, stream>>>(B, (int)N, (int)K, (int)group, rowsum);
    return cuda_status(cudaGetLastError(), "weight_rowsum launch");
}

}  // namespace flh
