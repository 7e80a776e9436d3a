// int4 x int4 GEMM with fused dequantisation on the legacy warp-level tensor path
// (mma.sync.m16n8k32 s8), two kernels:
//   * gemm_tile_kernel    128x128x128 CTA tiles, cp.async ring; any M.  Bring-up cross-check for
//                         the tcgen05 kernel and the "legacy mma.sync" line of the benchmark.
//   * gemm_stream_kernel  decode shapes (M <= 32): every CTA streams a 32-row slab of packed
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
// Streaming kernel for decode: CTA = 4 warps, 32 weight rows (8 per warp), K in blocks of 256
// (128 packed bytes per row per stage), SSTAGES-deep ring.  The MT*16 activation rows ride in
// the same ring.  16-byte chunk c of row r sits at chunk c ^ ((r & 1) << 2), so the eight lanes of
// a quarter warp (two rows x four chunks) touch all 32 banks once.
constexpr int SBN = 32, SSTAGES = 8;

template <int MT, bool A_UNSIGNED>
__global__ void __launch_bounds__(128)
gemm_stream_kernel(const GemmParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int STAGE_BYTES = (SBN + MT * 16) * 128;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * SBN;
    const int KB2 = (p.K + 255) / 256;          // 256-K stages; the last may be half full
    const long ldk = p.K / 2;

    auto load_stage = [&](int stage, int kb2) {
        uint8_t *sB = smem + stage * STAGE_BYTES, *sA = sB + SBN * 128;
        const int kbytes = (int)ldk - kb2 * 128;     // bytes left in the row from this stage on
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int ch = tid + i * 128, row = ch >> 3, c = ch & 7;
            const bool ok = c * 16 < kbytes;
            cp_async16(smem_u32(sB + row * 128 + ((c ^ ((row & 1) << 2)) << 4)),
                       p.B + (long)(n0 + row) * ldk + kb2 * 128 + (ok ? c * 16 : 0), ok ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            const int ch = tid + i * 128, row = ch >> 3, c = ch & 7;
            const bool ok = row < p.M && c * 16 < kbytes;
            cp_async16(smem_u32(sA + row * 128 + ((c ^ ((row & 1) << 2)) << 4)),
                       p.A + (long)(row < p.M ? row : p.M - 1) * ldk + kb2 * 128 + (c * 16 < kbytes ? c * 16 : 0),
                       ok ? 16 : 0);
        }
    };

    int32_t c[MT][4];
    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) { c[i][k] = 0; acc[i][k] = 0.0f; }

#pragma unroll
    for (int s = 0; s < SSTAGES - 1; ++s) {
        if (s < KB2) load_stage(s, s);
        cp_async_commit();
    }
    const bool has_zero = p.a_zero != nullptr;
    const int KB = p.K / 128;

    for (int kb2 = 0; kb2 < KB2; ++kb2) {
        cp_async_wait<SSTAGES - 2>();
        __syncthreads();
        if (kb2 + SSTAGES - 1 < KB2) load_stage((kb2 + SSTAGES - 1) % SSTAGES, kb2 + SSTAGES - 1);
        cp_async_commit();

        const uint8_t *sB = smem + (kb2 % SSTAGES) * STAGE_BYTES, *sA = sB + SBN * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int kb = kb2 * 2 + half;
            if (kb >= KB) break;
            const int brow = warp * 8 + g;
            const uint4 bv = *reinterpret_cast<const uint4 *>(sB + brow * 128 + (((half * 4 + t) ^ ((brow & 1) << 2)) << 4));
            const uint32_t b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int r_lo = i * 16 + g, r_hi = r_lo + 8;
                const uint4 a_lo = *reinterpret_cast<const uint4 *>(sA + r_lo * 128 + (((half * 4 + t) ^ ((r_lo & 1) << 2)) << 4));
                const uint4 a_hi = *reinterpret_cast<const uint4 *>(sA + r_hi * 128 + (((half * 4 + t) ^ ((r_hi & 1) << 2)) << 4));
                const uint32_t al[4] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w}, ah[4] = {a_hi.x, a_hi.y, a_hi.z, a_hi.w};
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    mma_i8<A_UNSIGNED>(c[i], even16(al[q]), even16(ah[q]), odd16(al[q]), odd16(ah[q]),
                                       even16(b[q]), odd16(b[q]));
                if (p.grouped) {
                    dequant_frag(c[i], acc[i], load_rowq(p, i * 16 + g, kb, has_zero),
                                 load_colq(p, n0 + warp * 8 + 2 * t, kb, has_zero));
#pragma unroll
                    for (int k = 0; k < 4; ++k) c[i][k] = 0;
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        if (!p.grouped)
            dequant_frag(c[i], acc[i], load_rowq(p, i * 16 + g, 0, has_zero),
                         load_colq(p, n0 + warp * 8 + 2 * t, 0, has_zero));
        const int col = n0 + warp * 8 + 2 * t;
        float b0 = 0.f, b1 = 0.f;
        if (p.bias) { b0 = __half2float(p.bias[col]); b1 = __half2float(p.bias[col + 1]); }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = i * 16 + g + 8 * h;
            if (r < p.M) {
                float v0 = acc[i][2 * h], v1 = acc[i][2 * h + 1];
                if (p.bias) { v0 = __fadd_rn(v0, b0); v1 = __fadd_rn(v1, b1); }
                store_pair(p.D, p.out_bf16, (long)r * p.N + col, v0, v1);
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

template <int MT, bool U>
static int launch_stream_t(const GemmParams &p, cudaStream_t stream) {
    const int smem = SSTAGES * (SBN + MT * 16) * 128;
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<MT, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "gemm_stream attribute");
    gemm_stream_kernel<MT, U><<<(unsigned)(p.N / SBN), 128, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "gemm_stream launch");
}

int launch_gemm_stream(const uint8_t *A, const uint8_t *B, const void *a_scale, const void *a_zero,
                       const void *b_scale, const int32_t *b_rowsum, const void *bias, void *D,
                       long M, long N, long K, long a_group, long b_group, int out_dtype,
                       cudaStream_t stream) {
    const GemmParams p = make_params(A, B, a_scale, a_zero, b_scale, b_rowsum, bias, D, M, N, K, a_group, b_group, out_dtype);
    if (M <= 16) return a_zero ? launch_stream_t<1, true>(p, stream) : launch_stream_t<1, false>(p, stream);
    return a_zero ? launch_stream_t<2, true>(p, stream) : launch_stream_t<2, false>(p, stream);
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
