// Group-wise (32/64/128) binary16 Walsh-Hadamard transform, fused symmetric int4 quantiser and
// nibble packing — the flh._CUDA activation path (hadamard_and_quantize_i4, quant_and_pack_i4,
// hadamard_transform_half and their group-size variants).
//
// Memory-bound: 2 B in, 0.5 B + 2/gs B out per element.  One thread owns 8 consecutive halves
// (one 128-bit load), so a group of gs spans gs/8 adjacent lanes: butterfly bits 0-2 are done in
// registers on half2 pairs, the remaining log2(gs)-3 bits with __shfl_xor, always in ascending bit
// order so that every binary16 rounding happens where the reference kernel has it
// (flh/kernels/had_and_quant.cu:13-56).  Each thread keeps U independent 16-byte loads in flight.
#include "common.cuh"
#include <stdlib.h>

namespace flh {

namespace {

constexpr int kUnroll = 4;
constexpr int kThreads = 256;

__device__ __forceinline__ __half2 u2h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// (a, b) -> (a + b, a - b), one rounding each (the product with +-1 is exact).
__device__ __forceinline__ __half2 bfly_inner(__half2 v) {
    const __half2 sgn = __halves2half2(__float2half(1.0f), __float2half(-1.0f));
    return __hfma2(__high2half2(v), sgn, __low2half2(v));
}

template <int LOG_GS>
__device__ __forceinline__ void fht_regs(__half2 (&h)[4], int lane_in_group) {
    // bits 0..2: in registers
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = bfly_inner(h[j]);
    {
        __half2 a = h[0], b = h[1], c = h[2], d = h[3];
        h[0] = __hadd2(a, b); h[1] = __hsub2(a, b);
        h[2] = __hadd2(c, d); h[3] = __hsub2(c, d);
    }
    {
        __half2 a = h[0], b = h[1], c = h[2], d = h[3];
        h[0] = __hadd2(a, c); h[2] = __hsub2(a, c);
        h[1] = __hadd2(b, d); h[3] = __hsub2(b, d);
    }
    // bits 3..LOG_GS-1: across lanes; the lane whose bit is set holds the upper element and
    // receives other - mine, the other lane mine + other.
#pragma unroll
    for (int s = 0; s < LOG_GS - 3; ++s) {
        const int mask = 1 << s;
        const float sg = (lane_in_group & mask) ? -1.0f : 1.0f;
        const __half2 sgn = __float2half2_rn(sg);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 other = u2h2(__shfl_xor_sync(0xffffffffu, h22u(h[j]), mask));
            h[j] = __hfma2(h[j], sgn, other);
        }
    }
}

// scale = __hdiv(max, 7) with a correctly rounded reciprocal (cuda_fp16.hpp __hdiv, device branch:
// reciprocal, multiply, round, one correction for tiny results); at most half(1e-6) -> 1.
__device__ __forceinline__ __half group_scale(__half m) {
    const float fm = __half2float(m);
    const float rcp7 = 1.0f / 7.0f;
    float fv = __fmul_rn(rcp7, fm);
    __half sh = __float2half_rn(fv);
    const unsigned short a = __half_as_ushort(sh) & 0x7fffu;
    if (a != 0 && a < 0x008Fu) {
        const float err = __fmaf_rn(-7.0f, fv, fm);
        fv = __fmaf_rn(rcp7, err, fv);
        sh = __float2half_rn(fv);
    }
    if (__half2float(sh) <= __half2float(__float2half_rn(1e-6f))) sh = __float2half_rn(1.0f);
    return sh;
}

// q = rint(half(x * rcp)) for the four half2 of eight consecutive elements -> eight packed nibbles.
// |x| <= max and scale = half(max / 7) keep |q| <= 7 for finite input, so the reference's clamp never acts.
// Adding 1032 (= 1024 + 8) in binary16 rounds to the nearest integer, ties to even, and leaves q + 8 in the
// low four bits of each half.
__device__ __forceinline__ uint32_t quant_pack8(const __half2 (&h)[4], float rcp) {
    const __half2 magic = __float2half2_rn(1032.0f);
    uint32_t nib[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        const __half2 t = __floats2half2_rn(__fmul_rn(f.x, rcp), __fmul_rn(f.y, rcp));
        nib[j] = (h22u(__hadd2(t, magic)) & 0x000F000Fu) ^ 0x00080008u;   // two's-complement nibbles at bits 0-3, 16-19
    }
    // nib[j] = [even code, 0, odd code, 0] as bytes; gather evens and odds, then byte j = even | odd << 4
    const uint32_t a01 = nib[1] * 256u + nib[0], a23 = nib[3] * 256u + nib[2];
    const uint32_t ev = __byte_perm(a01, a23, 0x5410), od = __byte_perm(a01, a23, 0x7632);
    return od * 16u + ev;
}

template <int LOG_GS, bool HADAMARD>
__global__ void __launch_bounds__(kThreads)
quant_group_sym_kernel(const uint4 *__restrict__ x, uint32_t *__restrict__ q,
                       __half *__restrict__ scales, long total_chunks) {
    constexpr int L = (1 << LOG_GS) / 8;          // lanes per group
    const long nthreads = (long)gridDim.x * kThreads;
    const long tid = (long)blockIdx.x * kThreads + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int lig = lane & (L - 1);

    for (long c0 = tid; c0 - lane < total_chunks; c0 += nthreads * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long c = c0 + u * nthreads;
            v[u] = (c < total_chunks) ? ldg_nc_v4(x + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long c = c0 + u * nthreads;
            if (c - lane >= total_chunks) break;   // warp-uniform
            __half2 h[4] = {u2h2(v[u].x), u2h2(v[u].y), u2h2(v[u].z), u2h2(v[u].w)};
            if (HADAMARD) fht_regs<LOG_GS>(h, lig);

            // max |x| over the group, in binary16
            __half2 m2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])),
                                 __hmax2(__habs2(h[2]), __habs2(h[3])));
            __half m = __hmax(__low2half(m2), __high2half(m2));
#pragma unroll
            for (int s = 1; s < L; s <<= 1) {
                const unsigned short o = __shfl_xor_sync(0xffffffffu, __half_as_ushort(m), s);
                m = __hmax(m, __ushort_as_half(o));
            }
            const __half sh = group_scale(m);
            const float rcp = __frcp_rn(__half2float(sh));

            const uint32_t packed = quant_pack8(h, rcp);
            if (c < total_chunks) {
                q[c] = packed;
                if (lig == 0) scales[c / L] = sh;
            }
        }
    }
}


// ---- one thread per group ------------------------------------------------------------------------------
// For large inputs: a lane owns a whole group (GS / 2 half2 registers), so all butterfly bits run in registers with
// no shuffle, and the scale is derived once per group instead of once per 8 elements.  A warp works on 32
// consecutive groups (64 GS bytes): they are staged in shared memory by coalesced 16-byte cp.async — chunk c of
// 128-byte line L lands at chunk c ^ key(L), key chosen per group size so that eight neighbouring lanes reading
// their own 16-byte chunks hit eight different bank groups — and the next tile of the persistent warp is in flight
// while this one is computed.
constexpr int kTWarps = 4;             // warps per CTA

// GS = 128: a lane reads lines 2 t and 2 t + 1, key (L >> 1) & 7.  GS = 64: line t, key L & 7.  GS = 32: half of
// line t >> 1, key L & 3 (bit 2 of the chunk index tells the two lanes of a line apart).
template <int GS>
__device__ __forceinline__ int swizzle_key(int line) {
    return GS == 128 ? (line >> 1) & 7 : GS == 64 ? line & 7 : line & 3;
}

template <int GS>
__device__ __forceinline__ void stage_groups(const uint8_t *x, long tile, long total_chunks, uint32_t stage, int lane) {
    constexpr int kCopies = GS / 8;                         // 16-byte copies per lane: 32 groups x 2 GS bytes / (32 lanes x 16)
    const long c0 = tile * (4 * GS) + lane;                 // 16-byte chunk index of this lane's first copy
#pragma unroll
    for (int i = 0; i < kCopies; ++i) {
        const long c = c0 + i * 32;
        const int line = 4 * i + (lane >> 3);
        const uint32_t dst = stage + line * 128 + (((lane & 7) ^ swizzle_key<GS>(line)) << 4);
        const int n = c < total_chunks ? 16 : 0;            // past the end: zero fill, nothing is read
        const uint8_t *src = x + (c < total_chunks ? c : 0) * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n));
    }
    asm volatile("cp.async.commit_group;" ::);
}

// NORM (GS = 128 only, rows of 4096 = one warp tile): RMS-normalise the row first, exactly as the per-token kernels do
// (each lane adds its 128 squares in order with fma, xor-shuffle tree 16 .. 1, c = 1 / sqrt(s / 4096 + eps) correctly
// rounded, y = half(x * c)).
template <int GS, bool HADAMARD, bool NORM = false>
__global__ void __launch_bounds__(kTWarps * 32, 4)
quant_group_thread_kernel(const uint8_t *__restrict__ x, uint4 *__restrict__ q, __half *__restrict__ scales, long groups, float eps = 0.0f) {
    static_assert(!NORM || GS == 128, "the fused norm is written for rows of 4096 = 32 groups of 128");
    constexpr int NH = GS / 2;                              // half2 registers of a group
    constexpr int kTile = 64 * GS;                          // bytes of one warp tile
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t *my = smem_raw + warp * kTile;
    const uint32_t stage = smem_u32(my);
    const long tiles = (groups + 31) >> 5, total_chunks = groups * (GS / 8);
    const long nwarps = (long)gridDim.x * kTWarps;
    long tile = (long)blockIdx.x * kTWarps + warp;
    if (tile < tiles) stage_groups<GS>(x, tile, total_chunks, stage, lane);

    for (; tile < tiles; tile += nwarps) {
        __half2 h[NH];
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int cc = 0; cc < GS / 8; ++cc) {               // this lane's chunks, in element order
            const int byte = lane * (2 * GS) + cc * 16;     // unswizzled position inside the tile
            const int line = byte >> 7, c = (byte >> 4) & 7;
            const uint4 w = *reinterpret_cast<const uint4 *>(my + line * 128 + ((c ^ swizzle_key<GS>(line)) << 4));
            h[cc * 4 + 0] = u2h2(w.x); h[cc * 4 + 1] = u2h2(w.y);
            h[cc * 4 + 2] = u2h2(w.z); h[cc * 4 + 3] = u2h2(w.w);
        }
        __syncwarp();                                       // the tile is in registers everywhere: refill the buffer
        if (tile + nwarps < tiles) stage_groups<GS>(x, tile + nwarps, total_chunks, stage, lane);

        if (NORM) {
            float ssq = 0.0f;
#pragma unroll
            for (int r = 0; r < NH; ++r) {
                const float2 f = __half22float2(h[r]);
                ssq = __fmaf_rn(f.x, f.x, ssq);
                ssq = __fmaf_rn(f.y, f.y, ssq);
            }
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) ssq = __fadd_rn(ssq, __shfl_xor_sync(0xffffffffu, ssq, sft));
            const float c = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(ssq, 1.0f / 4096.0f), eps)));
#pragma unroll
            for (int r = 0; r < NH; ++r) {
                const float2 f = __half22float2(h[r]);
                h[r] = __floats2half2_rn(__fmul_rn(f.x, c), __fmul_rn(f.y, c));
            }
        }
        if (HADAMARD) {
#pragma unroll
            for (int r = 0; r < NH; ++r) h[r] = bfly_inner(h[r]);                 // bit 0
#pragma unroll
            for (int d = 1; d < NH; d <<= 1) {                                    // the remaining bits
#pragma unroll
                for (int r = 0; r < NH; ++r) {
                    if ((r & d) == 0) {
                        const __half2 a = h[r], b = h[r + d];
                        h[r] = __hadd2(a, b);
                        h[r + d] = __hsub2(a, b);
                    }
                }
            }
        }
        __half2 m2 = __habs2(h[0]);
#pragma unroll
        for (int r = 1; r < NH; ++r) m2 = __hmax2(m2, __habs2(h[r]));
        const __half m = __hmax(__low2half(m2), __high2half(m2));
        const __half sh = group_scale(m);
        const float rcp = __frcp_rn(__half2float(sh));
        const long g = tile * 32 + lane;
        if (g < groups) {
#pragma unroll
            for (int v = 0; v < GS / 32; ++v) {
                uint32_t o[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const __half2 hh[4] = {h[16 * v + 4 * w], h[16 * v + 4 * w + 1], h[16 * v + 4 * w + 2], h[16 * v + 4 * w + 3]};
                    o[w] = quant_pack8(hh, rcp);
                }
                q[g * (GS / 32) + v] = make_uint4(o[0], o[1], o[2], o[3]);
            }
            scales[g] = sh;
        }
    }
}

template <int LOG_GS>
__global__ void __launch_bounds__(kThreads)
fht_inplace_kernel(uint4 *__restrict__ x, long total_chunks) {
    constexpr int L = (1 << LOG_GS) / 8;
    const long nthreads = (long)gridDim.x * kThreads;
    const long tid = (long)blockIdx.x * kThreads + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int lig = lane & (L - 1);
    for (long c0 = tid; c0 - lane < total_chunks; c0 += nthreads * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long c = c0 + u * nthreads;
            v[u] = (c < total_chunks) ? x[c] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long c = c0 + u * nthreads;
            if (c - lane >= total_chunks) break;
            __half2 h[4] = {u2h2(v[u].x), u2h2(v[u].y), u2h2(v[u].z), u2h2(v[u].w)};
            fht_regs<LOG_GS>(h, lig);
            if (c < total_chunks) x[c] = make_uint4(h22u(h[0]), h22u(h[1]), h22u(h[2]), h22u(h[3]));
        }
    }
}

// One wave of resident CTAs (a multiple of the SM count); the grid-stride loop covers the rest.
template <typename K>
int grid_for(K kernel, long total_chunks) {
    // resident CTAs per SM, remembered per kernel address (a handful of template instances)
    static const void *known[16];
    static int occ[16];
    int per_sm = 0;
    for (int i = 0; i < 16 && known[i]; ++i)
        if (known[i] == reinterpret_cast<const void *>(kernel)) per_sm = occ[i];
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, 0) != cudaSuccess || n < 1) n = 4;
        per_sm = n;
        for (int i = 0; i < 16; ++i)
            if (!known[i]) { occ[i] = n; known[i] = reinterpret_cast<const void *>(kernel); break; }
    }
    long blocks = (total_chunks + (long)kThreads * kUnroll - 1) / ((long)kThreads * kUnroll);
    const long cap = (long)kNumSMs * per_sm;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

// Groups from which the thread-per-group kernel is used (it measured faster from a few thousand groups on; below
// that the several-lanes-per-group kernel spreads a small input over more warps).  FLH_B200_GROUP_THREAD_MIN_ROWS
// overrides it (tuning aid).
static long group_thread_min_rows() {
    static long v = -1;
    if (v < 0) {
        const char *e = getenv("FLH_B200_GROUP_THREAD_MIN_ROWS");
        v = e ? atol(e) : 4096;
        if (v < 0) v = 0;
    }
    return v;
}

int launch_quant_group_sym(const void *x, long rows, int gs, int hadamard, uint8_t *q,
                           void *scales, cudaStream_t stream) {
    const long chunks = rows * (gs / 8);
    // many groups of 128: the thread-per-group kernel (a full wave of its persistent warps has 32 groups each)
    if (rows >= group_thread_min_rows()) {
        const long tiles = (rows + 31) / 32;
        long grid = (tiles + kTWarps - 1) / kTWarps;
        if (grid > 4L * kNumSMs) grid = 4L * kNumSMs;
        const uint8_t *xb = static_cast<const uint8_t *>(x);
        uint4 *qo4 = reinterpret_cast<uint4 *>(q);
        __half *so4 = static_cast<__half *>(scales);
#define FLH_TLAUNCH(GS_, H_) quant_group_thread_kernel<GS_, H_><<<(unsigned)grid, kTWarps * 32, kTWarps * 64 * GS_, stream>>>(xb, qo4, so4, rows)
        if (gs == 128) { if (hadamard) FLH_TLAUNCH(128, true); else FLH_TLAUNCH(128, false); }
        else if (gs == 64) { if (hadamard) FLH_TLAUNCH(64, true); else FLH_TLAUNCH(64, false); }
        else { if (hadamard) FLH_TLAUNCH(32, true); else FLH_TLAUNCH(32, false); }
#undef FLH_TLAUNCH
        return cuda_status(cudaGetLastError(), "quant_group_thread launch");
    }
    const uint4 *xi = static_cast<const uint4 *>(x);
    uint32_t *qo = reinterpret_cast<uint32_t *>(q);
    __half *so = static_cast<__half *>(scales);
#define FLH_LAUNCH(LG, H) quant_group_sym_kernel<LG, H><<<grid_for(quant_group_sym_kernel<LG, H>, chunks), kThreads, 0, stream>>>(xi, qo, so, chunks)
    if (gs == 128) { if (hadamard) FLH_LAUNCH(7, true); else FLH_LAUNCH(7, false); }
    else if (gs == 64) { if (hadamard) FLH_LAUNCH(6, true); else FLH_LAUNCH(6, false); }
    else { if (hadamard) FLH_LAUNCH(5, true); else FLH_LAUNCH(5, false); }
#undef FLH_LAUNCH
    return cuda_status(cudaGetLastError(), "quant_group_sym launch");
}

// rows of 4096 halves: RMS-norm + group-128 (transform +) symmetric int4 + pack
int launch_rmsnorm_quant_group(const void *x, long M, int hadamard, float eps, uint8_t *q, void *scales, cudaStream_t stream) {
    const long groups = M * 32;
    const long tiles = M;
    long grid = (tiles + kTWarps - 1) / kTWarps;
    if (grid > 4L * kNumSMs) grid = 4L * kNumSMs;
    const uint8_t *xb = static_cast<const uint8_t *>(x);
    uint4 *qo4 = reinterpret_cast<uint4 *>(q);
    __half *so4 = static_cast<__half *>(scales);
    if (hadamard) quant_group_thread_kernel<128, true, true><<<(unsigned)grid, kTWarps * 32, kTWarps * 64 * 128, stream>>>(xb, qo4, so4, groups, eps);
    else quant_group_thread_kernel<128, false, true><<<(unsigned)grid, kTWarps * 32, kTWarps * 64 * 128, stream>>>(xb, qo4, so4, groups, eps);
    return cuda_status(cudaGetLastError(), "rmsnorm_quant_group launch");
}

int launch_fht_inplace(void *x, long rows, int n, cudaStream_t stream) {
    const long chunks = rows * (n / 8);
    uint4 *xi = static_cast<uint4 *>(x);
    if (n == 128) fht_inplace_kernel<7><<<grid_for(fht_inplace_kernel<7>, chunks), kThreads, 0, stream>>>(xi, chunks);
    else if (n == 64) fht_inplace_kernel<6><<<grid_for(fht_inplace_kernel<6>, chunks), kThreads, 0, stream>>>(xi, chunks);
    else fht_inplace_kernel<5><<<grid_for(fht_inplace_kernel<5>, chunks), kThreads, 0, stream>>>(xi, chunks);
    return cuda_status(cudaGetLastError(), "fht_inplace launch");
}

}  // namespace flh
