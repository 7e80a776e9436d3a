// One-shot all-reduce of the small f16 / bf16 messages of tensor-parallel decode (the partial outputs of a
// row-parallel linear: at most a few MB), over peer-mapped buffers with plain stores and loads across NVLink.
// The reference has no multi-GPU code; this replaces the NCCL all-reduce behind RowParallelLinearFLH for messages
// whose cost is latency, not bandwidth.
//
// Every rank owns one device buffer: a control block, arrival flags [parity][source rank][CTA] and receive slots
// [parity][source rank][max_bytes]; the peers' buffers are mapped through CUDA IPC (other processes) or directly
// (same process).  One launch per rank, CTA c of every rank working on the same piece c of the message:
//   1. PUSH   the piece of this rank's message into slot [parity][rank] of every peer (16-byte stores),
//   2. SIGNAL flag [parity][rank][c] = epoch in every peer, a system-scope release store,
//   3. WAIT   until the local flags [parity][src][c] of all peers show the epoch (bounded: after 2 s the CTA records
//             status and goes on, so the kernel always ends),
//   4. SUM    own piece + the received pieces in rank order in binary32, round once, store: every rank gets the same bits.
// The epoch is a counter in the control block, advanced by the last CTA of a launch, so the same launch can be
// replayed from a CUDA graph.  Two parities suffice: a rank can start epoch e + 2 (overwriting the slots of e) only
// after every peer has pushed e + 1, i.e. has finished the launch that read the slots of e.
// A CTA waits only for the matching CTAs of its peers, and pushes before it waits, so ranks never deadlock on CTA
// scheduling; the grid is at most 128 CTAs (all resident on 148 SMs).
//
// With fewer GPUs than ranks the same kernel runs all ranks in ONE cooperative launch (blockIdx.y = rank, every
// rank's buffer on this device): ranks that wait on one another must not be separate launches on one GPU.
#include <stddef.h>
#include <string.h>

#include "token_common.cuh"

struct flh_b200_ar {
    int world, rank, device;
    size_t max_bytes, total_bytes;
    uint8_t *base;                 // this rank's buffer
    uint8_t *peer[8];              // every rank's buffer as seen from this device (peer[rank] = base)
    bool opened[8];                // mapped through IPC (to be closed)
};

namespace flh {
namespace {

constexpr int kArMaxWorld = 8;
constexpr int kArMaxCtas = 128;
constexpr int kArThreads = 512;
constexpr size_t kArCtrlBytes = 4096;
constexpr size_t kArFlagBytes = 2 * kArMaxWorld * kArMaxCtas * 4;     // 8 KiB
constexpr unsigned long long kArWaitNs = 2000000000ull;

struct ArCtrl { uint32_t epoch, done; int status[4]; };

struct ArRank {
    uint8_t *peer[kArMaxWorld];
    const void *x;
    void *out;                     // plain all-reduce: the sum; fused form: the residual stream (read, then residual + sum)
    uint8_t *q;                    // fused form: codes, scales, zero-points of the normalised rows
    __half *scale, *zero;
    int rank;
};
struct ArParams {
    ArRank r[kArMaxWorld];         // [0] only, unless all ranks run in one launch
    long nvec;                     // 16-byte pieces of the message
    size_t max_bytes;
    int world;
    int K;                         // fused form: row length (4096 or 8192)
    float eps, clip;
};

__device__ __forceinline__ uint32_t *ar_flag(uint8_t *base, int parity, int src, int cta) {
    return reinterpret_cast<uint32_t *>(base + kArCtrlBytes) + (parity * kArMaxWorld + src) * kArMaxCtas + cta;
}
__device__ __forceinline__ uint4 *ar_slot(uint8_t *base, size_t max_bytes, int world, int parity, int src) {
    return reinterpret_cast<uint4 *>(base + kArCtrlBytes + kArFlagBytes + ((size_t)parity * world + src) * max_bytes);
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const uint4 *p) {     // L2 only: the line was written by another GPU
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ar_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

template <bool BF16> __device__ __forceinline__ void acc8(float (&a)[8], const uint4 &v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (BF16) {
            a[2 * i] += __uint_as_float(w[i] << 16);
            a[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            a[2 * i] += f.x;
            a[2 * i + 1] += f.y;
        }
    }
}
template <bool BF16> __device__ __forceinline__ uint4 round8(const float (&a)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (BF16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        } else {
            const __half2 h = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Steps 1-3 for the pieces [v0, v1) of CTA `cta`: push them into every peer's slot of this rank, raise the flags, wait for the
// peers' flags (bounded).  Ends with a CTA barrier: after it the local slots of all ranks hold the pieces.
__device__ __forceinline__ void ar_exchange(const ArParams &p, const ArRank &me, ArCtrl *ctrl, uint32_t epoch, long v0, long v1, int cta) {
    const int rank = me.rank, world = p.world, tid = threadIdx.x, parity = (int)(epoch & 1u);
    uint8_t *base = me.peer[rank];
    const uint4 *x = reinterpret_cast<const uint4 *>(me.x);
    for (long v = v0 + tid; v < v1; v += kArThreads) {
        const uint4 val = x[v];
        for (int i = 1; i < world; ++i) {
            const int dst = (rank + i) % world;
            ar_slot(me.peer[dst], p.max_bytes, world, parity, rank)[v] = val;
        }
    }
    __syncthreads();
    if (tid < world && tid != rank) {                    // thread t handles peer t
        // the release orders the whole CTA's stores (made visible to this thread by the barrier) before the flag
        st_release_sys(ar_flag(me.peer[tid], parity, rank, cta), epoch);
        const uint32_t *f = ar_flag(base, parity, tid, cta);
        const unsigned long long t0 = ar_timer();
        uint32_t spins = 0;
        // poll with plain system-scope loads; one acquire load once the flag is up orders the slot reads after it
        while ((int)(ld_relaxed_sys(f) - epoch) < 0) {
            if ((++spins & 1023u) == 0 && ar_timer() - t0 > kArWaitNs) {
                if (atomicCAS(&ctrl->status[0], 0, 1) == 0) { ctrl->status[1] = tid; ctrl->status[2] = cta; ctrl->status[3] = (int)epoch; }
                break;
            }
        }
        (void)ld_acquire_sys(f);
    }
    __syncthreads();
}

// The last CTA of a launch to get here advances the call counter (every CTA read it at its start).
__device__ __forceinline__ void ar_finish(ArCtrl *ctrl, uint32_t epoch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&ctrl->done, 1u) == gridDim.x - 1) {
            ctrl->done = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(&ctrl->epoch) = epoch;
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArParams p) {
    const ArRank &me = p.r[blockIdx.y];
    const int rank = me.rank, world = p.world, cta = blockIdx.x, tid = threadIdx.x;
    uint8_t *base = me.peer[rank];
    ArCtrl *ctrl = reinterpret_cast<ArCtrl *>(base);
    // every CTA reads the counter before the last one advances it (that one first sees all the others done)
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&ctrl->epoch) + 1;
    const int parity = (int)(epoch & 1u);
    const long per = (p.nvec + gridDim.x - 1) / gridDim.x;
    const long v0 = (long)cta * per, v1 = v0 + per < p.nvec ? v0 + per : p.nvec;
    const uint4 *x = reinterpret_cast<const uint4 *>(me.x);

    ar_exchange(p, me, ctrl, epoch, v0, v1, cta);       // 1. push, 2. signal, 3. wait
    // 4. sum in rank order
    uint4 *out = reinterpret_cast<uint4 *>(me.out);
    for (long v = v0 + tid; v < v1; v += kArThreads) {
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < world; ++src)
            acc8<BF16>(a, src == rank ? x[v] : ld_cg_v4(ar_slot(base, p.max_bytes, world, parity, src) + v));
        out[v] = round8<BF16>(a);
    }
    ar_finish(ctrl, epoch);
}

template <bool BF16> __device__ __forceinline__ float cvt16(uint16_t h) {
    return BF16 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
}
template <bool BF16> __device__ __forceinline__ uint16_t rnd16(float f) {
    if (BF16) { const __nv_bfloat16 b = __float2bfloat16_rn(f); return *reinterpret_cast<const uint16_t *>(&b); }
    return __half_as_ushort(__float2half_rn(f));
}

// The all-reduce above FUSED with what follows a row-parallel linear in the decoder (modeling_llama.py: o_proj /
// down_proj -> residual add -> RMS-norm -> per-token asymmetric int4 quantiser of the next linear's input):
// CTA c owns token row c, so after step 3 it holds the whole row and goes on without another launch:
//   sum16 = round16(sum of the partial outputs, rank order, binary32);  x = round16(residual + sum16)  -> residual stream
//   y = round16(x * c),  c = 1 / sqrt(mean(x^2) + eps)   (norm weight 1)                                 -> not stored
//   scale, zero-point, codes of y as flh_b200_rmsnorm_quant_token_asym_i4 makes them                      -> q, scale, zero
// Bit for bit the chain all-reduce -> f16 add -> flh_b200_rmsnorm_quant_token_asym_i4: the sum of squares is taken the way
// that kernel takes it (K / 128 chains of 128 consecutive elements by fma, joined by xor-shuffles 16 .. 1 inside a warp,
// then warp 0 + warp 1), everything after it is element-wise or a min / max.
template <bool BF16>
__global__ void __launch_bounds__(kArThreads) allreduce_norm_quant_kernel(const ArParams p) {
    __shared__ __align__(16) uint16_t rowbuf[8192];
    __shared__ float red_sq[2], red_mm[2][kArThreads / 32], bc[3];
    const ArRank &me = p.r[blockIdx.y];
    const int rank = me.rank, world = p.world, cta = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint8_t *base = me.peer[rank];
    ArCtrl *ctrl = reinterpret_cast<ArCtrl *>(base);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&ctrl->epoch) + 1;
    const int parity = (int)(epoch & 1u);
    const int K = p.K, rv = K / 8;                       // 16-byte pieces per row
    const long v0 = (long)cta * rv;
    const uint4 *x = reinterpret_cast<const uint4 *>(me.x);

    ar_exchange(p, me, ctrl, epoch, v0, v0 + rv, cta);
    // the row: sum, residual add, into the residual stream and into shared memory
    uint4 *res = reinterpret_cast<uint4 *>(me.out);
    for (int i = tid; i < rv; i += kArThreads) {
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < world; ++src)
            acc8<BF16>(a, src == rank ? x[v0 + i] : ld_cg_v4(ar_slot(base, p.max_bytes, world, parity, src) + v0 + i));
        const uint4 s16 = round8<BF16>(a);
        const uint4 r = res[v0 + i];
        const uint32_t sw[4] = {s16.x, s16.y, s16.z, s16.w}, rw[4] = {r.x, r.y, r.z, r.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint16_t lo = rnd16<BF16>(__fadd_rn(cvt16<BF16>((uint16_t)rw[k]), cvt16<BF16>((uint16_t)sw[k])));
            const uint16_t hi = rnd16<BF16>(__fadd_rn(cvt16<BF16>((uint16_t)(rw[k] >> 16)), cvt16<BF16>((uint16_t)(sw[k] >> 16))));
            o[k] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
        const uint4 xn = make_uint4(o[0], o[1], o[2], o[3]);
        res[v0 + i] = xn;
        reinterpret_cast<uint4 *>(rowbuf)[i ^ ((i >> 4) & 7)] = xn;      // piece i of chain i / 16, swizzled: the chains' reads below do not collide
    }
    __syncthreads();
    // sum of squares: chain t adds elements [128 t, 128 t + 128) in order
    const int chains = K / 128;                          // 32 or 64: whole warps
    if (tid < chains) {
        float ssq = 0.0f;
#pragma unroll 4
        for (int cc = 0; cc < 16; ++cc) {
            const uint4 w4 = reinterpret_cast<const uint4 *>(rowbuf)[(tid * 16 + cc) ^ (tid & 7)];
            const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a = cvt16<BF16>((uint16_t)w[k]), b = cvt16<BF16>((uint16_t)(w[k] >> 16));
                ssq = __fmaf_rn(a, a, ssq);
                ssq = __fmaf_rn(b, b, ssq);
            }
        }
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) ssq = __fadd_rn(ssq, __shfl_xor_sync(0xffffffffu, ssq, sft));
        if (lane == 0) red_sq[warp] = ssq;
    }
    __syncthreads();
    if (tid == 0) {
        const float ssq = chains == 64 ? __fadd_rn(red_sq[0], red_sq[1]) : red_sq[0];
        bc[0] = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(ssq, 1.0f / (float)K), p.eps)));
    }
    __syncthreads();
    const float c = bc[0];
    // y = round16(x c) for this thread's elements (at most two pieces of eight), row minimum and maximum
    float y[16];
    float vmin = 0.0f, vmax = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = tid + j * kArThreads;
        if (i < rv) {
            const uint4 w4 = reinterpret_cast<const uint4 *>(rowbuf)[i ^ ((i >> 4) & 7)];
            const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint16_t h = (uint16_t)(w[e >> 1] >> ((e & 1) * 16));
                const float v = cvt16<BF16>(rnd16<BF16>(__fmul_rn(cvt16<BF16>(h), c)));
                y[j * 8 + e] = v;
                vmin = fminf(vmin, v); vmax = fmaxf(vmax, v);
            }
        }
    }
    vmin = warp_min(vmin); vmax = warp_max(vmax);
    if (lane == 0) { red_mm[0][warp] = vmin; red_mm[1][warp] = vmax; }
    __syncthreads();
    if (tid == 0) {
        float a = red_mm[0][0], b = red_mm[1][0];
        for (int w = 1; w < kArThreads / 32; ++w) { a = fminf(a, red_mm[0][w]); b = fmaxf(b, red_mm[1][w]); }
        bc[1] = a; bc[2] = b;
    }
    __syncthreads();
    const TokenRowParams rp = token_row_params(bc[1], bc[2], p.clip, 1.0f);
    if (tid == 0) { me.scale[cta] = rp.scale; me.zero[cta] = __float2half_rn(rp.zero); }
    const float lo = -rp.zero, hi = 15.0f - rp.zero;
    const int zi = (int)rp.zero;
    uint32_t *qrow = reinterpret_cast<uint32_t *>(me.q + (long)cta * (K / 2));
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = tid + j * kArThreads;
        if (i < rv) {
            uint32_t w = 0;
#pragma unroll
            for (int e = 7; e >= 0; --e) {
                float r = __fmul_rn(y[j * 8 + e], rp.rd);
                if (rp.clamp) r = fmaxf(fminf(r, hi), lo);
                w = w * 16u + (uint32_t)((int)rintf(r) + zi);
            }
            qrow[i] = w;
        }
    }
    ar_finish(ctrl, epoch);
}

int ar_grid(long nvec) {
    long g = (nvec + 2 * kArThreads - 1) / (2 * kArThreads);      // two 16-byte pieces per thread
    return (int)(g < 1 ? 1 : g > kArMaxCtas ? kArMaxCtas : g);
}

int ar_check(const flh_b200_ar *h, const void *x, const void *out, long n) {
    FLH_REQUIRE(h && x && out, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(n > 0 && n % 8 == 0, FLH_B200_EINVAL, "n=%ld must be a positive multiple of 8 elements", n);
    FLH_REQUIRE((size_t)n * 2 <= h->max_bytes, FLH_B200_EINVAL, "message of %ld bytes exceeds the %zu bytes this all-reduce was made for", n * 2, h->max_bytes);
    FLH_REQUIRE(aligned16(x) && aligned16(out), FLH_B200_EALIGN, "x and out must be 16-byte aligned");
    for (int r = 0; r < h->world; ++r) FLH_REQUIRE(h->peer[r], FLH_B200_EINVAL, "the buffer of rank %d is not attached", r);
    return 0;
}

}  // namespace
}  // namespace flh

using namespace flh;

extern "C" {

int flh_b200_ar_create(int world, int rank, size_t max_bytes, flh_b200_ar **out) {
    FLH_REQUIRE(out, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(world >= 1 && world <= kArMaxWorld && rank >= 0 && rank < world, FLH_B200_EINVAL, "bad world=%d rank=%d (at most %d ranks)", world, rank, kArMaxWorld);
    FLH_REQUIRE(max_bytes >= 16 && max_bytes % 16 == 0 && max_bytes <= ((size_t)64 << 20), FLH_B200_EINVAL, "max_bytes=%zu must be a multiple of 16, at most 64 MiB", max_bytes);
    flh_b200_ar *h = new flh_b200_ar();
    h->world = world; h->rank = rank; h->max_bytes = max_bytes;
    h->total_bytes = kArCtrlBytes + kArFlagBytes + 2 * (size_t)world * max_bytes;
    for (int r = 0; r < 8; ++r) { h->peer[r] = nullptr; h->opened[r] = false; }
    cudaError_t e = cudaGetDevice(&h->device);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&h->base), h->total_bytes);
    if (e == cudaSuccess) e = cudaMemset(h->base, 0, kArCtrlBytes + kArFlagBytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { delete h; return cuda_status(e, "all-reduce buffer"); }
    h->peer[rank] = h->base;
    *out = h;
    return 0;
}

int flh_b200_ar_export(flh_b200_ar *h, void *ipc64) {
    FLH_REQUIRE(h && ipc64, FLH_B200_EINVAL, "null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    return cuda_status(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(ipc64), h->base), "IPC export");
}

int flh_b200_ar_import(flh_b200_ar *h, int peer, const void *ipc64) {
    FLH_REQUIRE(h && ipc64, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(peer >= 0 && peer < h->world && peer != h->rank && !h->peer[peer], FLH_B200_EINVAL, "bad or already attached peer %d", peer);
    cudaIpcMemHandle_t m;
    memcpy(&m, ipc64, sizeof(m));
    void *ptr = nullptr;
    const int rc = cuda_status(cudaIpcOpenMemHandle(&ptr, m, cudaIpcMemLazyEnablePeerAccess), "IPC import");
    if (rc) return rc;
    h->peer[peer] = static_cast<uint8_t *>(ptr);
    h->opened[peer] = true;
    return 0;
}

int flh_b200_ar_attach(flh_b200_ar *h, int peer, flh_b200_ar *other) {
    FLH_REQUIRE(h && other, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(peer >= 0 && peer < h->world && peer != h->rank && !h->peer[peer], FLH_B200_EINVAL, "bad or already attached peer %d", peer);
    FLH_REQUIRE(other->rank == peer && other->world == h->world && other->max_bytes == h->max_bytes, FLH_B200_EINVAL, "rank %d's all-reduce does not match", peer);
    if (other->device != h->device) {
        int can = 0;
        cudaError_t e = cudaDeviceCanAccessPeer(&can, h->device, other->device);
        if (e != cudaSuccess) return cuda_status(e, "peer query");
        FLH_REQUIRE(can, FLH_B200_EUNSUPPORTED, "device %d cannot map memory of device %d", h->device, other->device);
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(h->device);
        e = cudaDeviceEnablePeerAccess(other->device, 0);
        cudaSetDevice(cur);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
        if (e != cudaSuccess) return cuda_status(e, "peer access");
    }
    h->peer[peer] = other->base;
    return 0;
}

int flh_b200_allreduce(flh_b200_ar *h, const void *x, void *out, long n, int dtype, void *stream) {
    if (const int rc = ar_check(h, x, out, n)) return rc;
    FLH_REQUIRE(dtype == FLH_B200_F16 || dtype == FLH_B200_BF16, FLH_B200_EINVAL, "dtype must be F16 or BF16");
    ArParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < h->world; ++r) p.r[0].peer[r] = h->peer[r];
    p.r[0].x = x; p.r[0].out = out; p.r[0].rank = h->rank;
    p.nvec = n / 8; p.max_bytes = h->max_bytes; p.world = h->world;
    const dim3 grid(ar_grid(p.nvec), 1);
    if (dtype == FLH_B200_BF16) allreduce_oneshot_kernel<true><<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    else allreduce_oneshot_kernel<false><<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cuda_status(cudaGetLastError(), "all-reduce launch");
}

int flh_b200_allreduce_ranks(flh_b200_ar *const *hs, int world, const void *const *xs, void *const *outs, long n, int dtype, void *stream) {
    FLH_REQUIRE(hs && xs && outs && world >= 1 && world <= kArMaxWorld, FLH_B200_EINVAL, "bad arguments");
    FLH_REQUIRE(dtype == FLH_B200_F16 || dtype == FLH_B200_BF16, FLH_B200_EINVAL, "dtype must be F16 or BF16");
    ArParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < world; ++r) {
        FLH_REQUIRE(hs[r] && hs[r]->world == world && hs[r]->rank == r && hs[r]->device == hs[0]->device, FLH_B200_EINVAL,
                    "rank %d: all ranks of a single launch live on one device, in rank order", r);
        if (const int rc = ar_check(hs[r], xs[r], outs[r], n)) return rc;
        for (int q = 0; q < world; ++q) p.r[r].peer[q] = hs[r]->peer[q];
        p.r[r].x = xs[r]; p.r[r].out = outs[r]; p.r[r].rank = r;
    }
    p.nvec = n / 8; p.max_bytes = hs[0]->max_bytes; p.world = world;
    int gx = ar_grid(p.nvec);
    if (gx * world > kNumSMs) gx = kNumSMs / world;               // every CTA of every rank resident at once
    const dim3 grid(gx, world);
    void *args[] = {&p};
    const void *fn = dtype == FLH_B200_BF16 ? reinterpret_cast<const void *>(allreduce_oneshot_kernel<true>)
                                            : reinterpret_cast<const void *>(allreduce_oneshot_kernel<false>);
    return cuda_status(cudaLaunchCooperativeKernel(fn, grid, dim3(kArThreads), args, 0, static_cast<cudaStream_t>(stream)), "all-reduce launch (all ranks)");
}

static int ar_fused_check(const flh_b200_ar *h, const void *y, const void *residual, long M, long K, int dtype, float eps, float clip,
                          const void *q, const void *scale, const void *zero) {
    FLH_REQUIRE(dtype == FLH_B200_F16 || dtype == FLH_B200_BF16, FLH_B200_EINVAL, "dtype must be F16 or BF16");
    FLH_REQUIRE(K == 4096 || K == 8192, FLH_B200_EUNSUPPORTED, "the fused form serves K = 4096 and 8192 (got %ld)", K);
    FLH_REQUIRE(M >= 1 && M <= kArMaxCtas, FLH_B200_EINVAL, "M=%ld: one CTA per token row, at most %d rows", M, kArMaxCtas);
    FLH_REQUIRE(eps >= 0.0f && clip > 0.0f && clip <= 1.0f, FLH_B200_EINVAL, "eps must be >= 0 and clip in (0, 1]");
    FLH_REQUIRE(residual && q && scale && zero, FLH_B200_EINVAL, "null pointer");
    FLH_REQUIRE(aligned16(q), FLH_B200_EALIGN, "q must be 16-byte aligned");
    return ar_check(h, y, residual, M * K);
}

int flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4(flh_b200_ar *h, const void *y, void *residual, long M, long K, int dtype,
                                                       float eps, float clip, uint8_t *q, void *scale, void *zero, void *stream) {
    if (const int rc = ar_fused_check(h, y, residual, M, K, dtype, eps, clip, q, scale, zero)) return rc;
    ArParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < h->world; ++r) p.r[0].peer[r] = h->peer[r];
    p.r[0].x = y; p.r[0].out = residual; p.r[0].q = q; p.r[0].scale = static_cast<__half *>(scale); p.r[0].zero = static_cast<__half *>(zero);
    p.r[0].rank = h->rank;
    p.nvec = M * K / 8; p.max_bytes = h->max_bytes; p.world = h->world; p.K = (int)K; p.eps = eps; p.clip = clip;
    const dim3 grid((unsigned)M, 1);
    if (dtype == FLH_B200_BF16) allreduce_norm_quant_kernel<true><<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    else allreduce_norm_quant_kernel<false><<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cuda_status(cudaGetLastError(), "fused all-reduce launch");
}

int flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4_ranks(flh_b200_ar *const *hs, int world, const void *const *ys, void *const *residuals,
                                                             long M, long K, int dtype, float eps, float clip, uint8_t *const *qs,
                                                             void *const *scales, void *const *zeros, void *stream) {
    FLH_REQUIRE(hs && ys && residuals && qs && scales && zeros && world >= 1 && world <= kArMaxWorld, FLH_B200_EINVAL, "bad arguments");
    FLH_REQUIRE(M * world <= kNumSMs, FLH_B200_EINVAL, "M * world = %ld CTAs must all be resident (at most %d)", M * world, kNumSMs);
    ArParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < world; ++r) {
        FLH_REQUIRE(hs[r] && hs[r]->world == world && hs[r]->rank == r && hs[r]->device == hs[0]->device, FLH_B200_EINVAL,
                    "rank %d: all ranks of a single launch live on one device, in rank order", r);
        if (const int rc = ar_fused_check(hs[r], ys[r], residuals[r], M, K, dtype, eps, clip, qs[r], scales[r], zeros[r])) return rc;
        for (int q = 0; q < world; ++q) p.r[r].peer[q] = hs[r]->peer[q];
        p.r[r].x = ys[r]; p.r[r].out = residuals[r]; p.r[r].q = qs[r];
        p.r[r].scale = static_cast<__half *>(scales[r]); p.r[r].zero = static_cast<__half *>(zeros[r]); p.r[r].rank = r;
    }
    p.nvec = M * K / 8; p.max_bytes = hs[0]->max_bytes; p.world = world; p.K = (int)K; p.eps = eps; p.clip = clip;
    const dim3 grid((unsigned)M, world);
    void *args[] = {&p};
    const void *fn = dtype == FLH_B200_BF16 ? reinterpret_cast<const void *>(allreduce_norm_quant_kernel<true>)
                                            : reinterpret_cast<const void *>(allreduce_norm_quant_kernel<false>);
    return cuda_status(cudaLaunchCooperativeKernel(fn, grid, dim3(kArThreads), args, 0, static_cast<cudaStream_t>(stream)), "fused all-reduce launch (all ranks)");
}

int flh_b200_ar_status(flh_b200_ar *h, int *out4) {
    FLH_REQUIRE(h && out4, FLH_B200_EINVAL, "null pointer");
    return cuda_status(cudaMemcpy(out4, h->base + offsetof(ArCtrl, status), 4 * sizeof(int), cudaMemcpyDeviceToHost), "all-reduce status");
}

int flh_b200_ar_destroy(flh_b200_ar *h) {
    if (!h) return 0;
    int rc = 0;
    for (int r = 0; r < h->world; ++r)
        if (h->opened[r] && h->peer[r]) rc |= cuda_status(cudaIpcCloseMemHandle(h->peer[r]), "IPC close");
    rc |= cuda_status(cudaFree(h->base), "all-reduce buffer free");
    delete h;
    return rc;
}

}  // extern "C"
