// One column block of GPTQ's quantise-and-compensate sweep (the inner loop of FLHGPTQ.fasterquant,
// flh/nn/gptq.py:198-232), as one launch instead of ~10 small launches per column.
//
// Within a block of up to 128 columns the sweep is sequential in the column index but independent across weight
// rows, so a warp owns one row: lane l keeps columns l, l + 32, l + 64, l + 96 in registers, the block of the
// inverse-Hessian Cholesky factor sits in shared memory, and step i is one shuffle (column i's current value),
// the quantiser, err = (w - q) / d_i and  w_j = w_j - err * Hinv[i][j]  for the columns j > i the lane holds.
// The arithmetic is the reference's, operation for operation in binary32 (a rounded product followed by a rounded
// subtraction, as its rank-1 matmul and in-place subtraction do; true division; round-half-even), so the block's
// Q and Err match a CPU restatement bit for bit.  The update of the columns right of the block,
// W[:, i2:] -= Err @ Hinv[i1:i2, i2:], is a plain GEMM and stays with the caller.
#include "common.cuh"

namespace flh {
namespace {

constexpr int kRowsPerCta = 16;     // warps per CTA

struct GptqParams {
    const float *W, *Hinv, *scale, *zero;
    const int *group_of_col;
    float *Q, *Err;
    long ldw, ldh, lds, ldq, rows;
    int count, maxq, sym;
    float clip_ratio;
};

__global__ void __launch_bounds__(32 * kRowsPerCta)
gptq_block_kernel(const GptqParams p) {
    extern __shared__ float hs[];                       // [count][count], then group_of_col as int[count]
    const int count = p.count;
    int *gi = reinterpret_cast<int *>(hs + count * count);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int idx = tid; idx < count * count; idx += blockDim.x) {
        const int r = idx / count, c = idx - r * count;
        hs[idx] = c >= r ? p.Hinv[(long)r * p.ldh + c] : 0.0f;
    }
    for (int c = tid; c < count; c += blockDim.x) gi[c] = p.group_of_col[c];
    __syncthreads();
    const long row = (long)blockIdx.x * kRowsPerCta + warp;
    if (row >= p.rows) return;

    float w[4], qv[4], ev[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int j = 32 * t + lane;
        w[t] = j < count ? p.W[row * p.ldw + j] : 0.0f;
        qv[t] = 0.0f; ev[t] = 0.0f;
    }
    const float *srow = p.scale + row * p.lds;
    const float *zrow = p.zero ? p.zero + row * p.lds : nullptr;
    const float fmaxq = (float)p.maxq;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll 4
        for (int l = 0; l < 32; ++l) {
            const int i = 32 * s + l;
            if (i >= count) break;
            const float wi = __shfl_sync(0xffffffffu, w[s], l);
            const float sc = srow[gi[i]];
            float x = wi;
            if (p.clip_ratio < 1.0f) {
                const float cv = __fmul_rn(__fmul_rn(sc, fmaxq), p.clip_ratio);
                x = fminf(fmaxf(x, -cv), cv);
            }
            float out;
            if (p.sym) {
                const float q = fminf(fmaxf(rintf(__fdiv_rn(x, sc)), -(fmaxq + 1.0f)), fmaxq);
                out = __fmul_rn(sc, q);
            } else {
                const float zr = zrow[gi[i]];
                const float q = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(x, sc), zr)), 0.0f), fmaxq);
                out = __fmul_rn(sc, __fsub_rn(q, zr));
            }
            const float err = __fdiv_rn(__fsub_rn(wi, out), hs[i * count + i]);
            if (lane == l) { qv[s] = out; ev[s] = err; }
            const float *hrow = hs + i * count;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int j = 32 * t + lane;
                if (j > i && j < count) w[t] = __fsub_rn(w[t], __fmul_rn(err, hrow[j]));
            }
        }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int j = 32 * t + lane;
        if (j < count) {
            p.Q[row * p.ldq + j] = qv[t];
            p.Err[row * count + j] = ev[t];
        }
    }
}

}  // namespace

int launch_gptq_block(const float *W, long ldw, const float *Hinv, long ldh, const float *scale, const float *zero,
                      long lds, const int *group_of_col, long rows, int count, int maxq, int sym, float clip_ratio,
                      float *Q, long ldq, float *Err, cudaStream_t stream) {
    GptqParams p;
    p.W = W; p.Hinv = Hinv; p.scale = scale; p.zero = zero; p.group_of_col = group_of_col;
    p.Q = Q; p.Err = Err;
    p.ldw = ldw; p.ldh = ldh; p.lds = lds; p.ldq = ldq; p.rows = rows;
    p.count = count; p.maxq = maxq; p.sym = sym; p.clip_ratio = clip_ratio;
    const int smem = count * count * 4 + count * 4;
    cudaError_t e = cudaFuncSetAttribute(gptq_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e, "gptq_block attribute");
    const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
    gptq_block_kernel<<<grid, 32 * kRowsPerCta, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "gptq_block launch");
}

}  // namespace flh
