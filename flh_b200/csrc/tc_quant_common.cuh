// Pieces of the tensor-core token quantiser (quant_token_tc.cu): descriptors, the TMA row load,
// packed binary32 helpers and the construction of the +-1 operand in shared memory.
#pragma once
#include "tc_common.cuh"

namespace flh {

__device__ __forceinline__ uint64_t umma_desc_tc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
    uint32_t r;
    asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}


// A = G (or diag(G, G) when two token rows share an MMA: R == 2) as a K-major tcgen05 operand with the 128-byte swizzle:
// element (m, k) lies in K atom kb = k / 64 at (kb * Mtot / 8 + m / 8) * 1024, row m % 8 of 128 bytes, 16-byte chunk
// ((k % 64) / 8) ^ (m % 8).  G[p'][p] = S[a'][a] * (-1)^popc(b' & b) with p = a * B + b (B a power of two, S the kfac x kfac
// factor given as bit rows, 1 = negative): per row the signs of the factor come as one bit row of the table (staged in
// shared memory at `sgn` first), the Sylvester part is a parity.  Contains a __syncthreads(): called by the whole CTA.
__device__ __forceinline__ void build_sign_operand(uint8_t *sm, uint32_t *sgn, const uint32_t *sign_bits, int kfac, int words, int P, int B,
                                                   int R, int Kdim, int Mtot, bool bf16, int tid, int nthreads) {
    if (sign_bits)
        for (int i = tid; i < kfac * words; i += nthreads) sgn[i] = sign_bits[i];
    __syncthreads();
    const int katoms = (Kdim + 63) >> 6;
    const int cpr = katoms * 8;                                         // 16-byte chunks per row of A
    const int chunks = Mtot * cpr;
    const int logB = 31 - __clz(B);
    const uint32_t one = bf16 ? 0x3F80u : 0x3C00u;
    for (int i = tid; i < chunks; i += nthreads) {
        const int m = i / cpr, kc = i - m * cpr;                        // row of A, 16-byte chunk along K
        const int pr = R == 2 ? (m & 63) : m, blk_m = R == 2 ? (m >> 6) : 0;
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        const int k0 = kc * 8;
        const int pc0 = R == 2 ? (k0 & 63) : k0, blk_k = R == 2 ? (k0 >> 6) : 0;
        if (pr < P && blk_k == blk_m && pc0 < P && k0 < Kdim) {
            const int ar = pr >> logB, br = pr & (B - 1);
            const uint32_t *row = sgn + ar * words;
            uint32_t neg8;                                              // bit e: the sign of element pc0 + e
            if (B >= 8) {
                // the eight columns share one column of the factor; their Sylvester bits are b0 .. b0 + 7 with b0 a multiple
                // of 8, so the parity splits into a common part and the 8-point Walsh row of br & 7
                const int ac = pc0 >> logB, bc0 = pc0 & (B - 1);
                uint32_t common = __popc((uint32_t)(br & bc0)) & 1u;
                if (sign_bits) common ^= (row[ac >> 5] >> (ac & 31)) & 1u;
                // Walsh rows of order 8 as bit masks: bit e of row r = parity(r & e)
                const uint32_t walsh8 = (0x00u) | (0xAAu << 8) | (0xCCu << 16) | (0x66u << 24);
                const uint32_t walsh8b = (0xF0u) | (0x5Au << 8) | (0x3Cu << 16) | (0x96u << 24);
                const int r7 = br & 7;
                const uint32_t wr = ((r7 < 4 ? walsh8 : walsh8b) >> (8 * (r7 & 3))) & 0xFFu;
                neg8 = wr ^ (common ? 0xFFu : 0u);
            } else if (B == 1) {
                neg8 = sign_bits ? (row[pc0 >> 5] >> (pc0 & 31)) & 0xFFu : 0u;   // eight neighbouring bits of the factor's row
            } else {
                neg8 = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int pc = pc0 + e, ac = pc >> logB, bc = pc & (B - 1);
                    uint32_t neg = __popc((uint32_t)(br & bc)) & 1u;
                    if (sign_bits && ac < kfac) neg ^= (row[ac >> 5] >> (ac & 31)) & 1u;
                    neg8 |= neg << e;
                }
            }
            const int nvalid = P - pc0 < 8 ? P - pc0 : 8;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (e < nvalid) w[e >> 1] |= (one | (((neg8 >> e) & 1u) << 15)) << (16 * (e & 1));
        }
        const int kb = kc >> 3, cc = kc & 7;
        *reinterpret_cast<uint4 *>(sm + (kb * (Mtot >> 3) + (m >> 3)) * 1024 + (m & 7) * 128 + ((cc ^ (m & 7)) << 4)) =
            make_uint4(w[0], w[1], w[2], w[3]);
    }
}

}  // namespace flh
