// Shared device/host helpers for the flh_b200 kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/flh_b200.h"

namespace flh {

constexpr int kNumSMs = 148;   // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// ---- error plumbing -----------------------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);
int cuda_status(cudaError_t e, const char *what);   // 0 or -(int)e, message recorded

#define FLH_REQUIRE(cond, code, ...)                 \
    do {                                             \
        if (!(cond)) return ::flh::fail(code, __VA_ARGS__); \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- small PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Packed binary32 pairs (sm_100): two IEEE adds / fused multiply-adds per instruction.
// Written as plain integer arithmetic (not an opaque asm mov) so that the compiler can keep the two
// halves in an aligned register pair without moving them.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    return (static_cast<uint64_t>(__float_as_uint(hi)) << 32) | __float_as_uint(lo);
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    lo = __uint_as_float(static_cast<uint32_t>(v));
    hi = __uint_as_float(static_cast<uint32_t>(v >> 32));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// a - b as fma(b, -1, a): the product is exact, so this is the IEEE difference.
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t r;
    const uint64_t neg1 = 0xBF800000BF800000ull;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(b), "l"(neg1), "l"(a));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// 16-byte global load that may stay in L1 (used where one thread reads a whole 128-byte line
// with eight such loads).
__device__ __forceinline__ uint4 ldg_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace flh
