// C-linkage doors onto the reference's own CUDA launchers, so that the tests can run the
// reference kernels (compiled from the FLH checkout, never copied) next to the B200 kernels.
// TEST INFRASTRUCTURE: built into oracle/_ref/libflh_ref.so by oracle/Makefile, loaded only by tests
// and the benchmark's comparison leg.
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

using Int4Storage = uint8_t;
// flh/kernels/had_and_quant.h:19-24, flh/kernels/quant_and_pack.h:19-24 (C++ linkage in the reference)
void had_and_quant_host(const half *data, Int4Storage *quantized_data, half *scales, uint32_t M);
void quant_and_pack_host(const half *data, Int4Storage *quantized_data, half *scales, uint32_t M);
// flh/kernels/gemm_and_dequant_i4.cu:471-480
extern "C" void flhDenseLayerGEMM_i4_o16(const uint8_t *A, const uint8_t *B, const half *A_scale,
                                         const half *B_scale, half *D, size_t M, size_t N, size_t K);

extern "C" {
void flh_ref_had_and_quant(const void *x, void *q, void *s, unsigned rows) {
    had_and_quant_host(static_cast<const half *>(x), static_cast<Int4Storage *>(q), static_cast<half *>(s), rows);
}
void flh_ref_quant_and_pack(const void *x, void *q, void *s, unsigned rows) {
    quant_and_pack_host(static_cast<const half *>(x), static_cast<Int4Storage *>(q), static_cast<half *>(s), rows);
}
void flh_ref_gemm_i4_o16(const void *A, const void *B, const void *sa, const void *sb, void *D, size_t M, size_t N, size_t K) {
    flhDenseLayerGEMM_i4_o16(static_cast<const uint8_t *>(A), static_cast<const uint8_t *>(B),
                             static_cast<const half *>(sa), static_cast<const half *>(sb), static_cast<half *>(D), M, N, K);
}
int flh_ref_sync(void) { return (int)cudaDeviceSynchronize(); }
int flh_ref_last_error(void) { return (int)cudaGetLastError(); }
}
