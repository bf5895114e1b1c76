// C entry points of the tcgen05 GEMM family (see gemm_tcgen05.cu for the operand conventions).
#pragma once
#include <stdint.h>

#define GEMM_EPI_BF16 0     // C is bf16 [M, N], overwritten
#define GEMM_EPI_F32 1      // C is fp32 [M, N], overwritten
#define GEMM_EPI_F32_ACC 2  // C is fp32 [M, N], C += A*B^T  (weight-gradient accumulation)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on a successful launch, a negative code on a rejected argument or launch error.
// `status` points to a device int32 that the kernel leaves at 0 unless one of its bounded
// waits ran out (codes in common.cuh).  tile_n: 0 = choose; 128 or 256 = 1-CTA kernel with that tile width;
// 2 = the CTA-pair kernel (256x256 tile per two SMs, gemm_tcgen05_2cta.cu).
int hsb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                  int a_mn_major, int b_mn_major, int epi, int tile_n, int* status, void* stream, int num_sms);

int hsb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                       int a_mn_major, int b_mn_major, int epi, int* status, void* stream, int num_sms);

#ifdef __cplusplus
}
#endif
