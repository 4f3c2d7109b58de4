// C launchers exported by the CUDA sources (one declaration per entry point).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {
int vb_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                 long long ldb, long long ldd, int a_mn, int b_mn, int out_f32, int accumulate, int max_ctas,
                 cudaStream_t stream);
int vb_gemm_status();
}
