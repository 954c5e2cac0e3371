// C ABI of libinnova_cuda.so. Every entry point takes raw device pointers and a CUDA stream
// (as void*), returns 0 on success or a negative code, and never synchronises the device.
// The Python layer (innova_b200/_native.py) binds these with ctypes.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// GEMM epilogues (inv_gemm_bf16)
enum {
  EPI_NONE = 0,    // C = alpha*acc (+ bias)
  EPI_GELU = 1,    // aux_out = alpha*acc + bias (optional); C = gelu(aux_out)
  EPI_DGELU = 2,   // C = alpha*acc * gelu'(aux_in)
  EPI_ADD = 3,     // C = alpha*acc + bias + aux_in   (residual add; aux_in may alias C)
  EPI_ATOMIC = 4,  // C(fp32) += alpha*acc            (split-K / gradient accumulation)
  EPI_GELU_DG = 5, // x = alpha*acc + bias; aux_out = gelu'(x); C = gelu(x)   (the backward then needs one multiply: EPI_MUL)
  EPI_MUL = 6,     // C = alpha*acc * aux_in
};
// epilogues that write a second bf16 output / read a second bf16 operand of C's shape
#define INV_EPI_WRITES_AUX(e) ((e) == EPI_GELU || (e) == EPI_GELU_DG)
#define INV_EPI_READS_AUX(e) ((e) == EPI_DGELU || (e) == EPI_ADD || (e) == EPI_MUL)

// C[M,N] = op(A)[M,K] * op(B)[N,K]^T. a_mn/b_mn = 0: operand stored [rows, K] row-major;
// = 1: operand stored [K, rows] row-major. lda/ldb/ldc/ld_aux in elements.
int inv_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn,
                  int epilogue, const void* bias, const void* aux_in, int ld_aux, void* aux_out, int c_f32, int split_k,
                  float alpha, int* status, void* stream, int kernel_select);

#ifdef __cplusplus
}
#endif
