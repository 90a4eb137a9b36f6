// fp32 GEMM at near-fp32 accuracy on the tf32 tensor-core path (see tf32_gemm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

// Split operand layout: [rows, 3 * kp] fp32 with kp = K rounded up to 32; role A rows hold [hi | hi | lo],
// role B rows hold [hi | lo | hi], so that one K-major product over 3 * kp sums hi*hi + hi*lo + lo*hi.
inline int64_t tf32_split_kp(int64_t K) { return (K + 31) / 32 * 32; }

// src: [batch, R, C] fp32 (row stride ld_src, batch stride stride_src).  transpose = 0: operand rows = src rows,
// K = C.  transpose = 1: operand rows = src columns, K = R.  dst: [batch, rows, 3 * kp] contiguous.
cudaError_t launch_tf32_split(const float* src, int64_t ld_src, int64_t stride_src, int R, int C, int batch, int transpose,
                              int role_b, float* dst, cudaStream_t stream);

// C[b] (fp32 [M, N], row stride ldc) = alpha * A3[b] * B3[b]^T over the split operands; status as in ns_gemm.
cudaError_t launch_tf32_gemm(const float* A3, const float* B3, int M, int N, int K, int batch, float alpha, float* C,
                             int64_t ldc, int64_t strideC, int* status, cudaStream_t stream);

}  // namespace hb
