// fp32 GEMM at near-fp32 accuracy on the tf32 tensor-core path, with fused epilogues (see tf32_gemm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

// Split operand layout: [rows, 2 * kp] fp32 with kp = K rounded up to 32; a row holds [hi | lo] with
// hi = tf32(x), lo = tf32(x - hi); columns [K, kp) of both halves are zero.  The same buffer serves as the A or
// the B operand of a product: the kernel walks A as (hi, hi, lo) and B as (hi, lo, hi) along K.
inline int64_t tf32_split_kp(int64_t K) { return (K + 31) / 32 * 32; }

// src: [batch, R, C] fp32 (row stride ld_src, batch stride stride_src).  Writes either or both of
//   dst_same : [batch, R, 2 * kp(C)]  operand rows = src rows,    K = C
//   dst_trans: [batch, C, 2 * kp(R)]  operand rows = src columns, K = R
// (null = not wanted).  One pass over the source.
cudaError_t launch_tf32_split(const float* src, int64_t ld_src, int64_t stride_src, int R, int C, int batch, float* dst_same,
                              float* dst_trans, cudaStream_t stream);

enum Tf32EpilogueMode : int {
  kEpiStore = 0,    // out = alpha * acc
  kEpiLerp = 1,     // C <- C + (alpha * acc - C) * w            (statistics update, in place on C)
  kEpiAdam = 2,     // x = alpha*acc; m <- lerp(m, x, 1-b1); v <- lerp(v, x*x, 1-b2); out = m / max(sqrt(v), eps)
  kEpiLaProp = 3,   // x = alpha*acc; v <- lerp(v, x*x, 1-b2); m <- lerp(m, x / max(sqrt(v), eps), 1-b1); out = m
  kEpiAdd = 4,      // C <- C + alpha * acc                       (Schur complements and solve updates, in place on C)
};

// What the epilogue does with the finished [M, N] tile values.  Any of C / S may be null.
struct Tf32Epilogue {
  int mode;
  float alpha;
  float w;                 // kEpiLerp weight
  float b1, b2, eps;       // kEpiAdam / kEpiLaProp: coefficients actually applied (already debiased)
  float* C;                // fp32 output [batch, M, ldc] (row-major); for kEpiLerp also the input
  int64_t ldc, strideC;
  float* S;                // split-operand output for a following product (layout above), or null
  int64_t kpS, strideS;    // kp of that operand's K (N if !s_transposed, M if s_transposed), batch stride in floats
  int s_transposed;        // 0: operand rows = output rows, K = N; 1: operand rows = output columns, K = M
  float* m;                // kEpiAdam / kEpiLaProp state, fp32 [batch, M, N] contiguous
  float* v;
  int tri;                 // A[i, k] = 0 for k < i and B[j, k] = 0 for k > j (an upper-triangular matrix times an upper-
                           // triangular matrix, M == N == K): a tile only walks the K range where both are non-zero,
                           // tiles below the diagonal are stored as zeros without a product
  int symmetric;           // A2 == B2 (so M == N and the product is symmetric): only tiles on or above the diagonal are
                           // computed and each is also stored transposed.  kEpiStore / kEpiLerp / kEpiAdd with C set and S null.
};

// out[b] = epilogue(A[b] * B[b]^T) over split operands A2: [batch, M, 2 * kp(K)], B2: [batch, N, 2 * kp(K)].
// `status` is set to 1 if a bounded wait expired (the CTA then drains, frees its tensor memory and returns).
cudaError_t launch_tf32_gemm(const float* A2, const float* B2, int M, int N, int K, int batch, const Tf32Epilogue& E,
                             int* status, cudaStream_t stream);

// Tile choice of launch_tf32_gemm: 0 = by problem size, 128 or 256 = forced.
int tf32_gemm_tile_override();
void set_tf32_gemm_tile_override(int tile);

}  // namespace hb
