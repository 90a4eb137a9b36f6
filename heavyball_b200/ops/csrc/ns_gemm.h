// Host-visible declarations for the Newton–Schulz GEMM family (ns_gemm.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

enum GemmMode : int { kModeGram = 0, kModePoly = 1, kModeApply = 2 };

// D[M, N] = A[M, K] * B[N, K]^T per batch entry; all leading dimensions and strides in elements.
struct GemmParams {
  int M, N, K, batch;
  int mode;
  int symmetric;            // compute tiles with tile_n >= tile_m only and mirror them through CT
  int same_operand;         // A and B are the same matrix (set by the launcher): diagonal tiles load it once
  __nv_bfloat16* C;         // bf16 output [M, N] (may be null)
  int64_t ldc, strideC;
  __nv_bfloat16* CT;        // bf16 transposed output [N, M] (may be null; equals C for symmetric results)
  int64_t ldct, strideCT;
  float* F;                 // fp32 output scaled by f_scale, [M, N] or [N, M] when f_transposed (may be null)
  int64_t ldf, strideF;
  int f_transposed;
  float f_scale;
  const __nv_bfloat16* S;   // poly mode: epilogue operand, same shape as the output
  int64_t lds, strideS;
  float ca, cb, cc;         // poly mode: D <- cc * acc + cb * S + ca * I
  int* status;              // set to 1 if a bounded wait expired
};

// Tile choice of launch_ns_gemm: 0 = by problem size (default), 128 / 256 = force that output tile (tests, tuning).
int ns_gemm_tile_override();
void set_ns_gemm_tile_override(int tile);

cudaError_t launch_ns_gemm(const void* A, int64_t lda, int64_t strideA, const void* B, int64_t ldb, int64_t strideB,
                           const GemmParams& P, cudaStream_t stream);
cudaError_t launch_ns_prepare(const void* const* srcs, int src_dt, int R, int C, int batch, const float* sumsq, float eps,
                              void* same, int64_t ld_same, int64_t stride_same, void* trans, int64_t ld_trans,
                              int64_t stride_trans, uint64_t seed, cudaStream_t stream);

}  // namespace hb
