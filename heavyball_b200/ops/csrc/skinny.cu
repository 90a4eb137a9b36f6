// fp32 product over a long dimension for block Gram-Schmidt with a narrow panel (the eigenbasis-refresh QR):
//
//   tall_t_mul : C[b] = X[b]^T W[b]     X: [n, m] (leading dimension ldx), W: [n, p], p <= 32, contraction over the
//                                       long dimension n.  The library's GEMM for this shape is a 32x32x16 SIMT
//                                       kernel that walks n serially (18 us whatever m is); here n is split over
//                                       CTAs and the partial products are kept apart (deterministic), to be summed
//                                       by the caller.
//
// 32-wide tiles staged in shared memory, plain FMAs: the products are tiny (at most 2 * 1024 * 1024 * 32 flops per
// matrix) and latency, not throughput, is what the panel loop pays for.  The matching rank-m update W -= X C has
// plenty of row parallelism and stays a library GEMM (a version written here the same way was slower).
#include "skinny.h"

namespace hb {
namespace {

constexpr int kRowsPerCta = 128;  // rows of the long dimension per CTA in tall_t_mul

// grid: (ceil(m / 32), splits, batch); block: 256 threads = 32 (column of W) x 8 (row groups of X^T)
__global__ void __launch_bounds__(256) tall_t_mul_kernel(const float* __restrict__ X, long long ldx, long long strideX,
                                                        const float* __restrict__ W, long long ldw, long long strideW,
                                                        int n, int m, int p, float* __restrict__ C, int splits) {
  __shared__ float xs[kRowsPerCta][33];
  __shared__ float ws[kRowsPerCta][33];
  const int b = blockIdx.z, split = blockIdx.y, m0 = blockIdx.x * 32;
  const float* x = X + (long long)b * strideX;
  const float* w = W + (long long)b * strideW;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // ty in 0..7
  float acc[4] = {0.f, 0.f, 0.f, 0.f};                    // outputs (m0 + ty + 8 i, tx)
  const int rows_per_split = (n + splits - 1) / splits;
  const int r_begin = split * rows_per_split, r_end = min(n, r_begin + rows_per_split);
  for (int r0 = r_begin; r0 < r_end; r0 += kRowsPerCta) {
    for (int i = ty; i < kRowsPerCta; i += 8) {
      const int r = r0 + i;
      const bool in = r < r_end;
      xs[i][tx] = (in && m0 + tx < m) ? x[(long long)r * ldx + m0 + tx] : 0.f;
      ws[i][tx] = (in && tx < p) ? w[(long long)r * ldw + tx] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int i = 0; i < kRowsPerCta; ++i) {
      const float wv = ws[i][tx];
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = fmaf(xs[i][ty + 8 * k], wv, acc[k]);
    }
    __syncthreads();
  }
  float* c = C + ((long long)split * gridDim.z + b) * m * p;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int row = m0 + ty + 8 * k;
    if (row < m && tx < p) c[(long long)row * p + tx] = acc[k];
  }
}

}  // namespace

int tall_splits(int n) {
  const int s = (n + 2 * kRowsPerCta - 1) / (2 * kRowsPerCta);
  return s < 1 ? 1 : (s > 16 ? 16 : s);
}

cudaError_t launch_tall_t_mul(const float* X, long long ldx, long long strideX, const float* W, long long ldw,
                              long long strideW, int batch, int n, int m, int p, float* C, cudaStream_t stream) {
  if (batch == 0 || m == 0 || p == 0) return cudaSuccess;
  const int splits = tall_splits(n);
  dim3 grid((m + 31) / 32, splits, batch);
  tall_t_mul_kernel<<<grid, 256, 0, stream>>>(X, ldx, strideX, W, ldw, strideW, n, m, p, C, splits);
  return cudaGetLastError();
}

}  // namespace hb
