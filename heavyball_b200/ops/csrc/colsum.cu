// Column sums of a row-major bf16 matrix: out[c] = sum_r x[r, c], fp32 accumulation.  This is the bias gradient of
// a linear layer (x = dY); the generic reduction it replaces runs at about 2 TB/s on [16384, 768..3072] inputs and
// was the largest non-GEMM item of a transformer training step.
//
// Stage 1: a CTA owns a strip of 64 columns (one 128-byte line per row) and 1/kSplits of the rows.  Its 256 threads
// are 8 vector lanes x 32 row lanes; each thread adds up 8 columns over every 32nd row of the strip with 16-byte
// loads, the 32 row lanes are combined through shared memory, and the strip's partial sums go to partial[split][c].
// Stage 2 adds the kSplits partials (deterministic: no atomics).
//
// Up to kColsumMaxBatch matrices of one shape go through one pair of launches (blockIdx.z picks the matrix) and
// land side by side in `out`: the three bias gradients of a packed q / k / v projection are one call, already
// concatenated.  At 25 MB per matrix a launch is about half fixed cost (ramp-up, the shared-memory combine, tail).
#include "colsum.h"

#include <cuda_bf16.h>

namespace hb {
namespace {

constexpr int kSplits = 32;

static_assert(kColsumMaxBatch == 4, "the pointer select below lists four entries");
struct ColsumPtrs {
  const __nv_bfloat16* x[kColsumMaxBatch];
};

__global__ void __launch_bounds__(256) colsum_partial_kernel(const ColsumPtrs ptrs, long long rows, int cols,
                                                            float* __restrict__ partial_all) {
  // selects instead of a dynamic index: the parameter struct stays in constant memory
  const __nv_bfloat16* __restrict__ x =
      blockIdx.z == 0 ? ptrs.x[0] : (blockIdx.z == 1 ? ptrs.x[1] : (blockIdx.z == 2 ? ptrs.x[2] : ptrs.x[3]));
  float* __restrict__ partial = partial_all + (long long)blockIdx.z * kSplits * cols;
  const int vec = threadIdx.x & 7, lane_r = threadIdx.x >> 3;
  const int c0 = blockIdx.x * 64 + vec * 8;
  const long long per = (rows + kSplits - 1) / kSplits;
  const long long r_begin = blockIdx.y * per, r_end = min(rows, r_begin + per);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < cols) {  // cols is a multiple of 8
    for (long long r = r_begin + lane_r; r < r_end; r += 32) {
      const uint4 q = *reinterpret_cast<const uint4*>(x + r * cols + c0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
  }
  __shared__ float red[32][65];
#pragma unroll
  for (int i = 0; i < 8; ++i) red[lane_r][vec * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) s += red[j][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < cols) partial[(long long)blockIdx.y * cols + c] = s;
  }
}

__global__ void colsum_final_kernel(const float* __restrict__ partial_all, int cols, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float* __restrict__ partial = partial_all + (long long)blockIdx.y * kSplits * cols;
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kSplits; ++j) s += partial[(long long)j * cols + c];
  out[(long long)blockIdx.y * cols + c] = s;
}

}  // namespace

int colsum_splits() { return kSplits; }

cudaError_t launch_colsum_bf16_batch(const void* const* xs, int n, long long rows, int cols, float* partial, float* out,
                                     cudaStream_t stream) {
  if (n < 1 || n > kColsumMaxBatch) return cudaErrorInvalidValue;
  ColsumPtrs ptrs;
  for (int i = 0; i < kColsumMaxBatch; ++i) ptrs.x[i] = static_cast<const __nv_bfloat16*>(xs[i < n ? i : 0]);
  dim3 grid((cols + 63) / 64, kSplits, n);
  colsum_partial_kernel<<<grid, 256, 0, stream>>>(ptrs, rows, cols, partial);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  colsum_final_kernel<<<dim3((cols + 255) / 256, n), 256, 0, stream>>>(partial, cols, out);
  return cudaGetLastError();
}

cudaError_t launch_colsum_bf16(const void* x, long long rows, int cols, float* partial, float* out, cudaStream_t stream) {
  return launch_colsum_bf16_batch(&x, 1, rows, cols, partial, out, stream);
}

}  // namespace hb
