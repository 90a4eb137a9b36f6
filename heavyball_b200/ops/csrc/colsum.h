// Column sums of a bf16 matrix with fp32 accumulation (see colsum.cu).
#pragma once
#include <cuda_runtime.h>

namespace hb {

constexpr int kColsumMaxBatch = 4;
int colsum_splits();
// x: [rows, cols] bf16, contiguous, cols % 8 == 0, 16-byte aligned; partial: [colsum_splits(), cols] fp32 scratch.
cudaError_t launch_colsum_bf16(const void* x, long long rows, int cols, float* partial, float* out, cudaStream_t stream);

// The same for n <= kColsumMaxBatch matrices of one shape: out[i * cols + c] = column sum c of xs[i];
// partial: [n, colsum_splits(), cols].
cudaError_t launch_colsum_bf16_batch(const void* const* xs, int n, long long rows, int cols, float* partial, float* out,
                                     cudaStream_t stream);

}  // namespace hb
