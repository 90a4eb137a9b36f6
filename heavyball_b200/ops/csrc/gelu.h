// tanh-approximated GELU on bf16 activations, and its backward fused with the bias gradient of the linear layer
// that produced the activations (see gelu.cu).
#pragma once
#include <cuda_runtime.h>

namespace hb {

// y = gelu_tanh(u); n elements, n % 8 == 0, both pointers 16-byte aligned.
cudaError_t launch_gelu_fwd(const void* u, void* y, long long n, cudaStream_t stream);

// Number of row splits (rows of `partial`) launch_gelu_bwd uses for a [rows, cols] input.
int gelu_bwd_splits(long long rows, int cols);

// du = dy * gelu_tanh'(u) in bf16, dbias[c] = sum_r du[r, c] in fp32 (summed before the rounding to bf16).
// dy, u, du: [rows, cols] bf16, contiguous, cols % 8 == 0, 16-byte aligned; partial: [gelu_bwd_splits, cols] fp32.
cudaError_t launch_gelu_bwd(const void* dy, const void* u, void* du, long long rows, int cols, float* partial,
                            float* dbias, cudaStream_t stream);

}  // namespace hb
