// Fused softmax cross-entropy forward + backward over bf16 logits (see cross_entropy.cu).
#pragma once
#include <cuda_runtime.h>

namespace hb {

// logits: [rows, ld] bf16, ld % 8 == 0, base 16-byte aligned; columns [vocab, ld) are padding.
// On return loss[r] holds the per-row loss (0 for ignored rows) and logits holds
// (softmax - onehot) * scale[0] (0 in padding columns and ignored rows).  scale is a device scalar.
cudaError_t launch_cross_entropy(void* logits, const long long* targets, float* loss, const float* scale,
                                 long long rows, int vocab, int ld, long long ignore_index, cudaStream_t stream);

}  // namespace hb
