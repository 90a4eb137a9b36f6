// LayerNorm forward / backward kernels for fp32 activations (see layer_norm.cu).
#pragma once
#include <cuda_runtime.h>

namespace hb {

// Row length D must be a multiple of 128 and at most 1024.
bool layer_norm_supported(int D);
// Number of CTAs (and rows of the partial-sum table, each 2 * D floats) the backward kernel uses.
int layer_norm_partial_ctas(long long rows);

// res (optional, bf16 or fp32, same shape as x): y = LN(x + res) and xsum = x + res.
cudaError_t launch_layer_norm_fwd(const float* x, const void* res, bool res_bf16, float* xsum, const float* gamma,
                                  const float* beta, void* y, bool y_bf16, float* mean, float* rstd, long long rows, int D,
                                  float eps, cudaStream_t stream);

// x is the normalised tensor (x + res when a residual was given).  dres (optional, fp32): added to dx.
// dx_bf16 (optional): receives a bf16 copy of dx.
cudaError_t launch_layer_norm_bwd(const void* dy, bool dy_bf16, const float* x, const float* gamma, const float* mean,
                                  const float* rstd, const float* dres, float* dx, void* dx_bf16, float* dgamma,
                                  float* dbeta, float* partial, int n_cta, long long rows, int D, cudaStream_t stream);

}  // namespace hb
