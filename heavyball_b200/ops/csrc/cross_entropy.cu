// Softmax cross-entropy over bf16 logits, forward and backward in one pass over HBM.
//
// One CTA owns one row and sweeps it three times with 16-byte accesses: the maximum (packed bf16 max, from
// DRAM), the sum of exponentials, and the write of the gradient of the mean loss, (softmax - onehot) * scale[0];
// the second and third sweep hit L2 (a row of 50k bf16 logits is 100 KB).  The logits buffer becomes the
// dlogits buffer and no fp32 copy of the logits ever exists.  Columns >= vocab are padding (the leading
// dimension is rounded up so that rows start on 16-byte boundaries and the producing GEMM stays on its aligned
// path): they are skipped by the reductions and zeroed by the write.  Rows whose target equals ignore_index get
// zero loss and zero gradient.  Separate sweeps keep the inner loops free of bounds checks and running-maximum
// rescaling: the kernel is issue-bound (two ex2 per element), not DRAM-bound.
//
// DRAM traffic: one read and one write of the logits, against about eight of each for the chain
// cast-to-fp32 / log_softmax / nll_loss / their backward kernels / cast-back that it replaces.
#include "cross_entropy.h"

#include <cuda_bf16.h>

namespace hb {
namespace {

constexpr int kThreads = 512;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

// Sum (or maximum) over the CTA of one float per thread; every thread gets the result.  `scratch` holds kThreads / 32 floats.
template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, off);
    v = kMax ? fmaxf(v, o) : v + o;
  }
  __syncthreads();  // scratch may still be read from a previous reduction
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = scratch[threadIdx.x & (kThreads / 32 - 1)];
#pragma unroll
  for (int off = kThreads / 64; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, r, off);
    r = kMax ? fmaxf(r, o) : r + o;
  }
  return r;
}

__global__ void __launch_bounds__(kThreads) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits,
                                                              const long long* __restrict__ targets,
                                                              float* __restrict__ loss,
                                                              const float* __restrict__ scale, int vocab, int ld,
                                                              long long ignore_index) {
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * (long long)ld;
  uint4* xv = reinterpret_cast<uint4*>(x);
  const long long target = targets[row];
  const int n_vec = ld >> 3;
  const int full_vec = vocab >> 3;  // vectors [0, full_vec) hold only real columns; at most one more is partly padding
  __shared__ float scratch[kThreads / 32];

  if (target == ignore_index || target < 0 || target >= vocab) {  // no loss, no gradient
    if (threadIdx.x == 0) loss[row] = 0.f;
    for (int v = threadIdx.x; v < n_vec; v += kThreads) xv[v] = make_uint4(0, 0, 0, 0);
    return;
  }

  // sweep 1 (from DRAM): row maximum, on packed bf16 pairs (max is exact in any precision)
  __nv_bfloat162 m2 = __float2bfloat162_rn(-INFINITY);
  for (int v = threadIdx.x; v < full_vec; v += kThreads) {
    const uint4 q = xv[v];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    m2 = __hmax2(__hmax2(m2, h[0]), __hmax2(h[1], __hmax2(h[2], h[3])));
  }
  float m = fmaxf(__low2float(m2), __high2float(m2));
  if (threadIdx.x == 0 && (vocab & 7)) {  // the vector that straddles the end of the vocabulary
    float f[8];
    unpack8(xv[full_vec], f);
    for (int i = 0; i < (vocab & 7); ++i) m = fmaxf(m, f[i]);
  }
  const float row_max = block_reduce<true>(m, scratch);
  const float bias = -row_max * kLog2e;

  // sweep 2 (from L2): sum of exponentials
  float s = 0.f;
  for (int v = threadIdx.x; v < full_vec; v += kThreads) {
    float f[8];
    unpack8(xv[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += exp2f(fmaf(f[i], kLog2e, bias));
  }
  if (threadIdx.x == 0 && (vocab & 7)) {
    float f[8];
    unpack8(xv[full_vec], f);
    for (int i = 0; i < (vocab & 7); ++i) s += exp2f(fmaf(f[i], kLog2e, bias));
  }
  const float total = block_reduce<false>(s, scratch);
  const float g = scale[0];
  const float coef = g / total;
  const float x_target = __bfloat162float(x[target]);
  __syncthreads();  // x[target] has been read by everyone before anyone overwrites the row
  if (threadIdx.x == 0) loss[row] = logf(total) + row_max - x_target;

  // sweep 3 (from L2): the row becomes softmax * g; the target entry is fixed up afterwards
  for (int v = threadIdx.x; v < full_vec; v += kThreads) {
    float f[8];
    unpack8(xv[v], f);
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      h[i] = __floats2bfloat162_rn(exp2f(fmaf(f[2 * i], kLog2e, bias)) * coef, exp2f(fmaf(f[2 * i + 1], kLog2e, bias)) * coef);
    xv[v] = out;
  }
  for (int v = full_vec + threadIdx.x; v < n_vec; v += kThreads) {  // padding (and the straddling vector)
    float f[8];
    unpack8(xv[v], f);
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (v << 3) + 2 * i;
      h[i] = __floats2bfloat162_rn(c < vocab ? exp2f(fmaf(f[2 * i], kLog2e, bias)) * coef : 0.f,
                                   c + 1 < vocab ? exp2f(fmaf(f[2 * i + 1], kLog2e, bias)) * coef : 0.f);
    }
    xv[v] = out;
  }
  __syncthreads();
  if (threadIdx.x == 0) x[target] = __float2bfloat16_rn(exp2f(fmaf(x_target, kLog2e, bias)) * coef - g);
}

}  // namespace

cudaError_t launch_cross_entropy(void* logits, const long long* targets, float* loss, const float* scale,
                                 long long rows, int vocab, int ld, long long ignore_index, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  ce_fwd_bwd_kernel<<<(unsigned)rows, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), targets, loss, scale,
                                                            vocab, ld, ignore_index);
  return cudaGetLastError();
}

}  // namespace hb
