// Softmax cross-entropy over bf16 logits, forward and backward in one pass over HBM.
//
// One CTA owns one row.  Pass 1 streams the row with 16-byte loads and keeps a running (max, sum of
// exponentials) per thread, merged across the CTA; pass 2 streams the same row again (it is still in L2: a row
// of 50k bf16 logits is 100 KB) and overwrites it with the gradient of the mean loss,
// (softmax - onehot) * scale[0], so the logits buffer becomes the dlogits buffer and no fp32 copy of the
// logits ever exists.  Columns >= vocab are padding (the leading dimension is rounded up so that rows start
// on 16-byte boundaries and the producing GEMM stays on its aligned path): they are skipped in pass 1 and
// zeroed in pass 2.  Rows whose target equals ignore_index get zero loss and zero gradient.
//
// DRAM traffic: one read and one write of the logits, against about eight of each for the chain
// cast-to-fp32 / log_softmax / nll_loss / their backward kernels / cast-back that it replaces.
#include "cross_entropy.h"

#include <cuda_bf16.h>

namespace hb {
namespace {

constexpr int kThreads = 512;
constexpr float kLog2e = 1.4426950408889634f;

struct MaxSum {
  float m, s;  // running maximum (natural units), sum of exp(x - m)
};

__device__ __forceinline__ MaxSum merge(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  // exp2f(-inf) = 0 covers the empty state (m = -inf, s = 0) as long as the merged maximum is finite
  const float sa = (a.m == -INFINITY) ? 0.f : a.s * exp2f((a.m - m) * kLog2e);
  const float sb = (b.m == -INFINITY) ? 0.f : b.s * exp2f((b.m - m) * kLog2e);
  return {m, sa + sb};
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

__global__ void __launch_bounds__(kThreads) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits,
                                                              const long long* __restrict__ targets,
                                                              float* __restrict__ loss,
                                                              const float* __restrict__ scale, int vocab, int ld,
                                                              long long ignore_index) {
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * (long long)ld;
  const long long target = targets[row];
  const int n_vec = ld >> 3;
  const bool ignored = target == ignore_index || target < 0 || target >= vocab;

  __shared__ MaxSum warp_part[kThreads / 32];
  __shared__ MaxSum total;

  MaxSum acc{-INFINITY, 0.f};
  if (!ignored) {
    for (int v = threadIdx.x; v < n_vec; v += kThreads) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(x)[v], f);
      const int base = v << 3;
      float vmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (base + i < vocab) vmax = fmaxf(vmax, f[i]);
      if (vmax == -INFINITY) continue;  // vector lies entirely in the padding
      const float m = fmaxf(acc.m, vmax);
      float s = (acc.m == -INFINITY) ? 0.f : acc.s * exp2f((acc.m - m) * kLog2e);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (base + i < vocab) s += exp2f((f[i] - m) * kLog2e);
      acc = {m, s};
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      MaxSum other{__shfl_xor_sync(0xffffffffu, acc.m, off), __shfl_xor_sync(0xffffffffu, acc.s, off)};
      acc = merge(acc, other);
    }
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
      MaxSum p = threadIdx.x < kThreads / 32 ? warp_part[threadIdx.x] : MaxSum{-INFINITY, 0.f};
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        MaxSum other{__shfl_xor_sync(0xffffffffu, p.m, off), __shfl_xor_sync(0xffffffffu, p.s, off)};
        p = merge(p, other);
      }
      if (threadIdx.x == 0) total = p;
    }
    __syncthreads();
  }

  const float row_max = ignored ? 0.f : total.m;
  const float inv_sum = ignored ? 0.f : 1.f / total.s;
  const float g = ignored ? 0.f : scale[0];
  if (threadIdx.x == 0)
    loss[row] = ignored ? 0.f : (logf(total.s) + row_max - __bfloat162float(x[target]));
  __syncthreads();  // x[target] is read before any thread overwrites it

  const int tvec = ignored ? -1 : (int)(target >> 3);
  for (int v = threadIdx.x; v < n_vec; v += kThreads) {
    uint4 out = make_uint4(0, 0, 0, 0);
    if (!ignored) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(x)[v], f);
      const int base = v << 3;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float p = (base + i < vocab) ? exp2f((f[i] - row_max) * kLog2e) * inv_sum : 0.f;
        if (v == tvec && base + i == (int)target) p -= 1.f;
        f[i] = p * g;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    }
    reinterpret_cast<uint4*>(x)[v] = out;
  }
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
