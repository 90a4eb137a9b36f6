// LayerNorm forward and backward for fp32 activations with an optional bf16 output / incoming gradient.
//
// Under bf16 autocast the framework's LayerNorm writes fp32 and the following linear layer casts to bf16 (one
// extra read + write of the activation); on the way back the bf16 gradient is cast to fp32 first, then
// three kernels compute dx and the column sums.  Here the forward kernel writes the consumer's dtype directly
// and the backward kernel reads the bf16 gradient, produces dx and accumulates dgamma / dbeta partial sums in
// registers while it streams the rows, so each tensor crosses HBM once.
//
// Layout: one warp per row, lane l owns columns {128 * v + 4 * l .. + 3 : v < VPL} (float4 granularity), so the
// row lives in registers and the statistics need only warp shuffles.  D = 128 * VPL, VPL <= 8 (the backward
// kernel keeps five row-sized register arrays).
#include "layer_norm.h"

#include <cuda_bf16.h>

namespace hb {
namespace {

constexpr int kWarps = 4;  // rows in flight per CTA

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// With `res` the kernel normalises s = x + res (res in bf16 or fp32) and also writes s to `xsum`: the residual add
// of a transformer block rides along instead of being a separate pass over the stream.
template <int VPL, typename OutT>
__global__ void __launch_bounds__(kWarps * 32) ln_fwd_kernel(const float* __restrict__ x, const void* __restrict__ res,
                                                            int res_bf16, float* __restrict__ xsum,
                                                            const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, OutT* __restrict__ y,
                                                            float* __restrict__ mean, float* __restrict__ rstd,
                                                            long long rows, float eps) {
  constexpr int D = VPL * 128;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* xr = x + row * D;
  float4 v[VPL];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = i * 128 + lane * 4;
    v[i] = load4<float>(xr + c);
    if (res != nullptr) {
      const float4 r = res_bf16 ? load4<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(res) + row * D + c)
                                : load4<float>(static_cast<const float*>(res) + row * D + c);
      v[i] = make_float4(v[i].x + r.x, v[i].y + r.y, v[i].z + r.z, v[i].w + r.w);
      store4<float>(xsum + row * D + c, v[i]);
    }
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mu = warp_sum(s) * (1.f / D);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const float a = v[i].x - mu, b = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
    q += (a * a + b * b) + (c * c + d * d);
  }
  const float rs = rsqrtf(warp_sum(q) * (1.f / D) + eps);
  if (lane == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
  OutT* yr = y + row * D;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = i * 128 + lane * 4;
    const float4 g = load4<float>(gamma + c), b = load4<float>(beta + c);
    store4<OutT>(yr + c, make_float4((v[i].x - mu) * rs * g.x + b.x, (v[i].y - mu) * rs * g.y + b.y,
                                     (v[i].z - mu) * rs * g.z + b.z, (v[i].w - mu) * rs * g.w + b.w));
  }
}

// Each CTA walks rows blockIdx.x * kWarps + warp, stepping by gridDim.x * kWarps; partial[cta][0][:] = dgamma,
// partial[cta][1][:] = dbeta.  All of a row's loads (x, dy and the gradient arriving on the residual stream) are
// issued before the first is used: a version that fetched `dres` after the row statistics paid two memory round
// trips per row and ran at 3.6 TB/s.  gamma is re-read per row (3 KB, stays in L1) to leave the registers to the
// row.  `dx16`, when given, receives a bf16 copy of dx (the gradient of a bf16 residual branch), which saves the
// cast kernel's read of dx.
template <int VPL, typename GradT>
__global__ void __launch_bounds__(kWarps * 32, VPL <= 6 ? 3 : 2)
    ln_bwd_kernel(const GradT* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
                  const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ dres,
                  float* __restrict__ dx, __nv_bfloat16* __restrict__ dx16, float* __restrict__ partial, long long rows) {
  constexpr int D = VPL * 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4 dg[VPL], db[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    dg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    db[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (long long row = (long long)blockIdx.x * kWarps + warp; row < rows; row += (long long)gridDim.x * kWarps) {
    float4 xh[VPL], g[VPL], r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = i * 128 + lane * 4;
      xh[i] = load4<float>(x + row * D + c);
      g[i] = load4<GradT>(dy + row * D + c);
      r[i] = dres != nullptr ? load4<float>(dres + row * D + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const float4 gam = load4<float>(gamma + i * 128 + lane * 4);
      const float4 d = g[i];
      xh[i] = make_float4((xh[i].x - mu) * rs, (xh[i].y - mu) * rs, (xh[i].z - mu) * rs, (xh[i].w - mu) * rs);
      g[i] = make_float4(d.x * gam.x, d.y * gam.y, d.z * gam.z, d.w * gam.w);
      s1 += (g[i].x + g[i].y) + (g[i].z + g[i].w);
      s2 += (g[i].x * xh[i].x + g[i].y * xh[i].y) + (g[i].z * xh[i].z + g[i].w * xh[i].w);
      dg[i].x += d.x * xh[i].x; dg[i].y += d.y * xh[i].y; dg[i].z += d.z * xh[i].z; dg[i].w += d.w * xh[i].w;
      db[i].x += d.x; db[i].y += d.y; db[i].z += d.z; db[i].w += d.w;
    }
    s1 = warp_sum(s1) * (1.f / D);
    s2 = warp_sum(s2) * (1.f / D);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = i * 128 + lane * 4;
      const float4 o = make_float4(rs * (g[i].x - s1 - xh[i].x * s2) + r[i].x, rs * (g[i].y - s1 - xh[i].y * s2) + r[i].y,
                                   rs * (g[i].z - s1 - xh[i].z * s2) + r[i].z, rs * (g[i].w - s1 - xh[i].w * s2) + r[i].w);
      store4<float>(dx + row * D + c, o);
      if (dx16 != nullptr) store4<__nv_bfloat16>(dx16 + row * D + c, o);
    }
  }
  // combine the CTA's warps through shared memory, one column vector at a time
  __shared__ float4 red[kWarps][32];
  float* out = partial + (long long)blockIdx.x * 2 * D;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      red[warp][lane] = which == 0 ? dg[i] : db[i];
      __syncthreads();
      if (warp == 0) {
        float4 a = red[0][lane];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) {
          const float4 b = red[w][lane];
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        store4<float>(out + which * D + i * 128 + lane * 4, a);
      }
      __syncthreads();
    }
  }
}

// dgamma / dbeta = column sums of the per-CTA partials ([n, 2 * D] table).  A block of 32 x 32 threads owns 32
// adjacent columns; the 32 thread rows stride over the n partials and are combined through shared memory (with 8
// thread rows the 444-row table took 11 us, a third of the backward kernel itself).
__global__ void __launch_bounds__(1024) ln_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                                         float* __restrict__ dbeta, int n, int D) {
  const int c = blockIdx.x * 32 + threadIdx.x;  // 2 * D is a multiple of 32
  float a = 0.f;
  for (int i = threadIdx.y; i < n; i += 32) a += partial[(long long)i * 2 * D + c];
  __shared__ float red[32][33];
  red[threadIdx.y][threadIdx.x] = a;
  __syncthreads();
  if (threadIdx.y == 0) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) s += red[j][threadIdx.x];
    if (c < D) dgamma[c] = s; else dbeta[c - D] = s;
  }
}

template <int VPL>
cudaError_t fwd_dispatch(const float* x, const void* res, bool res_bf16, float* xsum, const float* gamma, const float* beta,
                         void* y, bool y_bf16, float* mean, float* rstd, long long rows, float eps, cudaStream_t stream) {
  const unsigned grid = (unsigned)((rows + kWarps - 1) / kWarps);
  if (y_bf16)
    ln_fwd_kernel<VPL, __nv_bfloat16><<<grid, kWarps * 32, 0, stream>>>(x, res, res_bf16, xsum, gamma, beta, static_cast<__nv_bfloat16*>(y), mean, rstd, rows, eps);
  else
    ln_fwd_kernel<VPL, float><<<grid, kWarps * 32, 0, stream>>>(x, res, res_bf16, xsum, gamma, beta, static_cast<float*>(y), mean, rstd, rows, eps);
  return cudaGetLastError();
}

template <int VPL>
cudaError_t bwd_dispatch(const void* dy, bool dy_bf16, const float* x, const float* gamma, const float* mean,
                         const float* rstd, const float* dres, float* dx, __nv_bfloat16* dx16, float* partial, int n_cta,
                         long long rows, cudaStream_t stream) {
  if (dy_bf16)
    ln_bwd_kernel<VPL, __nv_bfloat16><<<n_cta, kWarps * 32, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), x, gamma, mean, rstd, dres, dx, dx16, partial, rows);
  else
    ln_bwd_kernel<VPL, float><<<n_cta, kWarps * 32, 0, stream>>>(static_cast<const float*>(dy), x, gamma, mean, rstd, dres, dx, dx16, partial, rows);
  return cudaGetLastError();
}

}  // namespace

bool layer_norm_supported(int D) { return D > 0 && D % 128 == 0 && D / 128 <= 8; }

int layer_norm_partial_ctas(long long rows) {
  const long long want = (rows + kWarps - 1) / kWarps;
  // the launch bounds hold the kernel to three CTAs of 128 threads per SM up to D = 768
  return (int)(want < 148 * 3 ? (want < 1 ? 1 : want) : 148 * 3);
}

#define HB_LN_SWITCH(D, CALL)            \
  switch ((D) / 128) {                   \
    case 1: return CALL(1);              \
    case 2: return CALL(2);              \
    case 3: return CALL(3);              \
    case 4: return CALL(4);              \
    case 5: return CALL(5);              \
    case 6: return CALL(6);              \
    case 7: return CALL(7);              \
    case 8: return CALL(8);              \
    default: return cudaErrorInvalidValue; \
  }

cudaError_t launch_layer_norm_fwd(const float* x, const void* res, bool res_bf16, float* xsum, const float* gamma,
                                  const float* beta, void* y, bool y_bf16, float* mean, float* rstd, long long rows, int D,
                                  float eps, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
#define CALL(V) fwd_dispatch<V>(x, res, res_bf16, xsum, gamma, beta, y, y_bf16, mean, rstd, rows, eps, stream)
  HB_LN_SWITCH(D, CALL)
#undef CALL
}

cudaError_t launch_layer_norm_bwd(const void* dy, bool dy_bf16, const float* x, const float* gamma, const float* mean,
                                  const float* rstd, const float* dres, float* dx, void* dx_bf16, float* dgamma,
                                  float* dbeta, float* partial, int n_cta, long long rows, int D, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  cudaError_t err;
  {
    auto run = [&]() -> cudaError_t {
#define CALL(V) bwd_dispatch<V>(dy, dy_bf16, x, gamma, mean, rstd, dres, dx, static_cast<__nv_bfloat16*>(dx_bf16), partial, n_cta, rows, stream)
      HB_LN_SWITCH(D, CALL)
#undef CALL
    };
    err = run();
  }
  if (err != cudaSuccess) return err;
  ln_reduce_kernel<<<2 * D / 32, dim3(32, 32), 0, stream>>>(partial, dgamma, dbeta, n_cta, D);
  return cudaGetLastError();
}

}  // namespace hb
