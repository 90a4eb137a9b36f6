// GELU (tanh form) between the two linear layers of a transformer MLP, on the bf16 activations [tokens, d_ff].
//
// Forward: one pass, 16-byte loads and stores, four independent loads per thread in flight.
//
// Backward: du = dy * gelu'(u), and in the same pass the column sums of du, i.e. the bias gradient of the linear
// layer that produced u.  Computed separately that is a second full read of du (100 MB for 16384 x 3072) by a
// column-sum kernel.  A CTA owns a strip of 256 columns (one warp reads 512 contiguous bytes of a row) and 1/splits
// of the rows; its 8 warps take every 8th row, two rows in flight per warp.  The kernel issues about 30 instructions
// per element (fp32 exp and reciprocal included), so it needs occupancy more than loads in flight: with four rows
// in flight (80 registers, three CTAs per SM) the issue slots were 67 % busy and DRAM 49 %.  Column sums are kept in fp32 registers
// (from the values before they are rounded to bf16), combined across the 8 warps through shared memory and written
// to partial[split][c]; a second kernel adds the splits (deterministic: no atomics).
//
// The math is fp32 throughout: gelu = u (1 + tanh z) / 2 with z = k0 (u + k1 u^3), evaluated through the logistic
// function of 2z (see below).
#include "gelu.h"

#include <cuda_bf16.h>
#include <stdint.h>

namespace hb {
namespace {

constexpr float kK0 = 0.7978845608028654f;  // sqrt(2 / pi)
constexpr float kK1 = 0.044715f;
constexpr int kStrip = 256;     // columns per CTA in the backward kernel
constexpr int kRowLanes = 8;    // warps per CTA, one row each per step
constexpr int kInFlight = 4;    // vectors per thread the forward kernel loads before any is consumed
constexpr int kBwdRows = 2;     // rows per warp the backward kernel loads (dy and u) before any is consumed
constexpr int kResident = 4;    // backward CTAs per SM the launch bounds ask for (63 registers per thread)
constexpr int kSMs = 148;
constexpr int kMaxSplits = 64;

// With z = k0 (u + k1 u^3) and s = sigmoid(2z) = (1 + tanh z) / 2:  gelu = u s  and, since 1 - tanh^2 z = 4 s (1 - s),
// gelu' = s (1 + 2 u (1 - s) k0 (1 + 3 k1 u^2)).  s and 1 - s = e s come from e = exp(-2z) without the cancellation
// that 1 + tanh z has for negative z.  For |z| >= 40 (|u| above about 9.6) the limits are returned: s is 0 or 1 far
// below fp32 resolution there, and e^{80} is the largest value the formulas see.
constexpr float kZMax = 40.f;

__device__ __forceinline__ float gelu_value(float u) {
  const float z = kK0 * (u + kK1 * u * u * u);
  if (fabsf(z) >= kZMax) return z > 0.f ? u : 0.f;
  return __fdividef(u, 1.f + __expf(-2.f * z));
}

__device__ __forceinline__ float gelu_slope(float u) {
  const float u2 = u * u;
  const float z = kK0 * (u + kK1 * u * u2);
  if (fabsf(z) >= kZMax) return z > 0.f ? 1.f : 0.f;
  const float e = __expf(-2.f * z);
  const float s = __fdividef(1.f, 1.f + e);
  return s * (1.f + 2.f * u * (e * s) * kK0 * (1.f + 3.f * kK1 * u2));
}

__global__ void __launch_bounds__(256) gelu_fwd_kernel(const uint4* __restrict__ u, uint4* __restrict__ y, long long n_vec) {
  const long long base = (long long)blockIdx.x * (256 * kInFlight) + threadIdx.x;
  uint4 q[kInFlight];
#pragma unroll
  for (int i = 0; i < kInFlight; ++i) {
    const long long idx = base + (long long)i * 256;
    q[i] = idx < n_vec ? u[idx] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < kInFlight; ++i) {
    const long long idx = base + (long long)i * 256;
    if (idx >= n_vec) continue;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      h[j] = __floats2bfloat162_rn(gelu_value(f.x), gelu_value(f.y));
    }
    y[idx] = q[i];
  }
}

__global__ void __launch_bounds__(256, kResident)
    gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ du,
                    long long rows, int cols, int splits, float* __restrict__ partial) {
  const int vec = threadIdx.x & 31, lane_r = threadIdx.x >> 5;
  const int c0 = blockIdx.x * kStrip + vec * 8;
  const long long per = (rows + splits - 1) / splits;
  const long long r_begin = (long long)blockIdx.y * per;
  const long long r_end = r_begin + per < rows ? r_begin + per : rows;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < cols) {  // cols is a multiple of 8: a vector is inside or outside as a whole
    for (long long r = r_begin + lane_r; r < r_end; r += kRowLanes * kBwdRows) {
      uint4 g[kBwdRows], a[kBwdRows];
#pragma unroll
      for (int i = 0; i < kBwdRows; ++i) {
        const long long rr = r + (long long)i * kRowLanes;
        if (rr < r_end) {
          g[i] = *reinterpret_cast<const uint4*>(dy + rr * cols + c0);
          a[i] = *reinterpret_cast<const uint4*>(u + rr * cols + c0);
        }
      }
#pragma unroll
      for (int i = 0; i < kBwdRows; ++i) {
        const long long rr = r + (long long)i * kRowLanes;
        if (rr >= r_end) continue;
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g[i]);
        const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a[i]);
        uint4 out;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gf = __bfloat1622float2(gh[j]), af = __bfloat1622float2(ah[j]);
          const float d0 = gf.x * gelu_slope(af.x), d1 = gf.y * gelu_slope(af.y);
          acc[2 * j] += d0;
          acc[2 * j + 1] += d1;
          oh[j] = __floats2bfloat162_rn(d0, d1);
        }
        *reinterpret_cast<uint4*>(du + rr * cols + c0) = out;
      }
    }
  }
  __shared__ float red[kRowLanes][kStrip + 1];
#pragma unroll
  for (int i = 0; i < 8; ++i) red[lane_r][vec * 8 + i] = acc[i];
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kRowLanes; ++j) s += red[j][threadIdx.x];
  const int c = blockIdx.x * kStrip + threadIdx.x;
  if (c < cols) partial[(long long)blockIdx.y * cols + c] = s;
}

__global__ void gelu_bias_final_kernel(const float* __restrict__ partial, int splits, int cols, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int j = 0; j < splits; ++j) s += partial[(long long)j * cols + c];
  out[c] = s;
}

}  // namespace

cudaError_t launch_gelu_fwd(const void* u, void* y, long long n, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const long long n_vec = n / 8;
  const long long per_cta = 256 * kInFlight;
  const unsigned grid = (unsigned)((n_vec + per_cta - 1) / per_cta);
  gelu_fwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(u), static_cast<uint4*>(y), n_vec);
  return cudaGetLastError();
}

int gelu_bwd_splits(long long rows, int cols) {
  // one full wave of resident CTAs over the strips; every split has at least one step of rows
  const int strips = (cols + kStrip - 1) / kStrip;
  long long s = (kSMs * kResident) / strips;
  const long long by_rows = (rows + kRowLanes * kBwdRows - 1) / (kRowLanes * kBwdRows);
  if (s > by_rows) s = by_rows;
  if (s > kMaxSplits) s = kMaxSplits;
  return s < 1 ? 1 : (int)s;
}

cudaError_t launch_gelu_bwd(const void* dy, const void* u, void* du, long long rows, int cols, float* partial,
                            float* dbias, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  const int splits = gelu_bwd_splits(rows, cols);
  dim3 grid((cols + kStrip - 1) / kStrip, splits);
  gelu_bwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(u),
                                            static_cast<__nv_bfloat16*>(du), rows, cols, splits, partial);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gelu_bias_final_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(partial, splits, cols, dbias);
  return cudaGetLastError();
}

}  // namespace hb
