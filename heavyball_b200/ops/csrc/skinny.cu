// fp32 product over a long dimension for block Gram-Schmidt with a narrow panel (the eigenbasis-refresh QR):
//
//   tall_t_mul : C[b] = X[b]^T W[b]     X: [n, m] (leading dimension ldx), W: [n, p], p <= 32, contraction over the
//                                       long dimension n.  The library's GEMM for this shape is a 32x32x16 SIMT
//                                       kernel that walks n serially (18 us whatever m is); here n is split over
//                                       CTAs and the partial products are kept apart (deterministic), to be summed
//                                       by the caller.
//
// Tiles staged in shared memory, 8 x 4 register tiles, plain FMAs: the products are tiny (at most 2 * 1024 * 1024 * 32 flops per
// matrix) and latency, not throughput, is what the panel loop pays for.  The matching rank-m update W -= X C has
// plenty of row parallelism and stays a library GEMM (a version written here the same way was slower).
#include "skinny.h"

#include <stdint.h>

namespace hb {
namespace {

constexpr int kTileM = 128;   // columns of X (rows of the result) per CTA
constexpr int kTileR = 64;    // rows of the long dimension staged at a time
constexpr int kMaxSplits = 16;

// grid: (ceil(m / 128), splits, batch); block: 128 threads = 16 (groups of 8 result rows) x 8 (groups of 4 columns).
// Each thread keeps an 8 x 4 register tile: per staged row it reads 8 + 4 values from shared memory (three 16-byte
// loads) for 32 FMAs.  A first version with one value per load and four FMAs was issue-bound at 20 us per call.
template <bool kVec>
__global__ void __launch_bounds__(128) tall_t_mul_kernel(const float* __restrict__ X, long long ldx, long long strideX,
                                                        const float* __restrict__ W, long long ldw, long long strideW,
                                                        int n, int m, int p, float* __restrict__ C, int splits) {
  __shared__ __align__(16) float xs[kTileR][kTileM];
  __shared__ __align__(16) float ws[kTileR][32];
  const int b = blockIdx.z, split = blockIdx.y, m0 = blockIdx.x * kTileM;
  const float* x = X + (long long)b * strideX;
  const float* w = W + (long long)b * strideW;
  const int t = threadIdx.x, tm = t >> 3, tp = t & 7;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int rows_per_split = (n + splits - 1) / splits;
  const int r_begin = split * rows_per_split, r_end = min(n, r_begin + rows_per_split);
  for (int r0 = r_begin; r0 < r_end; r0 += kTileR) {
    // stage X[r0 .. r0+63][m0 .. m0+127] and W[r0 .. r0+63][0 .. 31]; loads are issued before any is consumed
    if (kVec) {
      float4 xv[16], wv[4];
#pragma unroll
      for (int it = 0; it < 16; ++it) {  // 64 rows x 32 float4 per row, 128 threads
        const int idx = t + 128 * it, rr = idx >> 5, c4 = (idx & 31) * 4;
        const int r = r0 + rr, c = m0 + c4;
        xv[it] = (r < r_end && c < m) ? *reinterpret_cast<const float4*>(x + (long long)r * ldx + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (c + 3 >= m && c < m) {  // tail of the m range: mask the lanes past it
          if (c + 1 >= m) xv[it].y = 0.f;
          if (c + 2 >= m) xv[it].z = 0.f;
          xv[it].w = 0.f;
        }
      }
#pragma unroll
      for (int it = 0; it < 4; ++it) {  // 64 rows x 8 float4 per row
        const int idx = t + 128 * it, rr = idx >> 3, c4 = (idx & 7) * 4;
        const int r = r0 + rr;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < r_end && c4 < p) {
          const float* src = w + (long long)r * ldw + c4;
          v.x = src[0];
          if (c4 + 1 < p) v.y = src[1];
          if (c4 + 2 < p) v.z = src[2];
          if (c4 + 3 < p) v.w = src[3];
        }
        wv[it] = v;
      }
#pragma unroll
      for (int it = 0; it < 16; ++it) {
        const int idx = t + 128 * it;
        *reinterpret_cast<float4*>(&xs[idx >> 5][(idx & 31) * 4]) = xv[it];
      }
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int idx = t + 128 * it;
        *reinterpret_cast<float4*>(&ws[idx >> 3][(idx & 7) * 4]) = wv[it];
      }
    } else {
      for (int idx = t; idx < kTileR * kTileM; idx += 128) {
        const int rr = idx >> 7, c = idx & 127, r = r0 + rr;
        xs[rr][c] = (r < r_end && m0 + c < m) ? x[(long long)r * ldx + m0 + c] : 0.f;
      }
      for (int idx = t; idx < kTileR * 32; idx += 128) {
        const int rr = idx >> 5, c = idx & 31, r = r0 + rr;
        ws[rr][c] = (r < r_end && c < p) ? w[(long long)r * ldw + c] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int rr = 0; rr < kTileR; ++rr) {
      const float4 a0 = *reinterpret_cast<const float4*>(&xs[rr][tm * 8]);
      const float4 a1 = *reinterpret_cast<const float4*>(&xs[rr][tm * 8 + 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&ws[rr][tp * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bw[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* c = C + ((long long)split * gridDim.z + b) * m * p;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + tm * 8 + i;
    if (row >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tp * 4 + j;
      if (col < p) c[(long long)row * p + col] = acc[i][j];
    }
  }
}

}  // namespace

int tall_splits(int n) {  // two staged tiles of rows per CTA, up to 16 splits; very long inputs (the flattened parameter
                          // vector of a low-rank preconditioner: millions of rows) are cut so that every SM gets several CTAs
  const int s = (n + 2 * kTileR - 1) / (2 * kTileR);
  const int cap = n > 65536 ? 2048 : kMaxSplits;
  return s < 1 ? 1 : (s > cap ? cap : s);
}

cudaError_t launch_tall_t_mul(const float* X, long long ldx, long long strideX, const float* W, long long ldw,
                              long long strideW, int batch, int n, int m, int p, float* C, cudaStream_t stream) {
  if (batch == 0 || m == 0 || p == 0) return cudaSuccess;
  const int splits = tall_splits(n);
  dim3 grid((m + kTileM - 1) / kTileM, splits, batch);
  const bool vec = (ldx % 4 == 0) && (strideX % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15) == 0);
  if (vec)
    tall_t_mul_kernel<true><<<grid, 128, 0, stream>>>(X, ldx, strideX, W, ldw, strideW, n, m, p, C, splits);
  else
    tall_t_mul_kernel<false><<<grid, 128, 0, stream>>>(X, ldx, strideX, W, ldw, strideW, n, m, p, C, splits);
  return cudaGetLastError();
}

namespace {

// One CTA inverts one upper-triangular block by back substitution; thread j produces column j of the inverse:
//   x_jj = 1 / t_jj,   x_ij = -(sum_{k = i+1 .. j} t_ik x_kj) / t_ii   for i = j-1 .. 0.
// Both the block and its inverse sit in shared memory (2 x 128 x 129 floats).  The work is O(blk^3 / 6) FMAs spread
// over 128 threads; at 64 blocks per call this takes tens of microseconds, against a library triangular solve per
// leaf that walks the batch one matrix at a time.
__global__ void __launch_bounds__(kTriBlock) tri_inv_blocks_kernel(const float* __restrict__ Q, long long ld, long long strideQ,
                                                                 int n, float* __restrict__ X) {
  extern __shared__ float tri_smem[];
  float (*t)[kTriBlock + 1] = reinterpret_cast<float (*)[kTriBlock + 1]>(tri_smem);
  float (*x)[kTriBlock + 1] = reinterpret_cast<float (*)[kTriBlock + 1]>(tri_smem + kTriBlock * (kTriBlock + 1));
  const int blk = blockIdx.x, b = blockIdx.y, nblk = gridDim.x;
  const int r0 = blk * kTriBlock, size = min(kTriBlock, n - r0);
  const float* q = Q + (long long)b * strideQ + (long long)r0 * ld + r0;
  const int j = threadIdx.x;
  for (int i = 0; i < kTriBlock; ++i) {  // row i of the block, coalesced over j
    float v = (i == j) ? 1.f : 0.f;
    if (i < size && j < size && j >= i) v = q[(long long)i * ld + j];
    t[i][j] = v;
    x[i][j] = 0.f;
  }
  __syncthreads();
  {
    x[j][j] = 1.0f / t[j][j];
    for (int i = j - 1; i >= 0; --i) {
      float s = 0.f;
      for (int k = i + 1; k <= j; ++k) s = fmaf(t[i][k], x[k][j], s);
      x[i][j] = -s / t[i][i];
    }
  }
  __syncthreads();
  float* out = X + ((long long)b * nblk + blk) * kTriBlock * kTriBlock;
  for (int i = 0; i < kTriBlock; ++i) out[i * kTriBlock + j] = x[i][j];
}

}  // namespace

cudaError_t launch_tri_inv_blocks(const float* Q, long long ld, long long strideQ, int batch, int n, float* X,
                                  cudaStream_t stream) {
  if (batch == 0 || n == 0) return cudaSuccess;
  constexpr int kBytes = 2 * kTriBlock * (kTriBlock + 1) * (int)sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tri_inv_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid((n + kTriBlock - 1) / kTriBlock, batch);
  tri_inv_blocks_kernel<<<grid, kTriBlock, kBytes, stream>>>(Q, ld, strideQ, n, X);
  return cudaGetLastError();
}


// ------------------------------------------------------------------------------------------ Cholesky leaf
// One CTA of 1024 threads factors one (up to) 128 x 128 symmetric positive definite block G = R^T R (R upper triangular)
// and inverts R, both in shared memory.
//   factor (right-looking, every trailing element has its own thread slot):
//     for k = 0 .. n-1:  r_kk = sqrt(g_kk);  r_kj = g_kj / r_kk (j > k);  g_ij -= r_ki r_kj (k < i <= j)
//   invert: the four 32 x 32 diagonal blocks by back substitution (one warp each, lane = column), then the blocks
//     above the diagonal by distance d = 1, 2, 3:  X_IJ = -X_II (sum_{K = I+1 .. J} R_IK X_KJ), J = I + d,
//     as 32 x 32 block products with one output element per thread.
// A non-positive or non-finite pivot is replaced by 1 and counted in info[b] (the result for that matrix is then
// meaningless, the others are unaffected).  The refresh of an eigenbasis factors 16 leaves per 2048-wide factor and
// round, one after the other, so the latency of this kernel is what counts: a thread-per-column version took 270 us
// (dependent shared-memory loads), the batched library factorisation plus a separate inversion 230 us.
namespace {

constexpr int kLeafThreads = 1024;
constexpr int kLeafLd = kTriBlock + 1;

__global__ void __launch_bounds__(kLeafThreads) chol_inv_leaf_kernel(const float* __restrict__ G, long long ldg, long long strideG,
                                                                     float* __restrict__ R, long long ldr, long long strideR,
                                                                     float* __restrict__ X, long long strideX, int size,
                                                                     int* __restrict__ info) {
  extern __shared__ float leaf_smem[];
  float(*t)[kLeafLd] = (float(*)[kLeafLd])leaf_smem;
  float(*x)[kLeafLd] = (float(*)[kLeafLd])(leaf_smem + kTriBlock * kLeafLd);
  __shared__ int failed;
  const int b = blockIdx.x, tid = threadIdx.x, ty = tid >> 5, tx = tid & 31;
  const float* g = G + (long long)b * strideG;
  if (tid == 0) failed = 0;
  for (int idx = tid; idx < kTriBlock * kTriBlock; idx += kLeafThreads) {  // upper part; a short block is completed by an identity
    const int i = idx >> 7, j = idx & (kTriBlock - 1);
    float v = (i == j) ? 1.f : 0.f;
    if (i < size && j < size && j >= i) v = g[(long long)i * ldg + j];
    t[i][j] = v;
    x[i][j] = 0.f;
  }
  __syncthreads();

  for (int k = 0; k < size; ++k) {
    const float d = t[k][k];  // written for the last time in the previous step's trailing update
    const bool ok = d > 0.f && d < 3.0e38f;
    const float inv_piv = ok ? rsqrtf(d) : 1.f;
    if (tid > k && tid < size) t[k][tid] *= inv_piv;
    __syncthreads();
    if (tid == 0) {
      t[k][k] = ok ? d * inv_piv : 1.f;  // sqrt(d); nobody reads the diagonal entry during the trailing update
      if (!ok) failed = 1;
    }
    for (int i = k + 1 + ty; i < size; i += 32) {
      const float rki = t[k][i];
      for (int j = i + tx; j < size; j += 32) t[i][j] = fmaf(-rki, t[k][j], t[i][j]);
    }
    __syncthreads();
  }

  if (tid < kTriBlock) {  // diagonal 32 x 32 blocks: warp = block, lane = column
    const int base = tid & ~31, jl = tid & 31, col = base + jl;
    x[col][col] = 1.0f / t[col][col];
    for (int i = jl - 1; i >= 0; --i) {
      float sum = 0.f;
      for (int k = i + 1; k <= jl; ++k) sum = fmaf(t[base + i][base + k], x[base + k][col], sum);
      x[base + i][col] = -sum / t[base + i][base + i];
    }
  }
  __syncthreads();
  for (int dist = 1; dist < kTriBlock / 32; ++dist) {
    // S_I = sum_K R_IK X_KJ, parked in the (otherwise unused) mirror position below the diagonal
    for (int I = 0; I + dist < kTriBlock / 32; ++I) {
      const int J = I + dist;
      float s0 = 0.f, s1 = 0.f;
      const float* rrow = &t[32 * I + ty][0];
      for (int k = 32 * (I + 1); k < 32 * (J + 1); k += 2) {
        s0 = fmaf(rrow[k], x[k][32 * J + tx], s0);
        s1 = fmaf(rrow[k + 1], x[k + 1][32 * J + tx], s1);
      }
      x[32 * J + ty][32 * I + tx] = s0 + s1;
    }
    __syncthreads();
    for (int I = 0; I + dist < kTriBlock / 32; ++I) {
      const int J = I + dist;
      float s0 = 0.f, s1 = 0.f;
      for (int k = ty; k < 32; k += 2) {  // X_II is upper triangular: columns below the row index are zero
        s0 = fmaf(x[32 * I + ty][32 * I + k], x[32 * J + k][32 * I + tx], s0);
        if (k + 1 < 32) s1 = fmaf(x[32 * I + ty][32 * I + k + 1], x[32 * J + k + 1][32 * I + tx], s1);
      }
      x[32 * I + ty][32 * J + tx] = -(s0 + s1);
    }
    __syncthreads();
  }

  float* r = R + (long long)b * strideR;
  float* out = X + (long long)b * strideX;
  for (int idx = tid; idx < kTriBlock * kTriBlock; idx += kLeafThreads) {
    const int i = idx >> 7, j = idx & (kTriBlock - 1);
    if (i < size && j < size) r[(long long)i * ldr + j] = j >= i ? t[i][j] : 0.f;
    out[idx] = j >= i ? x[i][j] : 0.f;
  }
  if (tid == 0 && failed && info != nullptr) atomicAdd(info + b, 1);
}

}  // namespace

cudaError_t launch_chol_inv_leaf(const float* G, long long ldg, long long strideG, float* R, long long ldr, long long strideR,
                                 float* X, long long strideX, int batch, int size, int* info, cudaStream_t stream) {
  if (batch == 0 || size == 0) return cudaSuccess;
  if (size > kTriBlock) return cudaErrorInvalidValue;
  constexpr int kBytes = 2 * kTriBlock * (kTriBlock + 1) * (int)sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(chol_inv_leaf_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  chol_inv_leaf_kernel<<<batch, kLeafThreads, kBytes, stream>>>(G, ldg, strideG, R, ldr, strideR, X, strideX, size, info);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------ packed upper triangles
// PSGD stores a triangular factor as the row-major upper triangle ("line").  Row i of the triangle is the contiguous
// piece dense[i, i:n] and sits at line offset i*n - i*(i-1)/2, so packing and unpacking are row copies: one block per
// (row, matrix), no index tensors (index_put / index_select read an 8-byte index per element and first materialise
// 16 n^2 bytes of indices).
namespace {

template <typename T>
__global__ void __launch_bounds__(256) triu_pack_kernel(const T* __restrict__ dense, T* __restrict__ line, int n) {
  const long long i = blockIdx.x, b = blockIdx.y;
  const long long len = (long long)n * (n + 1) / 2;
  const T* src = dense + (b * n + i) * n + i;
  T* dst = line + b * len + i * n - i * (i - 1) / 2;
  for (int j = threadIdx.x; j < n - (int)i; j += blockDim.x) dst[j] = src[j];
}

template <typename T>
__global__ void __launch_bounds__(256) triu_unpack_kernel(const T* __restrict__ line, T* __restrict__ dense, int n) {
  const long long i = blockIdx.x, b = blockIdx.y;
  const long long len = (long long)n * (n + 1) / 2;
  const T* src = line + b * len + i * n - i * (i - 1) / 2 - i;  // indexed by the dense column
  T* dst = dense + (b * n + i) * n;
  for (int j = threadIdx.x; j < n; j += blockDim.x) dst[j] = j >= (int)i ? src[j] : T(0);
}

}  // namespace

cudaError_t launch_triu_pack(const void* dense, void* line, int elem_bytes, int batch, int n, cudaStream_t stream) {
  if (batch == 0 || n == 0) return cudaSuccess;
  dim3 grid(n, batch);
  if (elem_bytes == 4) triu_pack_kernel<uint32_t><<<grid, 256, 0, stream>>>((const uint32_t*)dense, (uint32_t*)line, n);
  else if (elem_bytes == 2) triu_pack_kernel<uint16_t><<<grid, 256, 0, stream>>>((const uint16_t*)dense, (uint16_t*)line, n);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_triu_unpack(const void* line, void* dense, int elem_bytes, int batch, int n, cudaStream_t stream) {
  if (batch == 0 || n == 0) return cudaSuccess;
  dim3 grid(n, batch);
  if (elem_bytes == 4) triu_unpack_kernel<uint32_t><<<grid, 256, 0, stream>>>((const uint32_t*)line, (uint32_t*)dense, n);
  else if (elem_bytes == 2) triu_unpack_kernel<uint16_t><<<grid, 256, 0, stream>>>((const uint16_t*)line, (uint16_t*)dense, n);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace hb
