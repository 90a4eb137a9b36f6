// fp32-in / fp32-out batched GEMM at near-fp32 accuracy on the tf32 tensor-core path of sm_100a ("3xTF32").
//
// The preconditioner algebra of SOAP and PSGD (eigenbasis projections, Gram statistics, Kronecker factor
// products; heavyball/utils.py:1211-1324, 2079-2236 of the reference run them as fp32 cuBLAS einsums) needs more
// than tf32's 10 mantissa bits, and fp32 SIMT GEMMs run at a twentieth of the tensor-core rate.  Each operand is
// therefore split once into hi = tf32(x) and lo = tf32(x - hi), and the product is taken as
//     A B^T ~= hi_a hi_b^T + hi_a lo_b^T + lo_a hi_b^T
// The split kernel lays the three terms out along K - A rows as [hi | hi | lo], B rows as [hi | lo | hi] - so the
// whole sum is ONE K-major tf32 GEMM over 3K with a single fp32 accumulator in tensor memory; the dropped
// lo*lo term and the rounding of lo to tf32 are both below 2^-21.  Measured error: about 2^-18 of |A||B|^T for
// K = 2048 (fp32 SIMT: 2^-21, one tf32 pass: 2^-11); it is set by the rounding of the tensor core's accumulator.
//
// GEMM kernel (one 128x128 output tile per CTA, 192 threads, two CTAs per SM):
//   warp 0     : TMA producer, cp.async.bulk.tensor 3-D loads (128-byte swizzle, 32 fp32 per row) into a 3-stage ring
//   warp 1     : tcgen05.mma.cta_group::1.kind::tf32, 128x128x8 per instruction, accumulator in 128 TMEM columns
//   warps 2..5 : tcgen05.ld, scale by alpha, stage the fp32 tile in the (now idle) ring, four bulk tensor stores
// Waits are bounded as in the bf16 kernels: on expiry the CTA flags `status`, drains, frees TMEM and returns.
#include "tf32_gemm.h"

#include "tc_common.cuh"

namespace hb {
namespace {

constexpr int TBM = 128, TBN = 128, TBK = 32;
constexpr int kTStages = 3;
constexpr int kTTileBytes = TBM * TBK * 4;           // 16 KiB per operand tile
constexpr int kTStageBytes = 2 * kTTileBytes;
constexpr int kTSmemBytes = kTStages * kTStageBytes + 1024;
constexpr int kTThreads = 192;
constexpr uint32_t kTTmemCols = 128;
// tf32 x tf32 -> fp32, both operands K-major, M = 128, N = 128
constexpr uint32_t kTf32InstrDesc =
    (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TBN >> 3) << 17) | ((uint32_t)(TBM >> 4) << 24);

__global__ void __launch_bounds__(kTThreads, 2)
tf32_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, int M, int N, int K3, float alpha, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kTStages];
  __shared__ __align__(8) uint64_t empty_bar[kTStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  if (status != nullptr && *(volatile const int*)status != 0) return;  // an earlier CTA gave up: do not pile on
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tiles_n = (N + TBN - 1) / TBN;
  const int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n, batch = blockIdx.y;
  const int num_kb = (K3 + TBK - 1) / TBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, kTTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int issued = 0;
  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kTStages, round = kb / kTStages;
        if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &abort_flag)) break;
        uint8_t* dst = tiles + s * kTStageBytes;
        mbar_expect_tx(&full_bar[s], kTStageBytes);
        tma_load_3d(dst, &map_a, &full_bar[s], kb * TBK, tm * TBM, batch);
        tma_load_3d(dst + kTTileBytes, &map_b, &full_bar[s], kb * TBK, tn * TBN, batch);
        issued = kb + 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kTStages, round = kb / kTStages;
        ok = mbar_wait(&full_bar[s], round & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * kTStageBytes);
        const uint64_t a_desc = make_smem_desc(a_addr), b_desc = make_smem_desc(a_addr + kTTileBytes);
#pragma unroll
        for (int k = 0; k < TBK / 8; ++k)  // 8 fp32 = 32 B along K inside the swizzle atom = +2 address units
          tc_mma_tf32(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kTf32InstrDesc, (kb | k) ? 1u : 0u);
        tc_commit(&empty_bar[s]);
      }
      if (ok) tc_commit(&accum_bar);
    }
  } else {
    const int quarter = warp & 3, r = quarter * 32 + lane;
    const bool have = (num_kb == 0) || mbar_wait(&accum_bar, 0, &abort_flag);
    tc_fence_after();
    if (have) {
      // every load has landed and every MMA has retired: the ring is free and stages the output tile as four
      // [128 rows x 32 fp32] boxes in the swizzled layout the bulk store expects
#pragma unroll 1
      for (int cb = 0; cb < TBN / 32; ++cb) {
        uint32_t acc[32];
        if (num_kb > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cb * 32), acc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0u;
        }
        uint8_t* box = tiles + cb * kTTileBytes;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *(float4*)(box + swz(r, q)) =
              make_float4(__uint_as_float(acc[q * 4]) * alpha, __uint_as_float(acc[q * 4 + 1]) * alpha,
                          __uint_as_float(acc[q * 4 + 2]) * alpha, __uint_as_float(acc[q * 4 + 3]) * alpha);
      }
    }
    tc_fence_before();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (have && warp == 2 && lane == 0) {
#pragma unroll
      for (int cb = 0; cb < TBN / 32; ++cb)
        if (tn * TBN + cb * 32 < N) tma_store_3d(&map_c, tiles + cb * kTTileBytes, tn * TBN + cb * 32, tm * TBM, batch);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
  }

  if (warp == 0 && lane == 0 && abort_flag) {  // let in-flight loads land before the CTA's shared memory goes away
    for (int kb = max(0, issued - kTStages); kb < issued; ++kb) {
      const int s = kb % kTStages, round = kb / kTStages;
      for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(&full_bar[s], round & 1)) break;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && status != nullptr) atomicExch(status, 1);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, kTTmemCols); }
}

__device__ __forceinline__ float tf32_hi(float x) {
  uint32_t bits;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x));
  return __uint_as_float(bits);
}

// One block moves a 64 x 64 tile of the source through shared memory and writes the three K segments of the
// operand rows it covers.  k runs over the source columns (transpose = 0) or rows (transpose = 1); the range
// [K, kp) of every segment is zero-filled.  256 threads = 16 float4 lanes x 16 rows, four passes each way; global
// accesses are 16 bytes wide (the source falls back to scalars when its rows are not 16-byte aligned).
// Grid: (ceil(kp / 64), ceil(rows / 64), batch).
__global__ void __launch_bounds__(256) tf32_split_kernel(const float* __restrict__ src, int64_t ld_src, int64_t stride_src,
                                                        int R, int C, int transpose, int role_b, float* __restrict__ dst,
                                                        int rows, int K, int kp) {
  __shared__ float tile[64][65];  // [operand row][k]
  const float* s = src + (int64_t)blockIdx.z * stride_src;
  float* d = dst + (int64_t)blockIdx.z * rows * 3 * kp;
  const int k0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int lane4 = (threadIdx.x & 15) * 4, line = threadIdx.x >> 4;
  const bool vec_ok = (ld_src & 3) == 0 && (stride_src & 3) == 0 && (((uintptr_t)src) & 15) == 0;
  // source tile: `line` walks the source rows, `lane4` the (contiguous) source columns
  const int src_row0 = transpose ? k0 : r0, src_col0 = transpose ? r0 : k0;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int lr = line + 16 * pass, sr = src_row0 + lr, sc = src_col0 + lane4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (sr < R) {
      const float* row = s + (int64_t)sr * ld_src;
      if (vec_ok && sc + 3 < C) {
        const float4 t = *reinterpret_cast<const float4*>(row + sc);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (sc + e < C) v[e] = row[sc + e];
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (transpose) tile[lane4 + e][lr] = v[e];
      else tile[lr][lane4 + e] = v[e];
    }
  }
  __syncthreads();
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int lr = line + 16 * pass, r = r0 + lr, k = k0 + lane4;
    if (r >= rows || k >= kp) continue;  // kp is a multiple of 32, so a float4 never straddles it
    float hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x = tile[lr][lane4 + e];
      // lo is rounded to tf32 here (the tensor core would truncate it): halves the error of the two cross terms
      hi[e] = tf32_hi(x);
      lo[e] = tf32_hi(x - hi[e]);
    }
    const float4 h4 = make_float4(hi[0], hi[1], hi[2], hi[3]), l4 = make_float4(lo[0], lo[1], lo[2], lo[3]);
    float* row = d + (int64_t)r * 3 * kp + k;
    *reinterpret_cast<float4*>(row) = h4;
    *reinterpret_cast<float4*>(row + kp) = role_b ? l4 : h4;
    *reinterpret_cast<float4*>(row + 2 * kp) = role_b ? h4 : l4;
  }
}

// fp32 tensor [batch, rows, cols], row stride ld elements; box = 32 columns x 128 rows, 128-byte swizzle.
bool make_f32_map(CUtensorMap* map, const void* base, int rows, int64_t cols, int64_t ld, int64_t batch_stride, int batch) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)batch_stride * 4};
  cuuint32_t box[3] = {TBK, TBM, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_tf32_split(const float* src, int64_t ld_src, int64_t stride_src, int R, int C, int batch, int transpose,
                              int role_b, float* dst, cudaStream_t stream) {
  const int rows = transpose ? C : R, K = transpose ? R : C;
  const int kp = (int)tf32_split_kp(K);
  if (rows == 0 || batch == 0) return cudaSuccess;
  dim3 grid((kp + 63) / 64, (rows + 63) / 64, batch);
  tf32_split_kernel<<<grid, 256, 0, stream>>>(src, ld_src, stride_src, R, C, transpose, role_b, dst, rows, K, kp);
  return cudaGetLastError();
}

cudaError_t launch_tf32_gemm(const float* A3, const float* B3, int M, int N, int K, int batch, float alpha, float* C,
                             int64_t ldc, int64_t strideC, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tf32_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  if (M == 0 || N == 0 || batch == 0) return cudaSuccess;
  const int64_t k3 = 3 * tf32_split_kp(K);
  CUtensorMap ma, mb, mc;
  if (!make_f32_map(&ma, A3, M, k3, k3, (int64_t)M * k3, batch) || !make_f32_map(&mb, B3, N, k3, k3, (int64_t)N * k3, batch) ||
      !make_f32_map(&mc, C, M, N, ldc, strideC, batch))
    return cudaErrorInvalidValue;
  dim3 grid(((M + TBM - 1) / TBM) * ((N + TBN - 1) / TBN), batch);
  tf32_gemm_kernel<<<grid, kTThreads, kTSmemBytes, stream>>>(ma, mb, mc, M, N, (int)k3, alpha, status);
  return cudaGetLastError();
}

}  // namespace hb
