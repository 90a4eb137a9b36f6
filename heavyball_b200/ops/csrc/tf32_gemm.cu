// fp32-in / fp32-out batched GEMM at near-fp32 accuracy on the tf32 tensor-core path of sm_100a ("3xTF32"), with the
// element-wise stages of SOAP and PSGD fused into its epilogue.
//
// The preconditioner algebra of SOAP and PSGD (eigenbasis projections, Gram statistics, Kronecker factor
// products; heavyball/utils.py:1205-1259, 1391-1411, 3084-3122, 3557-3576 of the reference run them as fp32 cuBLAS
// einsums) needs more than tf32's 10 mantissa bits, and fp32 SIMT GEMMs run at a twentieth of the tensor-core rate.
// Each operand is therefore split once into hi = tf32(x) and lo = tf32(x - hi), stored side by side as rows of
// [hi | lo], and the product is taken as
//     A B^T ~= hi_a hi_b^T + hi_a lo_b^T + lo_a hi_b^T
// by walking A as (hi, hi, lo) and B as (hi, lo, hi) along K: ONE K-major tf32 GEMM over 3K with a single fp32
// accumulator in tensor memory.  The dropped lo*lo term and the rounding of lo to tf32 are both below 2^-21.
// Measured error: about 2^-18 of |A||B|^T for K = 2048 (fp32 SIMT: 2^-21, one tf32 pass: 2^-11); it is set by the
// rounding of the tensor core's accumulator.  One split buffer serves as either operand, so a symmetric product
// X X^T needs one split of X, and matrices that change rarely (eigenbases, preconditioner factors) stay split.
//
// GEMM kernel (one 128x128 output tile per CTA, 192 threads, two CTAs per SM):
//   warp 0     : TMA producer, cp.async.bulk.tensor 3-D loads (128-byte swizzle, 32 fp32 per row) into a 3-stage ring
//   warp 1     : tcgen05.mma.cta_group::1.kind::tf32, 128x128x8 per instruction, accumulator in 128 TMEM columns
//   warps 2..5 : tcgen05.ld, then the epilogue.  Plain stores go through the (now idle) ring and four bulk tensor
//                stores.  Fused epilogues work in registers and store directly: scale; lerp into the statistics
//                matrix (GG <- lerp(GG, G G^T)); Adam / LaProp in the eigenbasis (moments read and written in
//                place, the preconditioned value goes on); and, for any of them, the result written in the split
//                [hi | lo] layout - as it is or transposed - so the next product of the chain needs no split pass.
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

__device__ __forceinline__ float tf32_hi(float x) {
  uint32_t bits;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x));
  return __uint_as_float(bits);
}

__device__ __forceinline__ float lerp_w(float s, float x, float w) { return s * (1.0f - w) + x * w; }

constexpr int kStageLd = 36;                         // floats per staged row: rows stay 16-byte aligned and float4
                                                     // accesses of a quarter-warp fall into distinct banks
constexpr int kStageWarpBytes = 32 * kStageLd * 4;   // one warp's 32 rows x 32 columns

// Fused epilogue of one warp: its 32 accumulator rows of the 128x128 tile, 32 columns at a time.  A thread reads
// its own row from tensor memory; global memory wants the other orientation (consecutive lanes on consecutive
// columns), so the block is turned through the warp's `stage` in shared memory (the idle operand ring):
//   pass 1 (lane = row):                   accumulators * alpha -> stage
//   pass 2 (8 lanes per row, 4 rows/step): moments, lerp, C store, split-operand store - every global access is a full
//                                          128-byte line per row; the final values go back to the stage when needed
//   pass 3 (lane = row):                   outputs that run along the rows: transposed split operand, mirror tile
// Values outside [M, N] are never stored; the zero padding of a split output (columns [K, kp) of the operand being
// produced) is.
// `tmem_warp`: tensor-memory address of the warp's first row and the tile's first column; `row0` / `col_base`: their
// global indices; `n_cb`: 32-column blocks in the tile; `off_diagonal`: the tile is not on the diagonal (mirror stores).
// `zero_acc`: the tile had no product (its accumulator was never written): the values are zeros.
__device__ __forceinline__ void epilogue_direct(uint32_t tmem_warp, int lane, float* stage, int row0, int col_base, int n_cb,
                                                bool off_diagonal, bool zero_acc, int batch, int M, int N,
                                                const Tf32Epilogue& E) {
  const int64_t b64 = batch;
  const bool state_vec = (N & 3) == 0;
  const bool c_vec = (E.ldc & 3) == 0 && ((E.strideC & 3) == 0) && ((((uintptr_t)E.C) & 15) == 0);
  const bool moments = E.mode == kEpiAdam || E.mode == kEpiLaProp;
  const bool mirror = E.symmetric && off_diagonal && E.C != nullptr;
  const bool along_rows = mirror || (E.S != nullptr && E.s_transposed);
  const bool s_rows = E.S != nullptr && !E.s_transposed;
  const int sub = lane >> 3, cg = (lane & 7) * 4;
  const float w1 = 1.0f - E.b1, w2 = 1.0f - E.b2;
  float* mine = stage + lane * kStageLd;
#pragma unroll 1
  for (int cb = 0; cb < n_cb; ++cb) {
    const int col0 = col_base + cb * 32;
    {
      uint32_t acc[32];
      if (!zero_acc) {
        tmem_ld32(tmem_warp + (uint32_t)(cb * 32), acc);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *(float4*)(mine + q * 4) =
            make_float4(__uint_as_float(acc[q * 4]) * E.alpha, __uint_as_float(acc[q * 4 + 1]) * E.alpha,
                        __uint_as_float(acc[q * 4 + 2]) * E.alpha, __uint_as_float(acc[q * 4 + 3]) * E.alpha);
    }
    __syncwarp();

    const int col = col0 + cg;
    // What the epilogue reads from global memory (moments, or the old value of C) is fetched four steps at a time
    // before the first of them is used: a step-by-step load -> compute -> store chain pays one memory round trip per step
    // (stores may alias the next step's loads, so the compiler cannot hoist them), which for the small products of a
    // blocked solve was longer than the product itself.
    const bool fast_state = moments && state_vec && col + 3 < N;
    const bool fast_old = (E.mode == kEpiLerp || E.mode == kEpiAdd) && E.C != nullptr && c_vec && col + 3 < N;
    float4 pa[4], pb[4];
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
    if (fast_state || fast_old) {
#pragma unroll
      for (int i4 = 0; i4 < 4; ++i4) {
        const int row = row0 + (half * 4 + i4) * 4 + sub;
        pa[i4] = make_float4(0.f, 0.f, 0.f, 0.f);
        pb[i4] = pa[i4];
        if (row < M) {
          if (fast_state) {
            pa[i4] = *(const float4*)(E.m + (b64 * M + row) * (int64_t)N + col);
            pb[i4] = *(const float4*)(E.v + (b64 * M + row) * (int64_t)N + col);
          } else {
            pa[i4] = *(const float4*)(E.C + b64 * E.strideC + (int64_t)row * E.ldc + col);
          }
        }
      }
    }
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
      const int it = half * 4 + i4;
      const int lr = it * 4 + sub, row = row0 + lr;
      float* sp = stage + lr * kStageLd + cg;
      const float4 x4 = *(const float4*)sp;
      float x[4] = {x4.x, x4.y, x4.z, x4.w};
      if (row < M && col < N) {
        if (moments) {
          float* mp = E.m + (b64 * M + row) * (int64_t)N + col;
          float* vp = E.v + (b64 * M + row) * (int64_t)N + col;
          const bool fast = fast_state;
          float m4[4], s4[4];
          if (fast) {
            const float4 a = pa[i4], c = pb[i4];
            m4[0] = a.x; m4[1] = a.y; m4[2] = a.z; m4[3] = a.w;
            s4[0] = c.x; s4[1] = c.y; s4[2] = c.z; s4[3] = c.w;
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              m4[e] = col + e < N ? mp[e] : 0.f;
              s4[e] = col + e < N ? vp[e] : 0.f;
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s4[e] = lerp_w(s4[e], x[e] * x[e], w2);
            const float d = fmaxf(sqrtf(s4[e]), E.eps);
            if (E.mode == kEpiAdam) {
              m4[e] = lerp_w(m4[e], x[e], w1);
              x[e] = m4[e] / d;
            } else {
              m4[e] = lerp_w(m4[e], x[e] / d, w1);
              x[e] = m4[e];
            }
          }
          if (fast) {
            *(float4*)mp = make_float4(m4[0], m4[1], m4[2], m4[3]);
            *(float4*)vp = make_float4(s4[0], s4[1], s4[2], s4[3]);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < N) { mp[e] = m4[e]; vp[e] = s4[e]; }
          }
        }
        if (E.C != nullptr) {
          float* cp = E.C + b64 * E.strideC + (int64_t)row * E.ldc + col;
          const bool fast = c_vec && col + 3 < N;
          if (E.mode == kEpiLerp || E.mode == kEpiAdd) {
            // lerp: o + (x - o) w;  add: o + x  (the same expression with the old value left out of the difference)
            const float keep = E.mode == kEpiLerp ? 1.f : 0.f, w = E.mode == kEpiLerp ? E.w : 1.f;
            if (fast) {
              const float4 o = pa[i4];
              x[0] = o.x + (x[0] - keep * o.x) * w; x[1] = o.y + (x[1] - keep * o.y) * w;
              x[2] = o.z + (x[2] - keep * o.z) * w; x[3] = o.w + (x[3] - keep * o.w) * w;
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (col + e < N) { const float o = cp[e]; x[e] = o + (x[e] - keep * o) * w; }
            }
          }
          if (fast) {
            *(float4*)cp = make_float4(x[0], x[1], x[2], x[3]);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < N) cp[e] = x[e];
          }
        }
      }
      if (s_rows && row < M && col < E.kpS) {  // operand rows = output rows, K over the output columns (zero from N to kp)
        float* srow = E.S + b64 * E.strideS + (int64_t)row * (2 * E.kpS) + col;
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float y = col + e < N ? x[e] : 0.f;
          hi[e] = tf32_hi(y);
          lo[e] = tf32_hi(y - hi[e]);
        }
        *(float4*)srow = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *(float4*)(srow + E.kpS) = make_float4(lo[0], lo[1], lo[2], lo[3]);
      }
      if (along_rows) *(float4*)sp = make_float4(x[0], x[1], x[2], x[3]);
    }
    }

    if (along_rows) {
      __syncwarp();
      const int row = row0 + lane;
      float v[32];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 t = *(const float4*)(mine + q * 4);
        v[q * 4] = t.x; v[q * 4 + 1] = t.y; v[q * 4 + 2] = t.z; v[q * 4 + 3] = t.w;
      }
      if (mirror && row < M) {  // consecutive lanes hold consecutive rows: one accumulator column is one contiguous line
        float* ccol = E.C + b64 * E.strideC + row;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < N) ccol[(int64_t)(col0 + j) * E.ldc] = v[j];
      }
      if (E.S != nullptr && E.s_transposed && row < E.kpS) {
        // operand rows = output columns, K over the output rows (zero from M up to kp)
        float* sb = E.S + b64 * E.strideS + row;
        const int64_t ld = 2 * E.kpS;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < N) {
            const float y = row < M ? v[j] : 0.f;
            const float hi = tf32_hi(y);
            float* dst = sb + (int64_t)(col0 + j) * ld;
            dst[0] = hi;
            dst[E.kpS] = tf32_hi(y - hi);
          }
        }
      }
    }
    __syncwarp();  // the stage is rewritten by the next block of columns
  }
}

__global__ void __launch_bounds__(kTThreads, 2)
tf32_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, int M, int N, int kp, const Tf32Epilogue E, int bulk_store,
                 int* status) {
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
  int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  if (E.symmetric) {  // blockIdx.x counts the tiles on or above the diagonal, row by row
    int left = blockIdx.x;
    tm = 0;
    while (left >= tiles_n - tm) { left -= tiles_n - tm; ++tm; }
    tn = tm + left;
  }
  const int batch = blockIdx.y;
  int kb_lo = 0, kb_hi = kp / TBK;  // K blocks of one term of the split product that this tile walks
  if (E.tri) {
    kb_lo = min(kb_hi, tm * (TBM / TBK));
    kb_hi = tn < tm ? kb_lo : min(kb_hi, (tn + 1) * (TBN / TBK));
  }
  const int seg_kb = kb_hi - kb_lo;
  const int num_kb = 3 * seg_kb;    // hi*hi, hi*lo, lo*hi
  const float alpha = E.alpha;

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
        const int seg = kb / seg_kb, k0 = (kb_lo + kb - seg * seg_kb) * TBK;
        mbar_expect_tx(&full_bar[s], kTStageBytes);
        tma_load_3d(dst, &map_a, &full_bar[s], k0 + (seg == 2 ? kp : 0), tm * TBM, batch);               // hi, hi, lo
        tma_load_3d(dst + kTTileBytes, &map_b, &full_bar[s], k0 + (seg == 1 ? kp : 0), tn * TBN, batch);  // hi, lo, hi
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
    if (have && bulk_store) {
      // every load has landed and every MMA has retired: the ring is free and stages the output tile as four
      // [128 rows x 32 fp32] boxes in the swizzled layout the bulk store expects
#pragma unroll 1
      for (int cb = 0; cb < TBN / 32; ++cb) {
        uint32_t acc[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cb * 32), acc);
        tmem_ld_wait();
        uint8_t* box = tiles + cb * kTTileBytes;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *(float4*)(box + swz(r, q)) =
              make_float4(__uint_as_float(acc[q * 4]) * alpha, __uint_as_float(acc[q * 4 + 1]) * alpha,
                          __uint_as_float(acc[q * 4 + 2]) * alpha, __uint_as_float(acc[q * 4 + 3]) * alpha);
      }
    } else if (have) {
      epilogue_direct(tmem_base + ((uint32_t)(quarter * 32) << 16), lane, (float*)(tiles + quarter * kStageWarpBytes),
                      tm * TBM + quarter * 32, tn * TBN, TBN / 32, tm != tn, num_kb == 0, batch, M, N, E);
    }
    tc_fence_before();
    if (bulk_store) {
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

// ------------------------------------------------------------------------------------------ 256 x 256 tiles
// A 128 x 128 tile asks the L2 for 32 KiB of operands per 256 tensor-core cycles (tf32 runs at half the bf16 rate on
// operands twice as wide), which is more than the L2 delivers to 148 SMs at once; a 256 x 256 tile needs half of that
// per FLOP.  One CTA per SM: four 128 x 128 fp32 accumulators = all 512 columns of tensor memory, 64 KiB ring stages
// (two 128-row boxes per operand), two 128 x 256 x 8 instructions per 8 of K sharing the B rows.  Eight epilogue
// warps: two per 32-lane quarter of tensor memory, one for each 128-row half of the tile.
constexpr int TBM2 = 256, TBN2 = 256;
constexpr int kTStageBytes2 = 4 * kTTileBytes;                  // 64 KiB
constexpr int kTSmemBytes2 = kTStages * kTStageBytes2 + 1024;
constexpr int kTThreads2 = 320;                                 // producer, MMA, 8 epilogue warps
constexpr uint32_t kTTmemCols2 = 512;
constexpr uint32_t kTf32InstrDesc256 =
    (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TBN2 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__global__ void __launch_bounds__(kTThreads2, 1)
tf32_gemm256_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, int M, int N, int kp,
                    const Tf32Epilogue E, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kTStages];
  __shared__ __align__(8) uint64_t empty_bar[kTStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  if (status != nullptr && *(volatile const int*)status != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tiles_n = (N + TBN2 - 1) / TBN2;
  int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  if (E.symmetric) {
    int left = blockIdx.x;
    tm = 0;
    while (left >= tiles_n - tm) { left -= tiles_n - tm; ++tm; }
    tn = tm + left;
  }
  const int batch = blockIdx.y;
  int kb_lo = 0, kb_hi = kp / TBK;
  if (E.tri) {
    kb_lo = min(kb_hi, tm * (TBM2 / TBK));
    kb_hi = tn < tm ? kb_lo : min(kb_hi, (tn + 1) * (TBN2 / TBK));
  }
  const int seg_kb = kb_hi - kb_lo;
  const int num_kb = 3 * seg_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, kTTmemCols2); tmem_relinquish(); }
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
        uint8_t* dst = tiles + s * kTStageBytes2;
        const int seg = kb / seg_kb, k0 = (kb_lo + kb - seg * seg_kb) * TBK;
        const int ka = k0 + (seg == 2 ? kp : 0), kb_col = k0 + (seg == 1 ? kp : 0);   // A: hi, hi, lo   B: hi, lo, hi
        mbar_expect_tx(&full_bar[s], kTStageBytes2);   // rows past the operand's end arrive as zeros and count as bytes
        tma_load_3d(dst, &map_a, &full_bar[s], ka, tm * TBM2, batch);
        tma_load_3d(dst + kTTileBytes, &map_a, &full_bar[s], ka, tm * TBM2 + 128, batch);
        tma_load_3d(dst + 2 * kTTileBytes, &map_b, &full_bar[s], kb_col, tn * TBN2, batch);
        tma_load_3d(dst + 3 * kTTileBytes, &map_b, &full_bar[s], kb_col, tn * TBN2 + 128, batch);
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
        const uint32_t base = smem_u32(tiles + s * kTStageBytes2);
        const uint64_t a_top = make_smem_desc(base), a_bot = make_smem_desc(base + kTTileBytes);
        // 256 B rows = 32 eight-row groups, 1 KiB apart: the two 128-row boxes are contiguous
        const uint64_t b_desc = make_smem_desc(base + 2 * kTTileBytes);
#pragma unroll
        for (int k = 0; k < TBK / 8; ++k) {
          const uint32_t acc = (kb | k) ? 1u : 0u;
          tc_mma_tf32(tmem_base, a_top + 2 * k, b_desc + 2 * k, kTf32InstrDesc256, acc);
          tc_mma_tf32(tmem_base + 256u, a_bot + 2 * k, b_desc + 2 * k, kTf32InstrDesc256, acc);
        }
        tc_commit(&empty_bar[s]);
      }
      if (ok) tc_commit(&accum_bar);
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;   // warps 2..5: rows 0..127 of the tile, warps 6..9: rows 128..255
    const bool have = (num_kb == 0) || mbar_wait(&accum_bar, 0, &abort_flag);
    tc_fence_after();
    const int row0 = tm * TBM2 + half * 128 + quarter * 32;
    if (have && row0 < M)
      epilogue_direct(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 256), lane,
                      (float*)(tiles + (warp - 2) * kStageWarpBytes), row0, tn * TBN2, TBN2 / 32, tm != tn, num_kb == 0,
                      batch, M, N, E);
    tc_fence_before();
  }

  if (warp == 0 && lane == 0 && abort_flag) {
    for (int kb = max(0, issued - kTStages); kb < issued; ++kb) {
      const int s = kb % kTStages, round = kb / kTStages;
      for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(&full_bar[s], round & 1)) break;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && status != nullptr) atomicExch(status, 1);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, kTTmemCols2); }
}

// One block moves a 64 x 64 tile of the source through shared memory and writes the [hi | lo] rows it covers of either
// or both operand orientations (see tf32_gemm.h).  The zero padding [K, kp) of every row is written too.  256 threads
// = 16 float4 lanes x 16 rows, four passes each way; global accesses are 16 bytes wide (the source falls back to
// scalars when its rows are not 16-byte aligned).  Grid: (ceil(kp(C) / 64), ceil(kp(R) / 64), batch).
__global__ void __launch_bounds__(256) tf32_split_kernel(const float* __restrict__ src, int64_t ld_src, int64_t stride_src,
                                                        int R, int C, float* __restrict__ dst_same,
                                                        float* __restrict__ dst_trans, int kpC, int kpR) {
  __shared__ float tile[64][65];  // [source row][source column]
  const float* s = src + (int64_t)blockIdx.z * stride_src;
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int lane4 = (threadIdx.x & 15) * 4, line = threadIdx.x >> 4;
  const bool vec_ok = (ld_src & 3) == 0 && (stride_src & 3) == 0 && (((uintptr_t)src) & 15) == 0;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int lr = line + 16 * pass, sr = r0 + lr, sc = c0 + lane4;
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
    for (int e = 0; e < 4; ++e) tile[lr][lane4 + e] = v[e];
  }
  __syncthreads();
  if (dst_same != nullptr) {  // rows = source rows, k = source columns
    float* d = dst_same + (int64_t)blockIdx.z * R * 2 * kpC;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int lr = line + 16 * pass, r = r0 + lr, k = c0 + lane4;
      if (r >= R || k >= kpC) continue;  // kp is a multiple of 32, so a float4 never straddles it
      float hi[4], lo[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x = tile[lr][lane4 + e];
        // lo is rounded to tf32 here (the tensor core would truncate it): halves the error of the two cross terms
        hi[e] = tf32_hi(x);
        lo[e] = tf32_hi(x - hi[e]);
      }
      float* row = d + (int64_t)r * 2 * kpC + k;
      *reinterpret_cast<float4*>(row) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<float4*>(row + kpC) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
  if (dst_trans != nullptr) {  // rows = source columns, k = source rows
    float* d = dst_trans + (int64_t)blockIdx.z * C * 2 * kpR;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int lc = line + 16 * pass, c = c0 + lc, k = r0 + lane4;
      if (c >= C || k >= kpR) continue;
      float hi[4], lo[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x = tile[lane4 + e][lc];
        hi[e] = tf32_hi(x);
        lo[e] = tf32_hi(x - hi[e]);
      }
      float* row = d + (int64_t)c * 2 * kpR + k;
      *reinterpret_cast<float4*>(row) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<float4*>(row + kpR) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
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

cudaError_t launch_tf32_split(const float* src, int64_t ld_src, int64_t stride_src, int R, int C, int batch, float* dst_same,
                              float* dst_trans, cudaStream_t stream) {
  if (R == 0 || C == 0 || batch == 0 || (dst_same == nullptr && dst_trans == nullptr)) return cudaSuccess;
  const int kpC = (int)tf32_split_kp(C), kpR = (int)tf32_split_kp(R);
  dim3 grid((kpC + 63) / 64, (kpR + 63) / 64, batch);
  tf32_split_kernel<<<grid, 256, 0, stream>>>(src, ld_src, stride_src, R, C, dst_same, dst_trans, kpC, kpR);
  return cudaGetLastError();
}

static int g_tf32_tile_override = 0;  // 0 = by size, 128 / 256 = forced (tests and measurements)
int tf32_gemm_tile_override() { return g_tf32_tile_override; }
void set_tf32_gemm_tile_override(int tile) { g_tf32_tile_override = (tile == 128 || tile == 256) ? tile : 0; }

cudaError_t launch_tf32_gemm(const float* A2, const float* B2, int M, int N, int K, int batch, const Tf32Epilogue& E,
                             int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tf32_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(tf32_gemm256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmemBytes2);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  if (M == 0 || N == 0 || batch == 0) return cudaSuccess;
  if ((E.mode == kEpiAdam || E.mode == kEpiLaProp) && (E.m == nullptr || E.v == nullptr)) return cudaErrorInvalidValue;
  if ((E.mode == kEpiLerp || E.mode == kEpiAdd) && E.C == nullptr) return cudaErrorInvalidValue;
  if (E.tri && (M != N || M != K || E.symmetric)) return cudaErrorInvalidValue;
  if (E.symmetric && (A2 != B2 || M != N || E.C == nullptr || E.S != nullptr || (E.mode != kEpiStore && E.mode != kEpiLerp && E.mode != kEpiAdd)))
    return cudaErrorInvalidValue;
  const int64_t kp = tf32_split_kp(K), ld = 2 * kp;
  CUtensorMap ma, mb, mc;
  if (!make_f32_map(&ma, A2, M, ld, ld, (int64_t)M * ld, batch) || !make_f32_map(&mb, B2, N, ld, ld, (int64_t)N * ld, batch))
    return cudaErrorInvalidValue;

  // big tiles once there are enough of them to fill the machine (one CTA per SM) and K is long enough to pay for a
  // serial epilogue; small problems keep 128 x 128 tiles, two CTAs per SM
  const int big_m = (M + TBM2 - 1) / TBM2, big_n = (N + TBN2 - 1) / TBN2;
  const int64_t big_tiles = (int64_t)(E.symmetric ? big_n * (big_n + 1) / 2 : big_m * big_n) * batch;
  bool big = M >= TBM2 && N >= TBN2 && K >= 512 && big_tiles >= 96;
  if (g_tf32_tile_override == 128) big = false;
  if (g_tf32_tile_override == 256) big = true;
  if (big) {
    dim3 grid(E.symmetric ? big_n * (big_n + 1) / 2 : big_m * big_n, batch);
    tf32_gemm256_kernel<<<grid, kTThreads2, kTSmemBytes2, stream>>>(ma, mb, M, N, (int)kp, E, status);
    return cudaGetLastError();
  }

  // plain products leave through the bulk-store path; everything else is written by the epilogue threads themselves
  const int bulk = (!E.symmetric && !E.tri && E.mode == kEpiStore && E.S == nullptr && E.C != nullptr && (E.ldc & 3) == 0 &&
                    (E.strideC & 3) == 0 && (((uintptr_t)E.C) & 15) == 0) ? 1 : 0;
  mc = ma;  // placeholder when the bulk-store path is not taken (never dereferenced then)
  if (bulk && !make_f32_map(&mc, E.C, M, N, E.ldc, E.strideC, batch)) return cudaErrorInvalidValue;
  const int tiles_m = (M + TBM - 1) / TBM, tiles_n = (N + TBN - 1) / TBN;
  dim3 grid(E.symmetric ? tiles_n * (tiles_n + 1) / 2 : tiles_m * tiles_n, batch);
  tf32_gemm_kernel<<<grid, kTThreads, kTSmemBytes, stream>>>(ma, mb, mc, M, N, (int)kp, E, bulk, status);
  return cudaGetLastError();
}

}  // namespace hb
