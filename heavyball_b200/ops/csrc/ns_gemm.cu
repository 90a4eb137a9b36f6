// Newton–Schulz / Polar-Express building blocks for sm_100a.
//
// One polynomial step X <- (a I + b S + c S^2) X with S = X X^T (heavyball/utils.py:550-577, 605-631)
// is executed as three batched bf16 GEMMs with fp32 accumulation in tensor memory:
//     gram : S  = X  X^T                       (symmetric: upper-triangular tiles only, mirrored)
//     poly : Y  = c S S + b S + a I            (symmetric; S is both operands and an epilogue input)
//     apply: X' = Y X                          (also writes X'^T, the K-major operand of the next step)
// All three are "TN" products D[M,N] = A[M,K] * B[N,K]^T with both operands K-major, so a single
// kernel serves them; only the epilogue differs.  Keeping X^T alongside X is what makes the third
// product K-major as well.
//
// Kernel structure (one 128x128 output tile per CTA, 192 threads, two CTAs resident per SM so one
// CTA's epilogue overlaps the other's main loop):
//   warp 0      : TMA producer  - cp.async.bulk.tensor (3-D maps, 128B swizzle) into a 3-stage ring
//   warp 1      : MMA issuer    - tcgen05.mma.cta_group::1.kind::f16, 128x128x16 per instruction,
//                                 accumulator = 128 TMEM columns; tcgen05.commit releases ring slots
//   warps 2..5  : epilogue      - tcgen05.ld 32x32b from their TMEM lane quarter, fused scalar math (the
//                                 S tile of the polynomial arrives by TMA in a freed ring slot), bf16
//                                 tile and its transpose staged in swizzled shared memory and written
//                                 with cp.async.bulk.tensor stores; fp32 final output stored directly
// Every mbarrier wait is bounded; on expiry the CTA raises a flag in global memory, drains what it
// issued, frees its TMEM columns and returns, so a protocol bug cannot wedge the device.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "ns_gemm.h"

#include <mutex>
#include <unordered_map>
#include "tc_common.cuh"

namespace hb {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 3;
constexpr int kTileBytes = BM * BK * 2;            // 16 KiB per operand tile
constexpr int kStageBytes = 2 * kTileBytes;        // A + B
constexpr int kSmemBytes = kStages * kStageBytes + 1024;  // + slack for 1 KiB alignment
constexpr int kGemmThreads = 192;
constexpr uint32_t kTmemCols = 128;

// bf16 x bf16 -> fp32, both operands K-major, M = 128, N = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// ------------------------------------------------------------------------------------------ kernel
__global__ void __launch_bounds__(kGemmThreads, 2)
ns_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_ct, const GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  // a previous CTA of this stream already gave up on a wait: do not pile more work on a broken pipeline
  if (P.status != nullptr && *(volatile const int*)P.status != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  // ---- tile coordinates
  const int tiles_m = (P.M + BM - 1) / BM, tiles_n = (P.N + BN - 1) / BN;
  int tm, tn;
  if (P.symmetric) {
    int idx = blockIdx.x;
    tm = 0;
    while (idx >= tiles_m - tm) { idx -= tiles_m - tm; ++tm; }
    tn = tm + idx;
  } else {
    tm = blockIdx.x / tiles_n;
    tn = blockIdx.x % tiles_n;
  }
  const int batch = blockIdx.y;
  const int num_kb = (P.K + BK - 1) / BK;
  const bool poly = P.mode == kModePoly;
  const bool same_ab = P.same_operand && tm == tn;  // A and B tiles coincide
  // after the main loop the ring is reused: slot sx receives the S tile (poly), the next two stage
  // the output tile and its transpose for the bulk stores
  const int sx = num_kb % kStages;
  uint8_t* s_tile = tiles + sx * kStageBytes;
  uint8_t* c_stage = tiles + ((sx + 1) % kStages) * kStageBytes;
  uint8_t* ct_stage = tiles + ((sx + 2) % kStages) * kStageBytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int issued = 0;  // producer: ring fills whose loads were issued
  if (warp == 0) {
    if (lane == 0) {
      const int total = num_kb + (poly ? 1 : 0);
      for (int kb = 0; kb < total; ++kb) {
        const int s = kb % kStages, round = kb / kStages;
        if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &abort_flag)) break;
        uint8_t* a_dst = tiles + s * kStageBytes;
        if (kb < num_kb) {
          // diagonal tiles of a symmetric product multiply a row block with itself: one load feeds both operands
          mbar_expect_tx(&full_bar[s], same_ab ? kTileBytes : kStageBytes);
          tma_load_3d(a_dst, &map_a, &full_bar[s], kb * BK, tm * BM, batch);
          if (!same_ab) tma_load_3d(a_dst + kTileBytes, &map_b, &full_bar[s], kb * BK, tn * BN, batch);
        } else {
          mbar_expect_tx(&full_bar[s], kStageBytes);  // S[tm-block, tn-block] for the polynomial epilogue, as two 64-column halves
          tma_load_3d(a_dst, &map_a, &full_bar[s], tn * BN, tm * BM, batch);
          tma_load_3d(a_dst + kTileBytes, &map_a, &full_bar[s], tn * BN + BK, tm * BM, batch);
        }
        issued = kb + 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kStages, round = kb / kStages;
        ok = mbar_wait(&full_bar[s], round & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * kStageBytes);
        const uint64_t a_desc = make_smem_desc(a_addr), b_desc = same_ab ? a_desc : make_smem_desc(a_addr + kTileBytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // advancing 16 bf16 (32 B) along K inside the swizzle atom = +2 in 16-byte address units
          tc_mma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kInstrDesc, (kb | k) ? 1u : 0u);
        }
        tc_commit(&empty_bar[s]);
      }
      if (ok) tc_commit(&accum_bar);
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps (128 threads)
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int r = quarter * 32 + lane;       // row inside the tile
    const int row = tm * BM + r;             // global output row
    bool have = (num_kb == 0) || mbar_wait(&accum_bar, 0, &abort_flag);
    if (have && poly) have = mbar_wait(&full_bar[sx], (num_kb / kStages) & 1, &abort_flag);
    tc_fence_after();
    const bool mirror = P.symmetric ? (tn != tm) : true;
    const bool want_c = P.C != nullptr, want_ct = P.CT != nullptr && mirror;
    if (have) {
      const int64_t b64 = batch;
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; ++cb) {
        uint32_t acc[32];
        if (num_kb > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cb * 32), acc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0u;
        }
        const int half = cb >> 1, q0 = (cb & 1) * 4;  // 64-column half of the tile, first 16-byte chunk in it
        const int col0 = tn * BN + cb * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);

        if (poly) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 sv = *(const uint4*)(s_tile + half * kTileBytes + swz(r, q0 + q));
            const uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int j = q * 8 + e;
              const float sval = bf16_bits_to_float((uint16_t)((w[e >> 1] >> ((e & 1) * 16)) & 0xFFFF));
              v[j] = P.cc * v[j] + P.cb * sval + ((col0 + j == row) ? P.ca : 0.f);
            }
          }
        }
        // rounded once, so that the tile and its mirrored / transposed copy agree bit for bit
        uint16_t h[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) h[j] = rne_bf16_bits(v[j]);

        if (want_c) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = (uint32_t)h[q * 8 + 0] | ((uint32_t)h[q * 8 + 1] << 16);
            o.y = (uint32_t)h[q * 8 + 2] | ((uint32_t)h[q * 8 + 3] << 16);
            o.z = (uint32_t)h[q * 8 + 4] | ((uint32_t)h[q * 8 + 5] << 16);
            o.w = (uint32_t)h[q * 8 + 6] | ((uint32_t)h[q * 8 + 7] << 16);
            *(uint4*)(c_stage + half * kTileBytes + swz(r, q0 + q)) = o;
          }
        }
        if (want_ct) {  // transposed tile: row = column of the accumulator, column = r
          uint8_t* dst = ct_stage + (r >> 6) * kTileBytes + (r & 7) * 2;
          const int qr = (r & 63) >> 3;
#pragma unroll
          for (int j = 0; j < 32; ++j) *(uint16_t*)(dst + swz(cb * 32 + j, qr)) = h[j];
        }
        if (P.F != nullptr && row < P.M) {
          float* f = P.F + b64 * P.strideF;
          if (P.f_transposed) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < P.N) f[(int64_t)(col0 + j) * P.ldf + row] = bf16_bits_to_float(h[j]) * P.f_scale;
          } else {
            float* frow = f + (int64_t)row * P.ldf + col0;
            if (col0 + 32 <= P.N && (P.ldf & 3) == 0 && (((uintptr_t)f) & 15) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *(float4*)(frow + q * 4) =
                    make_float4(bf16_bits_to_float(h[q * 4]) * P.f_scale, bf16_bits_to_float(h[q * 4 + 1]) * P.f_scale,
                                bf16_bits_to_float(h[q * 4 + 2]) * P.f_scale, bf16_bits_to_float(h[q * 4 + 3]) * P.f_scale);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < P.N) frow[j] = bf16_bits_to_float(h[j]) * P.f_scale;
            }
          }
        }
      }
    }
    tc_fence_before();
    if (want_c || want_ct) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the bulk copy
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (have && warp == 2 && lane == 0) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (want_c && tn * BN + hh * BK < P.N)
            tma_store_3d(&map_c, c_stage + hh * kTileBytes, tn * BN + hh * BK, tm * BM, batch);
          if (want_ct && tm * BM + hh * BK < P.M)
            tma_store_3d(&map_ct, ct_stage + hh * kTileBytes, tm * BM + hh * BK, tn * BN, batch);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
    }
  }

  // ---- teardown: the producer makes sure nothing it issued is still landing in shared memory
  if (warp == 0 && lane == 0 && abort_flag) {
    for (int kb = max(0, issued - kStages); kb < issued; ++kb) {
      const int s = kb % kStages, round = kb / kStages;
      for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(&full_bar[s], round & 1)) break;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && P.status != nullptr) atomicExch(P.status, 1);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

// ------------------------------------------------------------------------------------------ large-tile kernel
// Same product, roles and barrier protocol with a 256x256 output tile per CTA (one CTA per SM).  A 128x128 tile reads
// 32 KiB of operands per 2.1 MFLOP k-block: at the tensor-core rate that is more than the L2 can deliver to 148 SMs, and
// large matrices (the 4096 x 14336 weights of an 8B model) stall at about 0.6 PFLOP/s.  A 256x256 tile reads 64 KiB per
// 8.4 MFLOP, half the bytes per flop, without any multicast: the CTA simply keeps four 128x128 accumulators - all 512
// columns of tensor memory - as two 128x256 instructions per 16 of K that share one B tile.  The price is that nothing is
// left to overlap the epilogue with, so this variant is chosen only when K is long enough to hide it.
//   ring stage : A rows 0..127 | A rows 128..255 | B rows 0..127 | B rows 128..255   (4 x 16 KiB, 3 stages = 192 KiB)
//   epilogue   : per 128-row half: [S half, poly only] | C staging | C^T staging      (3 x 64 KiB, the idle ring)
constexpr int BM2 = 256, BN2 = 256;
constexpr int kStageBytes2 = 4 * kTileBytes;                    // 64 KiB
constexpr int kSmemBytes2 = kStages * kStageBytes2 + 1024;
constexpr uint32_t kTmemCols2 = 512;
constexpr uint32_t kInstrDesc256 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__global__ void __launch_bounds__(kGemmThreads, 1)
ns_gemm256_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_ct, const GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  if (P.status != nullptr && *(volatile const int*)P.status != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  const int tiles_m = (P.M + BM2 - 1) / BM2, tiles_n = (P.N + BN2 - 1) / BN2;
  int tm, tn;
  if (P.symmetric) {
    int idx = blockIdx.x;
    tm = 0;
    while (idx >= tiles_m - tm) { idx -= tiles_m - tm; ++tm; }
    tn = tm + idx;
  } else {
    tm = blockIdx.x / tiles_n;
    tn = blockIdx.x % tiles_n;
  }
  const int batch = blockIdx.y;
  const int num_kb = (P.K + BK - 1) / BK;
  const bool poly = P.mode == kModePoly;
  const bool same_ab = P.same_operand && tm == tn;
  uint8_t* s_tile = tiles;                          // epilogue regions: the ring is idle by then
  uint8_t* c_stage = tiles + kStageBytes2;
  uint8_t* ct_stage = tiles + 2 * kStageBytes2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    mbar_init(&s_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, kTmemCols2); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int issued = 0;
  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages, round = kb / kStages;
        if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &abort_flag)) break;
        uint8_t* dst = tiles + s * kStageBytes2;
        mbar_expect_tx(&full_bar[s], same_ab ? 2 * kTileBytes : kStageBytes2);
        tma_load_3d(dst, &map_a, &full_bar[s], kb * BK, tm * BM2, batch);
        tma_load_3d(dst + kTileBytes, &map_a, &full_bar[s], kb * BK, tm * BM2 + 128, batch);
        if (!same_ab) {
          tma_load_3d(dst + 2 * kTileBytes, &map_b, &full_bar[s], kb * BK, tn * BN2, batch);
          tma_load_3d(dst + 3 * kTileBytes, &map_b, &full_bar[s], kb * BK, tn * BN2 + 128, batch);
        }
        issued = kb + 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kStages, round = kb / kStages;
        ok = mbar_wait(&full_bar[s], round & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t base = smem_u32(tiles + s * kStageBytes2);
        const uint64_t a_top = make_smem_desc(base), a_bot = make_smem_desc(base + kTileBytes);
        // 256 operand rows = 32 eight-row groups, 1 KiB apart: the two 128-row boxes are contiguous
        const uint64_t b_desc = same_ab ? a_top : make_smem_desc(base + 2 * kTileBytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint32_t acc = (kb | k) ? 1u : 0u;
          tc_mma_bf16(tmem_base, a_top + 2 * k, b_desc + 2 * k, kInstrDesc256, acc);
          tc_mma_bf16(tmem_base + 256u, a_bot + 2 * k, b_desc + 2 * k, kInstrDesc256, acc);
        }
        tc_commit(&empty_bar[s]);
      }
      if (ok) tc_commit(&accum_bar);
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    bool have = (num_kb == 0) || mbar_wait(&accum_bar, 0, &abort_flag);
    tc_fence_after();
    const bool mirror = P.symmetric ? (tn != tm) : true;
    const bool want_c = P.C != nullptr, want_ct = P.CT != nullptr && mirror;
    const int64_t b64 = batch;
#pragma unroll 1
    for (int hm = 0; hm < 2; ++hm) {
      const int row0 = tm * BM2 + hm * 128;   // first global row of this half
      const int row = row0 + r;
      const bool live = row0 < P.M;            // the second half of a ragged last tile may be empty
      if (have && poly && live) {
        if (warp == 2 && lane == 0) {
          mbar_expect_tx(&s_bar, kStageBytes2);
#pragma unroll
          for (int j = 0; j < 4; ++j) tma_load_3d(s_tile + j * kTileBytes, &map_a, &s_bar, tn * BN2 + j * BK, row0, batch);
        }
        have = mbar_wait(&s_bar, hm & 1, &abort_flag);
      }
      if (have && live) {
#pragma unroll 1
        for (int cb = 0; cb < BN2 / 32; ++cb) {
          uint32_t acc[32];
          if (num_kb > 0) {
            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(hm * 256 + cb * 32), acc);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0u;
          }
          const int box = cb >> 1, q0 = (cb & 1) * 4;
          const int col0 = tn * BN2 + cb * 32;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
          if (poly) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 sv = *(const uint4*)(s_tile + box * kTileBytes + swz(r, q0 + q));
              const uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const int j = q * 8 + e;
                const float sval = bf16_bits_to_float((uint16_t)((w[e >> 1] >> ((e & 1) * 16)) & 0xFFFF));
                v[j] = P.cc * v[j] + P.cb * sval + ((col0 + j == row) ? P.ca : 0.f);
              }
            }
          }
          uint16_t h[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) h[j] = rne_bf16_bits(v[j]);
          if (want_c) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = (uint32_t)h[q * 8 + 0] | ((uint32_t)h[q * 8 + 1] << 16);
              o.y = (uint32_t)h[q * 8 + 2] | ((uint32_t)h[q * 8 + 3] << 16);
              o.z = (uint32_t)h[q * 8 + 4] | ((uint32_t)h[q * 8 + 5] << 16);
              o.w = (uint32_t)h[q * 8 + 6] | ((uint32_t)h[q * 8 + 7] << 16);
              *(uint4*)(c_stage + box * kTileBytes + swz(r, q0 + q)) = o;
            }
          }
          if (want_ct) {  // transposed half tile: rows = the 256 columns (two 128-row groups), columns = r (two 64-wide boxes)
            uint8_t* dst = ct_stage + ((cb >> 2) * 2 + (r >> 6)) * kTileBytes + (r & 7) * 2;
            const int qr = (r & 63) >> 3, ct_row0 = (cb & 3) * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) *(uint16_t*)(dst + swz(ct_row0 + j, qr)) = h[j];
          }
          if (P.F != nullptr && row < P.M) {
            float* f = P.F + b64 * P.strideF;
            if (P.f_transposed) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < P.N) f[(int64_t)(col0 + j) * P.ldf + row] = bf16_bits_to_float(h[j]) * P.f_scale;
            } else {
              float* frow = f + (int64_t)row * P.ldf + col0;
              if (col0 + 32 <= P.N && (P.ldf & 3) == 0 && (((uintptr_t)f) & 15) == 0) {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  *(float4*)(frow + q * 4) =
                      make_float4(bf16_bits_to_float(h[q * 4]) * P.f_scale, bf16_bits_to_float(h[q * 4 + 1]) * P.f_scale,
                                  bf16_bits_to_float(h[q * 4 + 2]) * P.f_scale, bf16_bits_to_float(h[q * 4 + 3]) * P.f_scale);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < P.N) frow[j] = bf16_bits_to_float(h[j]) * P.f_scale;
              }
            }
          }
        }
      }
      if (want_c || want_ct || poly) {
        // staged tile -> global, and nobody may refill the staging (or the S region) before the copies have read it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (have && live && warp == 2 && lane == 0 && (want_c || want_ct)) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (want_c && tn * BN2 + j * BK < P.N) tma_store_3d(&map_c, c_stage + j * kTileBytes, tn * BN2 + j * BK, row0, batch);
            const int ct_r = tn * BN2 + (j >> 1) * 128, ct_c = row0 + (j & 1) * BK;
            if (want_ct && ct_r < P.N && ct_c < P.M) tma_store_3d(&map_ct, ct_stage + j * kTileBytes, ct_c, ct_r, batch);
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
    tc_fence_before();
  }

  if (warp == 0 && lane == 0 && abort_flag) {
    for (int kb = max(0, issued - kStages); kb < issued; ++kb) {
      const int s = kb % kStages, round = kb / kStages;
      for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(&full_bar[s], round & 1)) break;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && P.status != nullptr) atomicExch(P.status, 1);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols2); }
}

// ------------------------------------------------------------------------------------------ prologue
// X = SR_bf16(G / max(||G||_F, eps)) written twice: in the source orientation and transposed (one of the
// two is the K-major operand X, the other X^T).  `sumsq[b]` holds ||G_b||_F^2.
// One block handles a 64 x 64 tile: 256 threads as 16 column-groups (4 columns each) x 16 rows, four row
// passes.  Loads are 16 B (fp32) / 8 B (bf16), both outputs are written with 8-byte stores; the
// transpose goes through shared memory.  Grid: (ceil(C/64), ceil(R/64), batch).
__global__ void __launch_bounds__(256) ns_prepare_kernel(const void* const* __restrict__ srcs, int src_dt, int R, int C,
                                                        const float* __restrict__ sumsq, float eps,
                                                        __nv_bfloat16* __restrict__ same, int64_t ld_same,
                                                        int64_t stride_same, __nv_bfloat16* __restrict__ trans,
                                                        int64_t ld_trans, int64_t stride_trans, uint64_t seed) {
  __shared__ uint16_t tile[64][66];
  const int b = blockIdx.z;
  const void* src = srcs[b];
  const float inv = 1.0f / fmaxf(sqrtf(sumsq[b]), eps);
  const Philox rng(seed);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int c0 = blockIdx.x * 64 + tx * 4;
  const bool vec = (C & 3) == 0 && (((uintptr_t)src) & 15) == 0;
  uint16_t* same_b = (uint16_t*)same + (int64_t)b * stride_same;
  uint16_t* trans_b = (uint16_t*)trans + (int64_t)b * stride_trans;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int rl = ty + 16 * pass, r = blockIdx.y * 64 + rl;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (r < R && c0 < C) {
      const int64_t idx = (int64_t)r * C + c0;
      if (vec) {
        if (src_dt == kF32) {
          const float4 t = *(const float4*)((const float*)src + idx);
          x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
        } else {
          const uint2 t = *(const uint2*)((const uint16_t*)src + idx);
          x[0] = bf16_bits_to_float(t.x & 0xFFFF); x[1] = bf16_bits_to_float(t.x >> 16);
          x[2] = bf16_bits_to_float(t.y & 0xFFFF); x[3] = bf16_bits_to_float(t.y >> 16);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (c0 + k < C)
            x[k] = src_dt == kF32 ? ((const float*)src)[idx + k] : bf16_bits_to_float(((const uint16_t*)src)[idx + k]);
      }
    }
    uint16_t h[4] = {0, 0, 0, 0};
    if (r < R && c0 < C) {
      const int64_t idx = (int64_t)r * C + c0;
      const uint4 rnd = rng((uint32_t)idx, (uint32_t)(idx >> 32), (uint32_t)b, 7u);
      const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c0 + k < C) h[k] = sr_bf16_bits(x[k] * inv, rr[k]);
      uint2 o;
      o.x = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
      o.y = (uint32_t)h[2] | ((uint32_t)h[3] << 16);
      *(uint2*)(same_b + (int64_t)r * ld_same + c0) = o;  // columns past C land in the row padding (ld is a multiple of 8)
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) tile[rl][tx * 4 + k] = h[k];
  }
  __syncthreads();
  // transposed output: this thread owns source rows r0..r0+3 (consecutive in the output row) of four source columns
  const int r0 = blockIdx.y * 64 + tx * 4;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int cl = ty + 16 * pass, c = blockIdx.x * 64 + cl;
    if (c < C && r0 < R) {
      uint2 o;
      o.x = (uint32_t)tile[tx * 4 + 0][cl] | ((uint32_t)tile[tx * 4 + 1][cl] << 16);
      o.y = (uint32_t)tile[tx * 4 + 2][cl] | ((uint32_t)tile[tx * 4 + 3][cl] << 16);
      *(uint2*)(trans_b + (int64_t)c * ld_trans + r0) = o;
    }
  }
}

// ------------------------------------------------------------------------------------------ host side
// bf16 tensor [batch, rows, cols] with leading dimension `ld` elements; box = 64 cols x 128 rows.
static bool encode_map(CUtensorMap* map, const void* base, int rows, int cols, int64_t ld, int64_t batch_stride, int batch);

// A step launches the same ~60 products over the same workspace addresses (the caching allocator hands the buffers
// back), and every launch needs up to four descriptors: they are kept by their defining values instead of being
// encoded again (about 0.6 us each on the host, which is what limits a step once the matrices are split over ranks).
static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int64_t ld, int64_t batch_stride, int batch) {
  struct Key {
    const void* base; int64_t ld, stride; int rows, cols, batch;
    bool operator==(const Key& o) const {
      return base == o.base && ld == o.ld && stride == o.stride && rows == o.rows && cols == o.cols && batch == o.batch;
    }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      size_t h = std::hash<const void*>()(k.base);
      for (int64_t v : {k.ld, k.stride, (int64_t)k.rows, (int64_t)k.cols, (int64_t)k.batch})
        h ^= std::hash<int64_t>()(v) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
      return h;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex guard;
  const Key key{base, ld, batch_stride, rows, cols, batch};
  std::lock_guard<std::mutex> lock(guard);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return true;
  }
  if (!encode_map(map, base, rows, cols, ld, batch_stride, batch)) return false;
  if (cache.size() >= 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

static bool encode_map(CUtensorMap* map, const void* base, int rows, int cols, int64_t ld, int64_t batch_stride, int batch) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[3] = {BK, BM, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int g_tile_override = 0;
int ns_gemm_tile_override() { return g_tile_override; }
void set_ns_gemm_tile_override(int tile) { g_tile_override = tile; }

cudaError_t launch_ns_gemm(const void* A, int64_t lda, int64_t strideA, const void* B, int64_t ldb, int64_t strideB,
                           const GemmParams& P, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(ns_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  GemmParams Q = P;
  Q.same_operand = (A == B && lda == ldb && strideA == strideB && P.M == P.N) ? 1 : 0;
  CUtensorMap ma, mb, mc, mct;
  if (!make_map(&ma, A, P.M, P.K, lda, strideA, P.batch) || !make_map(&mb, B, P.N, P.K, ldb, strideB, P.batch))
    return cudaErrorInvalidValue;
  mc = ma;
  mct = ma;  // placeholders when an output is absent (never dereferenced by the kernel then)
  if (P.C != nullptr && !make_map(&mc, P.C, P.M, P.N, P.ldc, P.strideC, P.batch)) return cudaErrorInvalidValue;
  if (P.CT != nullptr && !make_map(&mct, P.CT, P.N, P.M, P.ldct, P.strideCT, P.batch)) return cudaErrorInvalidValue;
  {
    // large problems: 256x256 tiles (half the operand bytes per flop); they need a long K to hide their epilogue and
    // enough tiles to fill the machine
    const int t2m = (P.M + BM2 - 1) / BM2, t2n = (P.N + BN2 - 1) / BN2;
    const long long big_tiles = (long long)(P.symmetric ? t2m * (t2m + 1) / 2 : t2m * t2n) * P.batch;
    const bool want_big = ns_gemm_tile_override() == 256 ||
                          (ns_gemm_tile_override() == 0 && P.K >= 1024 && P.M >= 1024 && P.N >= 1024 && big_tiles >= 96);
    if (want_big) {
      static bool configured2 = false;
      if (!configured2) {
        cudaError_t e = cudaFuncSetAttribute(ns_gemm256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2);
        if (e != cudaSuccess) return e;
        configured2 = true;
      }
      dim3 grid2((unsigned)(P.symmetric ? t2m * (t2m + 1) / 2 : t2m * t2n), P.batch);
      ns_gemm256_kernel<<<grid2, kGemmThreads, kSmemBytes2, stream>>>(ma, mb, mc, mct, Q);
      return cudaGetLastError();
    }
  }
  const int tiles_m = (P.M + BM - 1) / BM, tiles_n = (P.N + BN - 1) / BN;
  const int tiles = P.symmetric ? tiles_m * (tiles_m + 1) / 2 : tiles_m * tiles_n;
  dim3 grid(tiles, P.batch);
  ns_gemm_kernel<<<grid, kGemmThreads, kSmemBytes, stream>>>(ma, mb, mc, mct, Q);
  return cudaGetLastError();
}

cudaError_t launch_ns_prepare(const void* const* srcs, int src_dt, int R, int C, int batch, const float* sumsq, float eps,
                              void* same, int64_t ld_same, int64_t stride_same, void* trans, int64_t ld_trans,
                              int64_t stride_trans, uint64_t seed, cudaStream_t stream) {
  dim3 grid((C + 63) / 64, (R + 63) / 64, batch), block(256);
  ns_prepare_kernel<<<grid, block, 0, stream>>>(srcs, src_dt, R, C, sumsq, eps, (__nv_bfloat16*)same, ld_same,
                                                stride_same, (__nv_bfloat16*)trans, ld_trans, stride_trans, seed);
  return cudaGetLastError();
}

}  // namespace hb
