// Multi-tensor fused optimizer chain: one launch executes, for every element of every tensor of a
// param group,  [ECC/bf16/fp32 decode] -> [MARS] -> [momentum / second-moment rule] -> [caution] ->
// [weight decay] -> [parameter write | update write] -> [stochastic-rounding / ECC encode].
//
// Replaces the per-tensor compiled regions of the reference (heavyball/utils.py:1842-2334 Adam family,
// 736-776 momentum, 3616-3627 MARS, 2373-2406 parameter update, 3652-3658 caution).  Arithmetic is
// restated from heavyball_b200/utils/first_order.py, which is also the test oracle.
//
// Work decomposition: tensors are cut into CHUNK-element chunks; block b owns chunk b and finds its
// tensor by binary search in a prefix table.  All tensor addresses come from a device-resident table,
// so the launch count is independent of the number of tensors.
#include "common.cuh"
#include "fused_chain.h"

namespace hb {

constexpr int kThreads = 256;
constexpr int kChunk = 8192;  // elements per block

// Random bits are only generated for storage kinds that consume them (bf16 rounding, ECC residuals).
__device__ inline uint4 draw(int dt, const Philox& rng, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) {
  if (dt == kF32 || dt == kF16 || dt == kNone) return make_uint4(0u, 0u, 0u, 0u);
  return rng(c0, c1, c2, c3);
}

__device__ inline float lerp_to(float s, float x, float beta) {  // s*beta' + x*(1-beta') in the oracle's order
  float w = 1.0f - beta;
  return s * (1.0f - w) + x * w;
}

template <bool kCountCaution>
__global__ void __launch_bounds__(kThreads, 4) fused_chain_kernel(const TensorMeta* __restrict__ metas,
                                                              const int* __restrict__ chunk_prefix, ChainParams P) {
  // ---- locate (tensor, chunk)
  int lo = 0, hi = P.n_tensors;
  const int b = blockIdx.x;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (chunk_prefix[mid] <= b) lo = mid; else hi = mid;
  }
  const int t = lo;
  const TensorMeta M = metas[t];
  const int64_t base = (int64_t)(b - chunk_prefix[t]) * kChunk;
  const bool vec_ok = M.vec_ok != 0;
  const Philox rng(P.seed);

  float cscale = 1.0f;
  if (P.use_tensor_scale && M.scale != nullptr) cscale = *M.scale;
  if (P.caution_apply && M.masked != nullptr) {
    float n = (float)M.numel;
    cscale *= n / fmaxf(n - (float)(*M.masked), 1.0f);
  }
  float gclip = 1.0f, ortho_c = 0.f;
  const bool ortho = P.g_clip_mode == kClipOrtho && M.gsq != nullptr;
  if (ortho) {
    const float px = M.gsq[0], pp = M.gsq[1], xx = M.gsq[2];
    ortho_c = px / (pp + P.g_clip_at);
    if (P.g_clip_numel != 0.f) {
      const float proj_sq = fmaxf(xx - 2.f * ortho_c * px + ortho_c * ortho_c * pp, 0.f);
      gclip = sqrtf(fmaxf(xx, 0.f)) / fmaxf(sqrtf(proj_sq), 1e-6f);
    }
  } else if (P.g_clip_mode != kClipNone && M.gsq != nullptr) {
    float sq = *M.gsq;
    if (P.g_clip_mode == kClipRms) sq /= (P.g_clip_numel > 0.f ? P.g_clip_numel : (float)M.numel);
    gclip = P.g_clip_at / fmaxf(sqrtf(sq), fmaxf(P.g_clip_at, 1e-8f));
  }
  float ugraft = 1.0f;
  if (P.u_op == kUopSignGraft && M.scale != nullptr) ugraft = sqrtf(fmaxf(M.scale[0], 0.f)) / fmaxf(sqrtf(M.scale[1]), 1e-6f);
  int masked_local = 0;
  float sumsq_local = 0.f, nonzero_local = 0.f;

#pragma unroll 2
  for (int it = 0; it < kChunk / (kThreads * 4); ++it) {
    const int64_t i = base + ((int64_t)it * kThreads + threadIdx.x) * 4;
    if (i >= M.numel) break;
    const int nv = (int)min((int64_t)4, M.numel - i);
    const uint32_t ctr = (uint32_t)(i >> 2), ctr_hi = (uint32_t)(i >> 34);

    // local state first, then the gradient: with peers the gradient loads are NVLink round trips (about 2 us each),
    // and everything issued before the first use of one of them overlaps with it
    F4 s0 = load4(M.s0, M.s0e, P.dt_s, i, nv, vec_ok);
    F4 s1 = load4(M.s1, M.s1e, P.dt_s, i, nv, vec_ok);
    F4 s2 = load4(M.s2, M.s2e, P.dt_s, i, nv, vec_ok);
    F4 g;
    if (P.n_src > 0 && P.g_mc_delta != 0 && vec_ok && nv == 4 && (P.dt_g == kF32 || P.dt_g == kBF16 || P.dt_g == kF16)) {
      // one load, summed over all ranks inside the NVSwitch
      g = mc_ld_reduce4((const char*)M.g + P.g_mc_delta, P.dt_g, i);
#pragma unroll
      for (int k = 0; k < 4; ++k) g.v[k] *= P.g_scale;
    } else if (P.n_src > 0) {  // reduce the same element over every rank's gradient slab (peer loads over NVLink)
#pragma unroll
      for (int k = 0; k < 4; ++k) g.v[k] = 0.f;
      for (int r0 = 0; r0 < P.n_src; r0 += 4) {  // four sources in flight at a time, summed in rank order
        F4 part[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (r0 + j < P.n_src) part[j] = load4((const char*)M.g + P.g_delta[r0 + j], nullptr, P.dt_g, i, nv, vec_ok);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (r0 + j < P.n_src) {
#pragma unroll
            for (int k = 0; k < 4; ++k) g.v[k] += part[j].v[k];
          }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) g.v[k] *= P.g_scale;
    } else {
      g = load4(M.g, nullptr, P.dt_g, i, nv, vec_ok);
    }
    F4 u = P.u_is_input ? load4(M.u, nullptr, P.dt_u, i, nv, vec_ok) : g;
    if (P.u_is_input && P.u_op == kUopTrustRegion) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x = u.v[k] * (1.0f / 1.5f);
        const float t = tanhf(x);
        const float y = copysignf(log1pf(fabsf(x)), t) * 0.1f + t * 0.9f;
        u.v[k] = fminf(fmaxf(y * 1.5f, -2.0f), 2.0f);
      }
    }
    if (P.u_is_input && (P.u_op == kUopSignGraft || P.u_op == kUopSign)) {
#pragma unroll
      for (int k = 0; k < 4; ++k) u.v[k] = u.v[k] > 0.f ? ugraft : (u.v[k] < 0.f ? -ugraft : 0.f);
    }
    F4 p = (P.out_mode == kOutParam || ortho || P.post_state == kPostDecayIn) ? load4(M.p, M.pe, P.dt_p, i, nv, vec_ok) : F4{};
    F4 out;

    if (ortho) {  // remove the component along the parameter (and keep the norm): caution still sees the raw gradient
#pragma unroll
      for (int k = 0; k < 4; ++k) u.v[k] = (u.v[k] - ortho_c * p.v[k]) * gclip;
    } else if (P.g_clip_mode != kClipNone && !P.u_is_input) {  // the clip acts on the update, caution still sees the raw gradient
#pragma unroll
      for (int k = 0; k < 4; ++k) u.v[k] *= gclip;
    }
    if (P.mars) {  // g <- lerp(g, g_prev, a); g_prev <- raw g
      F4 old = load4(M.mars, M.marse, P.dt_s, i, nv, vec_ok);
      F4 raw = u;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        u.v[k] = u.v[k] * (1.0f - P.mars_a) + old.v[k] * P.mars_a;
        g.v[k] = u.v[k];
      }
      store4(M.mars, M.marse, P.dt_s, i, nv, vec_ok, raw, draw(P.dt_s, rng, ctr, ctr_hi ^ 0x40000000u, (uint32_t)t, 4u));
    }

#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float x = u.v[k], r;
      switch (P.algo) {
        case kAdam: {
          s0.v[k] = lerp_to(s0.v[k], x, P.b1);
          s1.v[k] = lerp_to(s1.v[k], x * x, P.b2);
          r = s0.v[k] / fmaxf(sqrtf(s1.v[k]), P.eps);
        } break;
        case kLaProp: {
          s1.v[k] = lerp_to(s1.v[k], x * x, P.b2);
          s0.v[k] = lerp_to(s0.v[k], x / fmaxf(sqrtf(s1.v[k]), P.eps), P.b1);
          r = s0.v[k];
        } break;
        case kAdopt: {
          s0.v[k] = lerp_to(s0.v[k], x / fmaxf(sqrtf(s1.v[k]), P.eps), P.b1);
          r = s0.v[k];
          s1.v[k] = s1.v[k] * (1.0f - P.b3) + x * x * P.b3;  // b3 = 1 - debiased beta2 of the next step
        } break;
        case kAdemamix: {
          s0.v[k] = lerp_to(s0.v[k], x, P.b1);
          s2.v[k] = lerp_to(s2.v[k], x, P.b3);
          s1.v[k] = lerp_to(s1.v[k], x * x, P.b2);
          r = (s0.v[k] + s2.v[k] * P.alpha) / fmaxf(sqrtf(s1.v[k]), P.eps);
        } break;
        case kRmsprop: {
          s1.v[k] = lerp_to(s1.v[k], x * x, P.b2);
          r = x / fmaxf(sqrtf(s1.v[k]), P.eps);
        } break;
        case kUnscaledAdam: {
          s1.v[k] = lerp_to(s1.v[k], x * x, P.b2);
          float d = fmaxf(sqrtf(s1.v[k]), P.eps);
          s0.v[k] = lerp_to(s0.v[k], x / d, P.b1);
          r = s0.v[k] * d;
        } break;
        case kExpAvg: {
          s0.v[k] = lerp_to(s0.v[k], x, P.b1);
          r = s0.v[k];
        } break;
        case kNesterovEma: {
          s0.v[k] = lerp_to(s0.v[k], x, P.b1);
          r = x + s0.v[k];
        } break;
        case kHeavyball: {
          s0.v[k] = s0.v[k] * P.b1 + x;
          r = s0.v[k];
        } break;
        case kNesterovMom: {
          s0.v[k] = s0.v[k] * P.b1 + x;
          r = x + s0.v[k] * P.b1;
        } break;
        case kNadam: {  // b3 = (1 - mu) / (1 - mu_product), alpha = mu_next / (1 - mu_product mu_next), set on the host
          s0.v[k] = lerp_to(s0.v[k], x, P.b1);
          s1.v[k] = lerp_to(s1.v[k], x * x, P.b2);
          float d = fmaxf(sqrtf(s1.v[k]), P.eps);
          r = x / d * P.b3 + s0.v[k] / d * P.alpha;
        } break;
        default:
          r = x;
      }
      out.v[k] = r;
    }

    if (P.post_state == kPostMsam) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float m = lerp_to(s0.v[k], out.v[k], P.b3);
        float d = P.wd;
        if (P.cautious_wd && ((__float_as_uint(s2.v[k]) ^ __float_as_uint(m)) >> 31)) d = 0.f;
        s0.v[k] = m;
        s2.v[k] = s2.v[k] * (1.0f - d * P.lr) + m * -P.lr;
        out.v[k] = m;
      }
    } else if (P.post_state == kPostDecayIn) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float d = P.wd;
        if (P.cautious_wd && ((__float_as_uint(p.v[k]) ^ __float_as_uint(out.v[k])) >> 31)) d = 0.f;
        out.v[k] += p.v[k] * d;
      }
    }

    // plain bf16 rounding consumes 16 random bits per element: the first two state tensors share one draw
    // (low / high halves); ECC residuals need 32 bits and keep a draw each
    const uint4 r0 = (P.n_state >= 1) ? draw(P.dt_s, rng, ctr, ctr_hi, (uint32_t)t, 0u) : make_uint4(0u, 0u, 0u, 0u);
    if (P.n_state >= 1) store4(M.s0, M.s0e, P.dt_s, i, nv, vec_ok, s0, r0);
    if (P.n_state >= 2)
      store4(M.s1, M.s1e, P.dt_s, i, nv, vec_ok, s1,
             P.dt_s == kBF16 ? make_uint4(r0.x >> 16, r0.y >> 16, r0.z >> 16, r0.w >> 16)
                             : draw(P.dt_s, rng, ctr, ctr_hi, (uint32_t)t, 1u));
    if (P.n_state >= 3) store4(M.s2, M.s2e, P.dt_s, i, nv, vec_ok, s2, draw(P.dt_s, rng, ctr, ctr_hi, (uint32_t)t, 2u));
    if (P.out_mode == kOutScheduleFree) {  // z lives in slot s2 (loaded above), p and z are both written
      F4 pp = load4(M.p, M.pe, P.dt_p, i, nv, vec_ok);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float uu = out.v[k];
        if (P.wd != 0.f) {
          float d = P.wd;
          if (P.cautious_wd && ((__float_as_uint(pp.v[k]) ^ __float_as_uint(uu)) >> 31)) d = 0.f;
          uu += pp.v[k] * d;
        }
        pp.v[k] = pp.v[k] + (s2.v[k] - pp.v[k]) * P.b3 + uu * (P.lr * (P.alpha * (1.0f - P.b3)) - P.lr);
        s2.v[k] = s2.v[k] + uu * -P.lr;
      }
      store4(M.s2, M.s2e, P.dt_s, i, nv, vec_ok, s2, draw(P.dt_s, rng, ctr, ctr_hi, (uint32_t)t, 2u));
      store4(M.p, M.pe, P.dt_p, i, nv, vec_ok, pp, draw(P.dt_p, rng, ctr, ctr_hi, (uint32_t)t, 3u));
      continue;
    }

    if (kCountCaution) {  // phase one of caution: mask, count, park the masked update
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        bool disagree = (__float_as_uint(g.v[k]) ^ __float_as_uint(out.v[k])) >> 31;
        if (k < nv && disagree) { out.v[k] = 0.f; ++masked_local; }
      }
      store4(M.u, nullptr, P.dt_u, i, nv, vec_ok, out, draw(P.dt_u, rng, ctr, ctr_hi, (uint32_t)t, 5u));
      continue;
    }
    if (P.out_mode == kOutUpdate) {
      store4(M.u, nullptr, P.dt_u, i, nv, vec_ok, out, draw(P.dt_u, rng, ctr, ctr_hi, (uint32_t)t, 5u));
      if (P.accum_sumsq) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < nv) {
            sumsq_local += out.v[k] * out.v[k];
            nonzero_local += out.v[k] != 0.f ? 1.f : 0.f;
          }
      }
      continue;
    }
    // parameter epilogue: p <- p (1 - d lr) - lr u
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float uu = out.v[k] * cscale;
      float d = P.wd;
      if (P.cautious_wd && ((__float_as_uint(p.v[k]) ^ __float_as_uint(uu)) >> 31)) d = 0.f;
      p.v[k] = p.v[k] * (1.0f - d * P.lr) + uu * -P.lr;
    }
    const uint4 prnd = draw(P.dt_p, rng, ctr, ctr_hi, (uint32_t)t, 3u);
    if (P.n_dst > 0 && P.p_mc_delta != 0 && vec_ok && nv == 4) {  // one store, replicated to every rank by the NVSwitch
      mc_store4((char*)M.p + P.p_mc_delta, M.pe, P.dt_p, i, p, prnd);
    } else if (P.n_dst > 0) {  // single writer per element: every replica receives bit-identical parameters
      for (int r = 0; r < P.n_dst; ++r)  // the residual of an error-corrected parameter stays with this rank (its only reader)
        store4((char*)M.p + P.p_delta[r], P.p_delta[r] == 0 ? M.pe : nullptr, P.dt_p, i, nv, vec_ok, p, prnd);
    } else {
      store4(M.p, M.pe, P.dt_p, i, nv, vec_ok, p, prnd);
    }
  }

  if (P.accum_sumsq && M.scale != nullptr) {  // per-tensor squared norm of the update just written (feeds Newton–Schulz)
    __shared__ float warp_sq[kThreads / 32];
    float v = sumsq_local;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xFFFFFFFFu, v, o);
    if ((threadIdx.x & 31) == 0) warp_sq[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < kThreads / 32; ++w) tot += warp_sq[w];
      atomicAdd(M.scale, tot);
    }
    if (P.accum_sumsq == 2) {  // block counts are exact integers (<= 8192); their sum stays exact up to 2^24 elements
      __syncthreads();
      float c = nonzero_local;
      for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xFFFFFFFFu, c, o);
      if ((threadIdx.x & 31) == 0) warp_sq[threadIdx.x >> 5] = c;
      __syncthreads();
      if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) tot += warp_sq[w];
        atomicAdd(M.scale + 1, tot);
      }
    }
  }
  if (kCountCaution) {
    __shared__ int warp_sums[kThreads / 32];
    int v = masked_local;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xFFFFFFFFu, v, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < kThreads / 32; ++w) tot += warp_sums[w];
      if (tot) atomicAdd(M.masked, tot);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Segmented sum of squares: out[t] += sum(x_t^2).  One block per chunk, one atomic per block.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) sumsq_kernel(const TensorMeta* __restrict__ metas,
                                                        const int* __restrict__ chunk_prefix, int n_tensors, int dt,
                                                        float* __restrict__ out) {
  int lo = 0, hi = n_tensors;
  const int b = blockIdx.x;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (chunk_prefix[mid] <= b) lo = mid; else hi = mid;
  }
  const TensorMeta M = metas[lo];
  const int64_t base = (int64_t)(b - chunk_prefix[lo]) * kChunk;
  float acc = 0.f;
#pragma unroll 2
  for (int it = 0; it < kChunk / (kThreads * 4); ++it) {
    const int64_t i = base + ((int64_t)it * kThreads + threadIdx.x) * 4;
    if (i >= M.numel) break;
    const int nv = (int)min((int64_t)4, M.numel - i);
    F4 x = load4(M.u, nullptr, dt, i, nv, M.vec_ok != 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) acc += x.v[k] * x.v[k];
  }
  __shared__ float warp_sums[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) tot += warp_sums[w];
    atomicAdd(out + lo, tot);
  }
}

// ---------------------------------------------------------------------------------------------
// Segmented dot product and absolute maximum over the same chunk table: out[t] = sum(x_t * y_t) or max |x_t|.
// x comes from TensorMeta::u, y from TensorMeta::g; `out` starts at zero.  One block per chunk; the block results
// meet in out[t] through one atomic each (float add; for the maximum an unsigned integer max on the bit pattern,
// which orders non-negative floats like their values and puts NaN above everything, so a NaN input gives NaN).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float nan_max(float acc, float a) { return (a > acc || a != a) ? a : acc; }

template <int OP>
__global__ void __launch_bounds__(kThreads) segmented_reduce_kernel(const TensorMeta* __restrict__ metas,
                                                                   const int* __restrict__ chunk_prefix, int n_tensors,
                                                                   int dt, float* __restrict__ out) {
  int lo = 0, hi = n_tensors;
  const int b = blockIdx.x;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (chunk_prefix[mid] <= b) lo = mid; else hi = mid;
  }
  const TensorMeta M = metas[lo];
  const int64_t base = (int64_t)(b - chunk_prefix[lo]) * kChunk;
  float acc = 0.f;
#pragma unroll 2
  for (int it = 0; it < kChunk / (kThreads * 4); ++it) {
    const int64_t i = base + ((int64_t)it * kThreads + threadIdx.x) * 4;
    if (i >= M.numel) break;
    const int nv = (int)min((int64_t)4, M.numel - i);
    const F4 x = load4(M.u, nullptr, dt, i, nv, M.vec_ok != 0);
    if (OP == kReduceDot) {
      const F4 y = load4(M.g, nullptr, dt, i, nv, M.vec_ok != 0);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc += x.v[k] * y.v[k];
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) acc = nan_max(acc, fabsf(x.v[k]));  // lanes past the end read as zero
    }
  }
  __shared__ float warp_res[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_down_sync(0xFFFFFFFFu, acc, o);
    acc = OP == kReduceDot ? acc + other : nan_max(acc, other);
  }
  if ((threadIdx.x & 31) == 0) warp_res[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = warp_res[0];
    for (int w = 1; w < kThreads / 32; ++w) tot = OP == kReduceDot ? tot + warp_res[w] : nan_max(tot, warp_res[w]);
    if (OP == kReduceDot)
      atomicAdd(out + lo, tot);
    else
      atomicMax(reinterpret_cast<unsigned int*>(out + lo), __float_as_uint(tot));
  }
}

int chain_chunk_elems() { return kChunk; }

cudaError_t launch_fused_chain(const TensorMeta* metas, const int* chunk_prefix, int total_chunks, const ChainParams& P,
                               bool count_caution, cudaStream_t stream) {
  if (total_chunks <= 0) return cudaSuccess;
  if (count_caution)
    fused_chain_kernel<true><<<total_chunks, kThreads, 0, stream>>>(metas, chunk_prefix, P);
  else
    fused_chain_kernel<false><<<total_chunks, kThreads, 0, stream>>>(metas, chunk_prefix, P);
  return cudaGetLastError();
}

cudaError_t launch_sumsq(const TensorMeta* metas, const int* chunk_prefix, int total_chunks, int n_tensors, int dt,
                         float* out, cudaStream_t stream) {
  if (total_chunks <= 0) return cudaSuccess;
  sumsq_kernel<<<total_chunks, kThreads, 0, stream>>>(metas, chunk_prefix, n_tensors, dt, out);
  return cudaGetLastError();
}

cudaError_t launch_segmented_reduce(const TensorMeta* metas, const int* chunk_prefix, int total_chunks, int n_tensors,
                                    int dt, int op, float* out, cudaStream_t stream) {
  if (total_chunks <= 0) return cudaSuccess;
  if (op == kReduceDot)
    segmented_reduce_kernel<kReduceDot><<<total_chunks, kThreads, 0, stream>>>(metas, chunk_prefix, n_tensors, dt, out);
  else if (op == kReduceAbsMax)
    segmented_reduce_kernel<kReduceAbsMax><<<total_chunks, kThreads, 0, stream>>>(metas, chunk_prefix, n_tensors, dt, out);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace hb
