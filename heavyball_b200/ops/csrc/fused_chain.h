// Host-visible declarations for the multi-tensor element-wise kernels (fused_chain.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

// One entry per tensor of the group.  Unused pointers are null.  `u` is the update buffer: an input
// when ChainParams::u_is_input, an output for kOutUpdate / caution phase one.
struct TensorMeta {
  void* p;      // parameter (primary)
  void* pe;     // parameter ECC residual
  void* g;      // gradient
  void* u;      // update buffer
  void* s0;     // first state slot (exp_avg / momentum / exp_avg_fast)
  void* s0e;
  void* s1;     // second state slot (exp_avg_sq)
  void* s1e;
  void* s2;     // third state slot (exp_avg_slow)
  void* s2e;
  void* mars;   // previous gradient for MARS
  void* marse;
  float* scale; // optional per-tensor multiplier applied to the update; accum_sumsq target ([sum u^2, count u != 0] for
                // accum_sumsq == 2 and kUopSignGraft)
  int* masked;  // caution: number of masked elements (written by phase one, read by phase two)
  const float* gsq;  // gradient clipping: sum of squares the clip factor is derived from (this tensor's, or the group's);
                     // kClipOrtho: this tensor's three dot products [p.x, p.p, x.x]
  int64_t numel;
  int32_t vec_ok;  // all buffers of this tensor are aligned for 4-wide access
  int32_t pad;
};

constexpr int kMaxPeers = 16;

enum Algo : int {
  kIdentity = 0, kAdam, kLaProp, kAdopt, kAdemamix, kRmsprop, kUnscaledAdam, kExpAvg, kNesterovEma, kHeavyball,
  kNesterovMom, kNadam
};
// kOutScheduleFree: the update moves the averaged iterate: with z in slot s2,
//   p <- lerp(p, z, b3) + u (lr (alpha (1 - b3)) - lr),  z <- z - lr u     (b3 = c_{k+1}, alpha = beta1)
enum OutMode : int { kOutParam = 0, kOutUpdate = 1, kOutScheduleFree = 2 };
// incoming-gradient clip: g <- g * clip_at / max(norm, clip_at, 1e-8), norm = sqrt(gsq) (kClipL2) or sqrt(gsq / n) (kClipRms)
// kClipOrtho (OrthoGrad): x <- a (x - c p) with c = p.x / (p.p + g_clip_at) and, when g_clip_numel != 0, a = |x| / |x - c p|
// (the projected vector keeps the norm of the original; |x - c p|^2 = x.x - 2 c p.x + c^2 p.p), else a = 1.  It acts on
// whatever the launch takes in: the gradient, or the update when u_is_input.
enum ClipMode : int { kClipNone = 0, kClipL2 = 1, kClipRms = 2, kClipOrtho = 3 };
// kUopTrustRegion: 0.9 tanh(x / 1.5) + 0.1 sign(x) log1p(|x| / 1.5), times 1.5, limited to +-2 (PSGD's default update clip)
// kUopSignGraft: sign(x) * sqrt(sum x^2) / max(sqrt(count x != 0), 1e-6) with both sums in TensorMeta::scale (written by an
// earlier launch with accum_sumsq == 2): the sign vector rescaled to the norm of x.  kUopSign: sign(x).
enum UpdateOp : int { kUopNone = 0, kUopTrustRegion = 1, kUopSignGraft = 2, kUopSign = 3 };

// What happens to the rule's output before anything is stored:
//   kPostMsam (Momentum-SAM): m = s0 <- lerp(s0, out, 1 - b3);  z = s2 <- z (1 - d lr) - lr m;  out <- m
//   kPostDecayIn:             out <- out + p d                  (weight decay folded into the update itself)
// with d = wd, or 0 where cautious_wd is set and the signs of the decayed value and the update differ.
enum PostState : int { kPostNone = 0, kPostMsam = 1, kPostDecayIn = 2 };

struct ChainParams {
  int n_tensors;
  int algo;
  int out_mode;
  int n_state;       // how many of s0..s2 are live
  int dt_p, dt_g, dt_u, dt_s;
  int u_is_input;    // read the incoming update from `u` instead of from `g`
  int mars;
  int cautious_wd;
  int caution_apply; // phase two: rescale by numel / (numel - masked)
  int use_tensor_scale;
  int accum_sumsq;   // kOutUpdate: add sum(update^2) of every tensor into its `scale` slot; 2: also the number of non-zero
                     // elements into the slot after it
  int post_state;    // see PostState
  int u_op;          // transformation of an incoming update (u_is_input) before anything else: see UpdateOp
  int g_clip_mode;   // see ClipMode; needs TensorMeta::gsq
  float g_clip_at;
  float g_clip_numel;  // kClipRms: element count behind gsq (0 = this tensor's)
  float lr, wd, eps;
  float b1, b2, b3, alpha;  // already debiased / scheduled on the host
  float mars_a;
  uint64_t seed;
  // Peer-memory data parallelism (n_src / n_dst = 0 turns it off).  Gradient = g_scale * sum over sources
  // of the same element in every source's gradient slab; parameters (and their ECC residuals) are
  // written to every destination.  Deltas are byte offsets from this rank's address to the peer's.
  int n_src, n_dst;
  float g_scale;
  int64_t g_delta[kMaxPeers];
  int64_t p_delta[kMaxPeers];
  // NVSwitch multicast (0 = off): byte offsets from this rank's address to the multicast address of the same element.
  // With g_mc_delta the gradient of all ranks is summed inside the switch by one multimem.ld_reduce per 16 bytes instead
  // of one peer load per rank; with p_mc_delta one multimem.st replaces the per-rank parameter stores.  Both need
  // 16-byte aligned, full 4-element accesses; ragged edges take the per-rank path.
  int64_t g_mc_delta;
  int64_t p_mc_delta;
};

int chain_chunk_elems();
cudaError_t launch_fused_chain(const TensorMeta* metas, const int* chunk_prefix, int total_chunks, const ChainParams& P,
                               bool count_caution, cudaStream_t stream);
cudaError_t launch_sumsq(const TensorMeta* metas, const int* chunk_prefix, int total_chunks, int n_tensors, int dt,
                         float* out, cudaStream_t stream);


// out[t] = sum(u_t * g_t) (kReduceDot) or max |u_t| (kReduceAbsMax); `out` must be zero on entry.
enum ReduceOp : int { kReduceDot = 0, kReduceAbsMax = 1 };
cudaError_t launch_segmented_reduce(const TensorMeta* metas, const int* chunk_prefix, int total_chunks, int n_tensors,
                                    int dt, int op, float* out, cudaStream_t stream);

}  // namespace hb
