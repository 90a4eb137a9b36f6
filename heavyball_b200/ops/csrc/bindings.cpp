// Python bindings: translate torch tensors into the raw tables the kernels consume.
// Kernels live in the .cu files and know nothing about torch; this file owns all torch-facing glue.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <vector>

#include "colsum.h"
#include "cross_entropy.h"
#include "fused_chain.h"
#include "gelu.h"
#include "layer_norm.h"
#include "ns_gemm.h"
#include "peer_sync.h"
#include "skinny.h"
#include "tf32_gemm.h"

namespace py = pybind11;
using OptT = std::optional<at::Tensor>;
using TList = std::vector<OptT>;

namespace {

void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

void* ptr_or_null(const TList& l, size_t i) {
  if (l.empty() || !l[i].has_value() || !l[i]->defined()) return nullptr;
  return l[i]->data_ptr();
}

bool aligned16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct Table {
  at::Tensor device_blob;  // metas followed by the chunk prefix
  const hb::TensorMeta* metas;
  const int* prefix;
  int total_chunks;
  int n;
};

// Builds the per-tensor table and uploads it with one async copy on the current stream.
Table upload(std::vector<hb::TensorMeta>& metas, const at::Device& dev) {
  const int n = (int)metas.size();
  const int chunk = hb::chain_chunk_elems();
  std::vector<int> prefix(n + 1, 0);
  for (int i = 0; i < n; ++i) prefix[i + 1] = prefix[i] + (int)((metas[i].numel + chunk - 1) / chunk);
  const size_t meta_bytes = sizeof(hb::TensorMeta) * n, prefix_bytes = sizeof(int) * (n + 1);
  std::vector<uint8_t> host(meta_bytes + prefix_bytes);
  memcpy(host.data(), metas.data(), meta_bytes);
  memcpy(host.data() + meta_bytes, prefix.data(), prefix_bytes);
  Table t;
  t.device_blob = at::empty({(int64_t)host.size()}, at::TensorOptions().dtype(at::kByte).device(dev));
  auto stream = at::cuda::getCurrentCUDAStream();
  check(cudaMemcpyAsync(t.device_blob.data_ptr(), host.data(), host.size(), cudaMemcpyHostToDevice, stream), "table upload");
  t.metas = reinterpret_cast<const hb::TensorMeta*>(t.device_blob.data_ptr());
  t.prefix = reinterpret_cast<const int*>((uint8_t*)t.device_blob.data_ptr() + meta_bytes);
  t.total_chunks = prefix[n];
  t.n = n;
  return t;
}

}  // namespace

// One fused pass over a param group.  Every list is either empty or has one entry per tensor.
// `cfg`: algo, out_mode, n_state, dt_p, dt_g, dt_u, dt_s, u_is_input, mars, cautious_wd, caution_apply,
// use_tensor_scale, count_caution (ints); lr, wd, eps, b1, b2, b3, alpha, mars_a (floats); seed.
void fused_chain(const TList& p, const TList& pe, const TList& g, const TList& u, const TList& s0, const TList& s0e,
                 const TList& s1, const TList& s1e, const TList& s2, const TList& s2e, const TList& mars,
                 const TList& marse, const OptT& scale, const OptT& masked, const OptT& gsq, const py::dict& cfg) {
  const size_t n = !g.empty() ? g.size() : (!u.empty() ? u.size() : p.size());
  if (n == 0) return;
  const at::Tensor& ref = !g.empty() ? *g[0] : (!u.empty() ? *u[0] : *p[0]);
  c10::cuda::CUDAGuard guard(ref.device());
  const int scale_stride = cfg.contains("scale_stride") ? std::max(1, cfg["scale_stride"].cast<int>()) : 1;
  const int gsq_stride = cfg.contains("gsq_stride") ? std::max(1, cfg["gsq_stride"].cast<int>()) : 1;
  {  // the kernel trusts the table: every buffer must be a contiguous CUDA tensor of the element count and storage
     // kind its slot is declared with, on the device of the launch
    // storage kinds as in common.cuh: 0 fp32, 1 bf16, 2 fp16, 3 bf16+8, 4 bf16+16, 5 fp16+8, 6 fp16+16, 7 none
    auto dt_of = [&](const char* k) { return cfg.contains(k) ? cfg[k].cast<int>() : 0; };
    auto primary_bytes = [](int dt) { return dt == 0 ? 4 : (dt == 7 ? 0 : 2); };
    auto residual_bytes = [](int dt) { return (dt == 3 || dt == 5) ? 1 : ((dt == 4 || dt == 6) ? 2 : 0); };
    struct Slot { const TList* list; const char* name; int dt; bool residual; };
    const int dp = dt_of("dt_p"), dg = dt_of("dt_g"), du = dt_of("dt_u"), ds = dt_of("dt_s");
    const Slot slots[] = {{&p, "p", dp, false}, {&pe, "pe", dp, true}, {&g, "g", dg, false}, {&u, "u", du, false},
                          {&s0, "s0", ds, false}, {&s0e, "s0e", ds, true}, {&s1, "s1", ds, false}, {&s1e, "s1e", ds, true},
                          {&s2, "s2", ds, false}, {&s2e, "s2e", ds, true}, {&mars, "mars", ds, false}, {&marse, "marse", ds, true}};
    for (const Slot& sl : slots) {
      if (sl.list->empty()) continue;
      TORCH_CHECK(sl.list->size() == n, "fused_chain: list '", sl.name, "' has ", sl.list->size(), " entries, expected ", n);
      const int want = sl.residual ? residual_bytes(sl.dt) : primary_bytes(sl.dt);
      for (size_t i = 0; i < n; ++i) {
        const OptT& t = (*sl.list)[i];
        TORCH_CHECK(t.has_value() && t->defined(), "fused_chain: '", sl.name, "'[", i, "] is missing");
        TORCH_CHECK(t->is_cuda() && t->device() == ref.device() && t->is_contiguous(), "fused_chain: '", sl.name, "'[", i,
                    "] must be a contiguous CUDA tensor on the launch device");
        TORCH_CHECK(want != 0 && (int)t->element_size() == want, "fused_chain: '", sl.name, "'[", i, "] has ", t->element_size(),
                    "-byte elements, its storage kind needs ", want);
      }
    }
    for (const at::Tensor* aux : {scale.has_value() ? &*scale : nullptr, masked.has_value() ? &*masked : nullptr}) {
      if (aux == nullptr) continue;
      const size_t per = aux == (scale.has_value() ? &*scale : nullptr) ? (size_t)scale_stride : 1;
      TORCH_CHECK(aux->is_cuda() && aux->is_contiguous() && (size_t)aux->numel() >= n * per && aux->element_size() == 4,
                  "fused_chain: per-tensor scalars need ", per, " 4-byte entries per tensor");
    }
    if (gsq.has_value())
      TORCH_CHECK(gsq->is_cuda() && gsq->is_contiguous() && gsq->scalar_type() == at::kFloat &&
                      (gsq->numel() == 1 || (size_t)gsq->numel() >= n * (size_t)gsq_stride),
                  "fused_chain: gsq needs one fp32 entry, or gsq_stride per tensor");
    const int clip_mode = cfg.contains("g_clip_mode") ? cfg["g_clip_mode"].cast<int>() : 0;
    TORCH_CHECK(clip_mode != hb::kClipOrtho || (gsq.has_value() && gsq_stride == 3 && !p.empty()),
                "fused_chain: the OrthoGrad projection needs the parameters and three dot products per tensor");
    const int uop = cfg.contains("u_op") ? cfg["u_op"].cast<int>() : 0;
    const int acc = cfg.contains("accum_sumsq") ? cfg["accum_sumsq"].cast<int>() : 0;
    TORCH_CHECK((uop != hb::kUopSignGraft && acc != 2) || (scale.has_value() && scale_stride == 2),
                "fused_chain: sign grafting keeps two sums per tensor in `scale`");
  }
  std::vector<hb::TensorMeta> metas(n);
  for (size_t i = 0; i < n; ++i) {
    hb::TensorMeta& m = metas[i];
    m.p = ptr_or_null(p, i); m.pe = ptr_or_null(pe, i); m.g = ptr_or_null(g, i); m.u = ptr_or_null(u, i);
    m.s0 = ptr_or_null(s0, i); m.s0e = ptr_or_null(s0e, i); m.s1 = ptr_or_null(s1, i); m.s1e = ptr_or_null(s1e, i);
    m.s2 = ptr_or_null(s2, i); m.s2e = ptr_or_null(s2e, i); m.mars = ptr_or_null(mars, i); m.marse = ptr_or_null(marse, i);
    m.scale = scale.has_value() ? scale->data_ptr<float>() + (int64_t)i * scale_stride : nullptr;
    m.masked = masked.has_value() ? masked->data_ptr<int>() + i : nullptr;
    m.gsq = gsq.has_value() ? gsq->data_ptr<float>() + (gsq->numel() == 1 ? 0 : (int64_t)i * gsq_stride) : nullptr;
    const at::Tensor& any = !g.empty() && g[i].has_value() ? *g[i] : (!u.empty() && u[i].has_value() ? *u[i] : *p[i]);
    m.numel = any.numel();
    for (const TList* l : {&p, &pe, &g, &u, &s0, &s0e, &s1, &s1e, &s2, &s2e, &mars, &marse})
      TORCH_CHECK(l->empty() || (*l)[i]->numel() == m.numel, "fused_chain: buffers of tensor ", i, " differ in element count");
    bool ok = true;
    for (void* q : {m.p, m.pe, m.g, m.u, m.s0, m.s0e, m.s1, m.s1e, m.s2, m.s2e, m.mars, m.marse}) ok = ok && aligned16(q);
    m.vec_ok = ok ? 1 : 0;
    m.pad = 0;
  }
  Table t = upload(metas, ref.device());
  hb::ChainParams P{};
  auto geti = [&](const char* k) { return cfg.contains(k) ? cfg[k].cast<int>() : 0; };
  auto getf = [&](const char* k) { return cfg.contains(k) ? cfg[k].cast<float>() : 0.f; };
  P.n_tensors = t.n;
  P.algo = geti("algo"); P.out_mode = geti("out_mode"); P.n_state = geti("n_state");
  P.dt_p = geti("dt_p"); P.dt_g = geti("dt_g"); P.dt_u = geti("dt_u"); P.dt_s = geti("dt_s");
  P.u_is_input = geti("u_is_input"); P.mars = geti("mars"); P.cautious_wd = geti("cautious_wd");
  P.caution_apply = geti("caution_apply"); P.use_tensor_scale = geti("use_tensor_scale");
  P.accum_sumsq = geti("accum_sumsq"); P.u_op = geti("u_op"); P.post_state = geti("post_state");
  TORCH_CHECK(P.post_state != hb::kPostMsam || (!s0.empty() && !s2.empty() && P.n_state == 3),
              "fused_chain: Momentum-SAM keeps its momentum in s0 and the unperturbed weights in s2");
  TORCH_CHECK(P.post_state != hb::kPostDecayIn || !p.empty(), "fused_chain: decay folded into the update reads the parameters");
  P.g_clip_mode = geti("g_clip_mode"); P.g_clip_at = getf("g_clip_at"); P.g_clip_numel = getf("g_clip_numel");
  P.lr = getf("lr"); P.wd = getf("wd"); P.eps = getf("eps");
  P.b1 = getf("b1"); P.b2 = getf("b2"); P.b3 = getf("b3"); P.alpha = getf("alpha"); P.mars_a = getf("mars_a");
  P.seed = cfg.contains("seed") ? cfg["seed"].cast<uint64_t>() : 0;
  if (cfg.contains("g_delta")) {
    auto d = cfg["g_delta"].cast<std::vector<int64_t>>();
    TORCH_CHECK((int)d.size() <= hb::kMaxPeers, "too many gradient sources");
    P.n_src = (int)d.size();
    for (size_t i = 0; i < d.size(); ++i) P.g_delta[i] = d[i];
    P.g_scale = getf("g_scale");
  }
  if (cfg.contains("p_delta")) {
    auto d = cfg["p_delta"].cast<std::vector<int64_t>>();
    TORCH_CHECK((int)d.size() <= hb::kMaxPeers, "too many parameter destinations");
    P.n_dst = (int)d.size();
    for (size_t i = 0; i < d.size(); ++i) P.p_delta[i] = d[i];
  }
  P.g_mc_delta = cfg.contains("g_mc_delta") ? cfg["g_mc_delta"].cast<int64_t>() : 0;
  P.p_mc_delta = cfg.contains("p_mc_delta") ? cfg["p_mc_delta"].cast<int64_t>() : 0;
  check(hb::launch_fused_chain(t.metas, t.prefix, t.total_chunks, P, geti("count_caution") != 0,
                               at::cuda::getCurrentCUDAStream()), "fused_chain launch");
}

// out[i] = sum(x_i^2) in fp32.
at::Tensor sumsq(const std::vector<at::Tensor>& xs, int dt) {
  TORCH_CHECK(!xs.empty(), "sumsq: empty list");
  c10::cuda::CUDAGuard guard(xs[0].device());
  std::vector<hb::TensorMeta> metas(xs.size());
  for (size_t i = 0; i < xs.size(); ++i) {
    memset(&metas[i], 0, sizeof(hb::TensorMeta));
    metas[i].u = xs[i].data_ptr();
    metas[i].numel = xs[i].numel();
    metas[i].vec_ok = aligned16(metas[i].u) ? 1 : 0;
  }
  Table t = upload(metas, xs[0].device());
  at::Tensor out = at::zeros({(int64_t)xs.size()}, xs[0].options().dtype(at::kFloat));
  check(hb::launch_sumsq(t.metas, t.prefix, t.total_chunks, t.n, dt, out.data_ptr<float>(),
                         at::cuda::getCurrentCUDAStream()), "sumsq launch");
  return out;
}

// out[i] = sum(x_i * y_i) (op 0) or max |x_i| (op 1, `ys` empty) in fp32; all tensors contiguous, one storage kind.
at::Tensor segmented_reduce(const std::vector<at::Tensor>& xs, const std::vector<at::Tensor>& ys, int dt, int op) {
  TORCH_CHECK(!xs.empty(), "segmented_reduce: empty list");
  TORCH_CHECK(op == hb::kReduceAbsMax ? ys.empty() : ys.size() == xs.size(), "segmented_reduce: one y per x for the dot product");
  c10::cuda::CUDAGuard guard(xs[0].device());
  std::vector<hb::TensorMeta> metas(xs.size());
  for (size_t i = 0; i < xs.size(); ++i) {
    TORCH_CHECK(xs[i].is_cuda() && xs[i].is_contiguous() && xs[i].scalar_type() == xs[0].scalar_type(), "segmented_reduce: contiguous CUDA tensors of one dtype");
    memset(&metas[i], 0, sizeof(hb::TensorMeta));
    metas[i].u = xs[i].data_ptr();
    metas[i].numel = xs[i].numel();
    bool ok = aligned16(metas[i].u);
    if (!ys.empty()) {
      TORCH_CHECK(ys[i].is_cuda() && ys[i].is_contiguous() && ys[i].scalar_type() == xs[0].scalar_type() &&
                      ys[i].numel() == xs[i].numel(), "segmented_reduce: y like x");
      metas[i].g = ys[i].data_ptr();
      ok = ok && aligned16(metas[i].g);
    }
    metas[i].vec_ok = ok ? 1 : 0;
  }
  Table t = upload(metas, xs[0].device());
  at::Tensor out = at::zeros({(int64_t)xs.size()}, xs[0].options().dtype(at::kFloat));
  check(hb::launch_segmented_reduce(t.metas, t.prefix, t.total_chunks, t.n, dt, op, out.data_ptr<float>(),
                                    at::cuda::getCurrentCUDAStream()), "segmented_reduce launch");
  return out;
}

// Normalise + stochastically round a batch of same-shape matrices into the two bf16 work layouts.
void ns_prepare(const std::vector<at::Tensor>& srcs, int src_dt, int64_t R, int64_t C, const at::Tensor& sumsq_t, double eps,
                at::Tensor same, int64_t ld_same, at::Tensor trans, int64_t ld_trans, uint64_t seed) {
  c10::cuda::CUDAGuard guard(same.device());
  std::vector<const void*> ptrs(srcs.size());
  for (size_t i = 0; i < srcs.size(); ++i) ptrs[i] = srcs[i].data_ptr();
  at::Tensor dev = at::empty({(int64_t)(ptrs.size() * sizeof(void*))}, same.options().dtype(at::kByte));
  auto stream = at::cuda::getCurrentCUDAStream();
  check(cudaMemcpyAsync(dev.data_ptr(), ptrs.data(), ptrs.size() * sizeof(void*), cudaMemcpyHostToDevice, stream),
        "pointer upload");
  check(hb::launch_ns_prepare((const void* const*)dev.data_ptr(), src_dt, (int)R, (int)C, (int)srcs.size(),
                              sumsq_t.data_ptr<float>(), (float)eps, same.data_ptr(), ld_same, R * ld_same,
                              trans.data_ptr(), ld_trans, C * ld_trans, seed, stream), "ns_prepare launch");
}

// D = A * B^T (bf16, K-major operands, batched) with the fused epilogues described in ns_gemm.h.
void ns_gemm(const at::Tensor& A, int64_t lda, int64_t strideA, const at::Tensor& B, int64_t ldb, int64_t strideB,
             int64_t M, int64_t N, int64_t K, int64_t batch, int mode, bool symmetric, const OptT& C, int64_t ldc,
             int64_t strideC, const OptT& CT, int64_t ldct, int64_t strideCT, const OptT& F, int64_t ldf, int64_t strideF,
             bool f_transposed, double f_scale, const OptT& S, int64_t lds, int64_t strideS, double ca, double cb,
             double cc, const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(A.device());
  hb::GemmParams P{};
  P.M = (int)M; P.N = (int)N; P.K = (int)K; P.batch = (int)batch; P.mode = mode; P.symmetric = symmetric ? 1 : 0;
  P.C = C.has_value() ? (__nv_bfloat16*)C->data_ptr() : nullptr; P.ldc = ldc; P.strideC = strideC;
  P.CT = CT.has_value() ? (__nv_bfloat16*)CT->data_ptr() : nullptr; P.ldct = ldct; P.strideCT = strideCT;
  P.F = F.has_value() ? F->data_ptr<float>() : nullptr; P.ldf = ldf; P.strideF = strideF;
  P.f_transposed = f_transposed ? 1 : 0; P.f_scale = (float)f_scale;
  P.S = S.has_value() ? (const __nv_bfloat16*)S->data_ptr() : nullptr; P.lds = lds; P.strideS = strideS;
  P.ca = (float)ca; P.cb = (float)cb; P.cc = (float)cc;
  P.status = status.data_ptr<int>();
  check(hb::launch_ns_gemm(A.data_ptr(), lda, strideA, B.data_ptr(), ldb, strideB, P, at::cuda::getCurrentCUDAStream()),
        "ns_gemm launch");
}

// The whole Newton-Schulz iteration of one shape bucket in one call: per step Gram, polynomial and apply launches (the
// last apply writes fp32 into `out`, in the caller's orientation).  x / xt: the two ping-pong pairs of the iterate
// [batch, m, ldx] and its transpose [batch, n, ldxt] (bf16), pair 0 prepared by ns_prepare; s, y: [batch, m, lds] (bf16).
void ns_chain(const std::vector<at::Tensor>& x, const std::vector<at::Tensor>& xt, const at::Tensor& s, const at::Tensor& y,
              at::Tensor& out, int64_t m, int64_t n, int64_t ldx, int64_t ldxt, int64_t lds, int64_t R, int64_t C,
              const std::vector<std::vector<double>>& coeffs, double out_scale, const at::Tensor& status) {
  TORCH_CHECK(x.size() == 2 && xt.size() == 2, "ns_chain: two ping-pong buffers per orientation");
  const int64_t batch = s.size(0);
  int cur = 0;
  const OptT none;
  for (size_t step = 0; step < coeffs.size(); ++step) {
    TORCH_CHECK(coeffs[step].size() == 3, "ns_chain: (a, b, c) per step");
    const bool last = step + 1 == coeffs.size();
    ns_gemm(x[cur], ldx, m * ldx, x[cur], ldx, m * ldx, m, m, n, batch, 0 /* gram */, true, s, lds, m * lds, s, lds, m * lds,
            none, 0, 0, false, 1.0, none, 0, 0, 0.0, 0.0, 0.0, status);
    ns_gemm(s, lds, m * lds, s, lds, m * lds, m, m, m, batch, 1 /* poly */, true, y, lds, m * lds, y, lds, m * lds, none, 0, 0,
            false, 1.0, s, lds, m * lds, coeffs[step][0], coeffs[step][1], coeffs[step][2], status);
    if (!last) {
      ns_gemm(y, lds, m * lds, xt[cur], ldxt, n * ldxt, m, n, m, batch, 2 /* apply */, false, x[1 - cur], ldx, m * ldx,
              xt[1 - cur], ldxt, n * ldxt, none, 0, 0, false, 1.0, none, 0, 0, 0.0, 0.0, 0.0, status);
      cur = 1 - cur;
    } else {
      ns_gemm(y, lds, m * lds, xt[cur], ldxt, n * ldxt, m, n, m, batch, 2 /* apply */, false, none, 0, 0, none, 0, 0, out, C,
              R * C, R > C, out_scale, none, 0, 0, 0.0, 0.0, 0.0, status);
    }
  }
}

// Store `epoch` into slot[rank] of every peer's flag array (after a system-scope fence).
void peer_signal(const std::vector<int64_t>& flag_ptrs, int slot, int rank, int epoch) {
  hb::PeerPtrs ptrs{};
  TORCH_CHECK((int)flag_ptrs.size() <= hb::kMaxWorld, "world size above kMaxWorld");
  for (size_t i = 0; i < flag_ptrs.size(); ++i) ptrs.ptr[i] = (uint64_t)flag_ptrs[i];
  check(hb::launch_peer_signal(ptrs, slot, rank, (int)flag_ptrs.size(), epoch, at::cuda::getCurrentCUDAStream()),
        "peer_signal launch");
}

// Wait (bounded) until every rank has stored `epoch` into `slot` of this rank's flag array.
void peer_wait(const at::Tensor& my_flags, int slot, int world, int epoch, double timeout_s, const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(my_flags.device());
  check(hb::launch_peer_wait(my_flags.data_ptr<int>(), slot, world, epoch, timeout_s, status.data_ptr<int>(),
                             at::cuda::getCurrentCUDAStream()), "peer_wait launch");
}

// In-place softmax cross-entropy: `logits` ([rows, ld] bf16) becomes the gradient of sum(loss) * scale[0];
// returns the per-row losses.
at::Tensor cross_entropy_(at::Tensor& logits, const at::Tensor& targets, const at::Tensor& scale, int64_t vocab,
                          int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kBFloat16, "logits: 2-D bf16 CUDA tensor");
  TORCH_CHECK(logits.is_contiguous() && logits.size(1) % 8 == 0 && aligned16(logits.data_ptr()),
              "logits must be contiguous with a row length that is a multiple of 8 (pad the vocabulary)");
  TORCH_CHECK(vocab > 0 && vocab <= logits.size(1), "vocab out of range");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
                  targets.numel() == logits.size(0), "targets: contiguous int64, one per row");
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == 1, "scale: fp32 device scalar");
  c10::cuda::CUDAGuard guard(logits.device());
  at::Tensor loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  check(hb::launch_cross_entropy(logits.data_ptr(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                                 loss.data_ptr<float>(), scale.data_ptr<float>(), logits.size(0), (int)vocab,
                                 (int)logits.size(1), ignore_index, at::cuda::getCurrentCUDAStream()),
        "cross_entropy launch");
  return loss;
}

// Split-tf32 operands of a contiguous fp32 [batch, R, C] tensor: rows of [hi | lo] (see tf32_gemm.h).  Returns
// (same, trans): same = [batch, R, 2 kp(C)] (operand rows = rows of x), trans = [batch, C, 2 kp(R)] (operand rows =
// columns of x); an orientation that was not asked for comes back undefined.
std::vector<at::Tensor> tf32_split(const at::Tensor& x, bool want_same, bool want_trans) {
  // views are welcome: any row and batch stride, unit inner stride
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 3 && x.stride(2) == 1 && x.size(0) >= 1 && x.size(1) >= 1 &&
                  x.size(2) >= 1, "tf32_split: fp32 [batch, rows, cols] CUDA tensor with unit inner stride");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t batch = x.size(0), R = x.size(1), C = x.size(2);
  at::Tensor same = want_same ? at::empty({batch, R, 2 * hb::tf32_split_kp(C)}, x.options().memory_format(at::MemoryFormat::Contiguous)) : at::Tensor();
  at::Tensor trans = want_trans ? at::empty({batch, C, 2 * hb::tf32_split_kp(R)}, x.options().memory_format(at::MemoryFormat::Contiguous)) : at::Tensor();
  check(hb::launch_tf32_split(x.data_ptr<float>(), x.stride(1), x.stride(0), (int)R, (int)C, (int)batch,
                              want_same ? same.data_ptr<float>() : nullptr, want_trans ? trans.data_ptr<float>() : nullptr,
                              at::cuda::getCurrentCUDAStream()), "tf32 split");
  return {same, trans};
}

// epilogue(A * B^T) over split operands a2: [batch, M, 2 kp(K)], b2: [batch, N, 2 kp(K)] (see tf32_gemm.h).
//   mode 0 store, 1 lerp into `c` with weight w, 2 Adam / 3 LaProp on the moments m, v ([batch, M, N] fp32, in place).
//   c: fp32 [batch, M, >= N] output (optional unless mode 1).  split_out: 0 none, 1 also / instead write the result as
//   a split operand with rows = output rows, 2 with rows = output columns; it is returned (undefined when 0).
at::Tensor tf32_gemm(const at::Tensor& a2, const at::Tensor& b2, int64_t K, int mode, double alpha, double w, double b1,
                     double b2c, double eps, const OptT& c, int split_out, const OptT& m, const OptT& v,
                     const at::Tensor& status) {
  TORCH_CHECK(a2.is_cuda() && b2.is_cuda() && a2.scalar_type() == at::kFloat && b2.scalar_type() == at::kFloat &&
                  a2.dim() == 3 && b2.dim() == 3 && a2.is_contiguous() && b2.is_contiguous() && a2.size(0) == b2.size(0),
              "tf32_gemm: contiguous fp32 split operands [batch, rows, 2 kp]");
  const int64_t batch = a2.size(0), M = a2.size(1), N = b2.size(1), kp = hb::tf32_split_kp(K);
  TORCH_CHECK(a2.size(2) == 2 * kp && b2.size(2) == 2 * kp, "tf32_gemm: operands were not split for K = ", K);
  c10::cuda::CUDAGuard guard(a2.device());
  hb::Tf32Epilogue E{};
  E.mode = mode; E.alpha = (float)alpha; E.w = (float)w; E.b1 = (float)b1; E.b2 = (float)b2c; E.eps = (float)eps;
  if (c.has_value() && c->defined()) {
    TORCH_CHECK(c->is_cuda() && c->scalar_type() == at::kFloat && c->dim() == 3 && c->size(0) == batch && c->size(1) == M &&
                    c->size(2) >= N && c->stride(2) == 1 && c->stride(1) >= N && c->device() == a2.device(),
                "tf32_gemm: c must be fp32 [batch, M, >= N] with unit inner stride");
    E.C = c->data_ptr<float>(); E.ldc = c->stride(1); E.strideC = c->stride(0);
  }
  at::Tensor s;
  if (split_out != 0) {
    const int64_t rows = split_out == 1 ? M : N, kps = hb::tf32_split_kp(split_out == 1 ? N : M);
    s = at::empty({batch, rows, 2 * kps}, a2.options());
    E.S = s.data_ptr<float>(); E.kpS = kps; E.strideS = rows * 2 * kps; E.s_transposed = split_out == 2 ? 1 : 0;
  }
  if (mode == hb::kEpiAdam || mode == hb::kEpiLaProp) {
    TORCH_CHECK(m.has_value() && v.has_value(), "tf32_gemm: moment buffers required");
    for (const at::Tensor* t : {&*m, &*v})
      TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == batch * M * N &&
                      t->device() == a2.device(), "tf32_gemm: moments must be contiguous fp32 [batch, M, N]");
    E.m = m->data_ptr<float>(); E.v = v->data_ptr<float>();
  }
  TORCH_CHECK(E.C != nullptr || E.S != nullptr, "tf32_gemm: no output requested");
  // X X^T (one buffer as both operands): upper tiles only, mirrored on store.  An in-place lerp target is then
  // symmetric by construction (it only ever receives symmetric increments).
  E.symmetric = (a2.data_ptr() == b2.data_ptr() && M == N && E.C != nullptr && E.S == nullptr &&
                 (mode == hb::kEpiStore || mode == hb::kEpiLerp || mode == hb::kEpiAdd)) ? 1 : 0;
  check(hb::launch_tf32_gemm(a2.data_ptr<float>(), b2.data_ptr<float>(), (int)M, (int)N, (int)K, (int)batch, E,
                             status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()), "tf32 gemm");
  return s;
}

// op(a) @ op(b) for batched fp32 matrices on the split-tf32 tensor-core path.  a: [batch, R, C]; ta = 0 uses a as
// [M, K], ta = 1 as [K, M]; likewise b is [K, N] for tb = 0 and [N, K] for tb = 1.  Returns [batch, M, N].
// upper_upper: op(a) and op(b) are both upper triangular (square, same size): only the non-zero K range of every tile
// is walked and the part below the diagonal comes back as zeros.
at::Tensor tf32x3_matmul(const at::Tensor& a, const at::Tensor& b, bool ta, bool tb, double alpha, const at::Tensor& status,
                         bool upper_upper) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat &&
                  a.dim() == 3 && b.dim() == 3 && a.is_contiguous() && b.is_contiguous() && a.size(0) == b.size(0),
              "tf32x3_matmul: contiguous fp32 [batch, rows, cols] CUDA tensors");
  const int64_t batch = a.size(0);
  const int64_t M = ta ? a.size(2) : a.size(1), K = ta ? a.size(1) : a.size(2);
  const int64_t N = tb ? b.size(1) : b.size(2), Kb = tb ? b.size(2) : b.size(1);
  TORCH_CHECK(K == Kb, "tf32x3_matmul: inner dimensions differ");
  c10::cuda::CUDAGuard guard(a.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t kp = hb::tf32_split_kp(K), ldc = (N + 3) / 4 * 4;
  at::Tensor a2 = at::empty({batch, M, 2 * kp}, a.options());
  const bool same_operand = a.data_ptr() == b.data_ptr() && a.sizes() == b.sizes() && ta != tb;  // X X^T or X^T X
  at::Tensor b2 = same_operand ? a2 : at::empty({batch, N, 2 * kp}, a.options());
  at::Tensor c = at::empty({batch, M, ldc}, a.options());
  check(hb::launch_tf32_split(a.data_ptr<float>(), a.size(2), a.size(1) * a.size(2), (int)a.size(1), (int)a.size(2),
                              (int)batch, ta ? nullptr : a2.data_ptr<float>(), ta ? a2.data_ptr<float>() : nullptr, stream),
        "tf32 split A");
  // B as the K-major [N, K] operand: b given as [K, N] must be transposed, b given as [N, K] is used as it is
  if (!same_operand)
    check(hb::launch_tf32_split(b.data_ptr<float>(), b.size(2), b.size(1) * b.size(2), (int)b.size(1), (int)b.size(2),
                                (int)batch, tb ? b2.data_ptr<float>() : nullptr, tb ? nullptr : b2.data_ptr<float>(), stream),
          "tf32 split B");
  hb::Tf32Epilogue E{};
  E.mode = hb::kEpiStore; E.alpha = (float)alpha; E.C = c.data_ptr<float>(); E.ldc = ldc; E.strideC = M * ldc;
  E.symmetric = same_operand ? 1 : 0;  // X X^T / X^T X: upper tiles, mirrored on store
  if (upper_upper) {
    TORCH_CHECK(M == N && M == K && !same_operand, "tf32x3_matmul: upper_upper needs two square matrices of one size");
    E.tri = 1;
  }
  check(hb::launch_tf32_gemm(a2.data_ptr<float>(), b2.data_ptr<float>(), (int)M, (int)N, (int)K, (int)batch, E,
                             status.data_ptr<int>(), stream), "tf32 gemm");
  return ldc == N ? c : c.narrow(2, 0, N);
}

// Partial products X^T W over the long dimension: x = first `m` columns of the contiguous [batch, n, k] tensor `base`,
// w: contiguous [batch, n, p], p <= 32.  Returns [splits, batch, m, p]; sum over dim 0 for the product.
at::Tensor tall_t_mul(const at::Tensor& base, int64_t m, const at::Tensor& w) {
  TORCH_CHECK(base.is_cuda() && w.is_cuda() && base.scalar_type() == at::kFloat && w.scalar_type() == at::kFloat &&
                  base.dim() == 3 && w.dim() == 3 && base.is_contiguous() && w.is_contiguous() &&
                  base.size(0) == w.size(0) && base.size(1) == w.size(1) && w.size(2) <= 32 && m >= 0 && m <= base.size(2),
              "tall_t_mul: contiguous fp32 [batch, n, k] and [batch, n, p <= 32]");
  c10::cuda::CUDAGuard guard(base.device());
  const int64_t batch = base.size(0), n = base.size(1), k = base.size(2), p = w.size(2);
  at::Tensor c = at::empty({hb::tall_splits((int)n), batch, m, p}, base.options());
  check(hb::launch_tall_t_mul(base.data_ptr<float>(), k, n * k, w.data_ptr<float>(), p, n * p, (int)batch, (int)n, (int)m,
                              (int)p, c.data_ptr<float>(), at::cuda::getCurrentCUDAStream()), "tall_t_mul launch");
  return c;
}

// Inverses of the 128 x 128 diagonal blocks of a batch of upper-triangular fp32 matrices q: [batch, n, n] (unit inner
// stride).  Returns [batch, ceil(n / 128), 128, 128]; entries below the diagonal of q are ignored.
at::Tensor tri_inv_blocks(const at::Tensor& q) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kFloat && q.dim() == 3 && q.size(1) == q.size(2) && q.stride(2) == 1,
              "tri_inv_blocks: fp32 [batch, n, n] CUDA tensor with unit inner stride");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t batch = q.size(0), n = q.size(1), nb = (n + hb::kTriBlock - 1) / hb::kTriBlock;
  at::Tensor x = at::empty({batch, nb, hb::kTriBlock, hb::kTriBlock}, q.options());
  check(hb::launch_tri_inv_blocks(q.data_ptr<float>(), q.stride(1), q.stride(0), (int)batch, (int)n, x.data_ptr<float>(),
                                  at::cuda::getCurrentCUDAStream()), "tri_inv_blocks launch");
  return x;
}

// Factors the diagonal leaf [lo, lo + size) of the batched symmetric positive definite fp32 matrices g ([batch, n, n], unit
// inner stride) as R^T R: writes R's block into r (same layout as g) and the block's inverse into inv[:, lo / 128]
// (inv: contiguous [batch, ceil(n / 128), 128, 128]); info: int32 [batch], incremented per matrix with a bad pivot.
void chol_inv_leaf(const at::Tensor& g, at::Tensor& r, at::Tensor& inv, int64_t lo, int64_t size, at::Tensor& info) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kFloat && g.dim() == 3 && g.size(1) == g.size(2) && g.stride(2) == 1 &&
                  r.is_cuda() && r.scalar_type() == at::kFloat && r.sizes() == g.sizes() && r.stride(2) == 1 &&
                  r.device() == g.device(), "chol_inv_leaf: fp32 [batch, n, n] CUDA tensors with unit inner stride");
  const int64_t batch = g.size(0), n = g.size(1), nb = (n + hb::kTriBlock - 1) / hb::kTriBlock;
  TORCH_CHECK(lo >= 0 && size >= 1 && size <= hb::kTriBlock && lo + size <= n && lo % hb::kTriBlock == 0,
              "chol_inv_leaf: leaf [lo, lo + size) must start on a multiple of 128 and hold at most 128 rows");
  TORCH_CHECK(inv.is_cuda() && inv.scalar_type() == at::kFloat && inv.is_contiguous() && inv.dim() == 4 && inv.size(0) == batch &&
                  inv.size(1) == nb && inv.size(2) == hb::kTriBlock && inv.size(3) == hb::kTriBlock && inv.device() == g.device(),
              "chol_inv_leaf: inv must be contiguous fp32 [batch, ceil(n / 128), 128, 128]");
  TORCH_CHECK(info.is_cuda() && info.scalar_type() == at::kInt && info.is_contiguous() && info.numel() == batch &&
                  info.device() == g.device(), "chol_inv_leaf: info must be int32 [batch]");
  c10::cuda::CUDAGuard guard(g.device());
  const int64_t blk = hb::kTriBlock * hb::kTriBlock;
  check(hb::launch_chol_inv_leaf(g.data_ptr<float>() + lo * g.stride(1) + lo, g.stride(1), g.stride(0),
                                 r.data_ptr<float>() + lo * r.stride(1) + lo, r.stride(1), r.stride(0),
                                 inv.data_ptr<float>() + (lo / hb::kTriBlock) * blk, nb * blk, (int)batch, (int)size,
                                 info.data_ptr<int>(), at::cuda::getCurrentCUDAStream()), "chol_inv_leaf launch");
}

// Row-major upper triangles of contiguous [batch, n, n] matrices (2- or 4-byte elements) as [batch, n (n + 1) / 2].
at::Tensor triu_pack(const at::Tensor& dense) {
  TORCH_CHECK(dense.is_cuda() && dense.dim() == 3 && dense.size(1) == dense.size(2) && dense.is_contiguous() &&
                  (dense.element_size() == 2 || dense.element_size() == 4) && dense.size(0) <= 65535,
              "triu_pack: contiguous [batch <= 65535, n, n] CUDA tensor with 2- or 4-byte elements");
  c10::cuda::CUDAGuard guard(dense.device());
  const int64_t n = dense.size(1);
  at::Tensor line = at::empty({dense.size(0), n * (n + 1) / 2}, dense.options());
  check(hb::launch_triu_pack(dense.data_ptr(), line.data_ptr(), (int)dense.element_size(), (int)dense.size(0), (int)n,
                             at::cuda::getCurrentCUDAStream()), "triu_pack launch");
  return line;
}

// Inverse of triu_pack; entries below the diagonal are zero.
at::Tensor triu_unpack(const at::Tensor& line, int64_t n) {
  TORCH_CHECK(line.is_cuda() && line.dim() == 2 && line.size(1) == n * (n + 1) / 2 && line.is_contiguous() &&
                  (line.element_size() == 2 || line.element_size() == 4) && line.size(0) <= 65535,
              "triu_unpack: contiguous [batch <= 65535, n (n + 1) / 2] CUDA tensor with 2- or 4-byte elements");
  c10::cuda::CUDAGuard guard(line.device());
  at::Tensor dense = at::empty({line.size(0), n, n}, line.options());
  check(hb::launch_triu_unpack(line.data_ptr(), dense.data_ptr(), (int)line.element_size(), (int)line.size(0), (int)n,
                               at::cuda::getCurrentCUDAStream()), "triu_unpack launch");
  return dense;
}

// fp32 column sums of a contiguous bf16 matrix [rows, cols] (cols % 8 == 0).
at::Tensor colsum_bf16(const at::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
                  x.size(1) % 8 == 0 && aligned16(x.data_ptr()), "colsum_bf16: contiguous bf16 [rows, cols], cols % 8 == 0");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({x.size(1)}, x.options().dtype(at::kFloat));
  at::Tensor partial = at::empty({hb::colsum_splits(), x.size(1)}, out.options());
  check(hb::launch_colsum_bf16(x.data_ptr(), x.size(0), (int)x.size(1), partial.data_ptr<float>(), out.data_ptr<float>(),
                               at::cuda::getCurrentCUDAStream()), "colsum launch");
  return out;
}

// Concatenated fp32 column sums of up to four contiguous bf16 matrices of one shape: out[i * cols + c].
at::Tensor colsum_bf16_batch(const std::vector<at::Tensor>& xs) {
  TORCH_CHECK(!xs.empty() && xs.size() <= (size_t)hb::kColsumMaxBatch, "colsum_bf16_batch: one to four matrices");
  const void* ptrs[hb::kColsumMaxBatch];
  for (size_t i = 0; i < xs.size(); ++i) {
    const at::Tensor& x = xs[i];
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.size(1) % 8 == 0 &&
                    aligned16(x.data_ptr()) && x.sizes() == xs[0].sizes() && x.device() == xs[0].device(),
                "colsum_bf16_batch: contiguous bf16 [rows, cols] of one shape, cols % 8 == 0");
    ptrs[i] = x.data_ptr();
  }
  c10::cuda::CUDAGuard guard(xs[0].device());
  const int64_t n = (int64_t)xs.size(), cols = xs[0].size(1);
  at::Tensor out = at::empty({n * cols}, xs[0].options().dtype(at::kFloat));
  at::Tensor partial = at::empty({n, hb::colsum_splits(), cols}, out.options());
  check(hb::launch_colsum_bf16_batch(ptrs, (int)n, xs[0].size(0), (int)cols, partial.data_ptr<float>(), out.data_ptr<float>(),
                                     at::cuda::getCurrentCUDAStream()), "colsum batch launch");
  return out;
}

// y = gelu_tanh(u) for a contiguous bf16 tensor whose element count is a multiple of 8.
at::Tensor gelu_fwd(const at::Tensor& u) {
  TORCH_CHECK(u.is_cuda() && u.scalar_type() == at::kBFloat16 && u.is_contiguous() && u.numel() % 8 == 0 &&
                  aligned16(u.data_ptr()), "gelu_fwd: contiguous bf16, numel % 8 == 0");
  c10::cuda::CUDAGuard guard(u.device());
  at::Tensor y = at::empty_like(u);
  check(hb::launch_gelu_fwd(u.data_ptr(), y.data_ptr(), u.numel(), at::cuda::getCurrentCUDAStream()), "gelu_fwd launch");
  return y;
}

// (du, dbias) = (dy * gelu_tanh'(u), column sums of that product in fp32) for contiguous bf16 [rows, cols], cols % 8 == 0.
std::vector<at::Tensor> gelu_bwd(const at::Tensor& dy, const at::Tensor& u) {
  TORCH_CHECK(u.is_cuda() && u.dim() == 2 && u.scalar_type() == at::kBFloat16 && u.is_contiguous() && u.size(1) % 8 == 0 &&
                  aligned16(u.data_ptr()), "gelu_bwd: u contiguous bf16 [rows, cols], cols % 8 == 0");
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.sizes() == u.sizes() &&
                  dy.device() == u.device() && aligned16(dy.data_ptr()), "gelu_bwd: dy like u");
  c10::cuda::CUDAGuard guard(u.device());
  const int64_t rows = u.size(0), cols = u.size(1);
  at::Tensor du = at::empty_like(u);
  at::Tensor dbias = rows > 0 ? at::empty({cols}, u.options().dtype(at::kFloat)) : at::zeros({cols}, u.options().dtype(at::kFloat));
  if (rows > 0 && cols > 0) {
    at::Tensor partial = at::empty({hb::gelu_bwd_splits(rows, (int)cols), cols}, dbias.options());
    check(hb::launch_gelu_bwd(dy.data_ptr(), u.data_ptr(), du.data_ptr(), rows, (int)cols, partial.data_ptr<float>(),
                              dbias.data_ptr<float>(), at::cuda::getCurrentCUDAStream()), "gelu_bwd launch");
  }
  return {du, dbias};
}

// LayerNorm over the last dimension of a contiguous fp32 tensor.  With `res` (same shape, bf16 or fp32) the normalised
// tensor is x + res, which is returned as a fourth tensor.  Returns (y, mean, rstd[, x + res]); y is bf16 when asked.
std::vector<at::Tensor> layer_norm_fwd(const at::Tensor& x, const OptT& res, const at::Tensor& gamma, const at::Tensor& beta,
                                       double eps, bool out_bf16) {
  const int64_t D = x.size(-1);
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous(), "x: contiguous fp32 CUDA tensor");
  TORCH_CHECK(hb::layer_norm_supported((int)D), "row length must be a multiple of 128, at most 1024");
  TORCH_CHECK(gamma.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && gamma.numel() == D &&
                  beta.numel() == D && gamma.is_contiguous() && beta.is_contiguous(), "gamma / beta: fp32 [D]");
  const bool has_res = res.has_value() && res->defined();
  if (has_res)
    TORCH_CHECK(res->is_cuda() && res->is_contiguous() && res->numel() == x.numel() &&
                    (res->scalar_type() == at::kFloat || res->scalar_type() == at::kBFloat16), "res: contiguous fp32 / bf16 like x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.numel() / D;
  at::Tensor y = at::empty(x.sizes(), x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  at::Tensor mean = at::empty({rows}, x.options()), rstd = at::empty({rows}, x.options());
  at::Tensor xsum = has_res ? at::empty_like(x) : at::Tensor();
  check(hb::launch_layer_norm_fwd(x.data_ptr<float>(), has_res ? res->data_ptr() : nullptr,
                                  has_res && res->scalar_type() == at::kBFloat16, has_res ? xsum.data_ptr<float>() : nullptr,
                                  gamma.data_ptr<float>(), beta.data_ptr<float>(), y.data_ptr(), out_bf16,
                                  mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, (int)D, (float)eps,
                                  at::cuda::getCurrentCUDAStream()), "layer_norm_fwd launch");
  if (has_res) return {y, mean, rstd, xsum};
  return {y, mean, rstd};
}

// Returns (dx, dgamma, dbeta[, bf16 copy of dx]) for dy in fp32 or bf16; `dres` (fp32, optional) is added to dx.
std::vector<at::Tensor> layer_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gamma,
                                       const at::Tensor& mean, const at::Tensor& rstd, const OptT& dres, bool dx_bf16) {
  const int64_t D = x.size(-1);
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.numel() == x.numel() &&
                  (dy.scalar_type() == at::kFloat || dy.scalar_type() == at::kBFloat16), "dy: contiguous fp32 / bf16");
  TORCH_CHECK(x.scalar_type() == at::kFloat && x.is_contiguous() && hb::layer_norm_supported((int)D), "x: contiguous fp32");
  const bool has_dres = dres.has_value() && dres->defined();
  if (has_dres)
    TORCH_CHECK(dres->is_cuda() && dres->is_contiguous() && dres->scalar_type() == at::kFloat && dres->numel() == x.numel(),
                "dres: contiguous fp32 like x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.numel() / D;
  const int n_cta = hb::layer_norm_partial_ctas(rows);
  at::Tensor dx = at::empty_like(x), dgamma = at::empty_like(gamma), dbeta = at::empty_like(gamma);
  at::Tensor partial = at::empty({n_cta, 2 * D}, x.options());
  at::Tensor dx16 = dx_bf16 ? at::empty(x.sizes(), x.options().dtype(at::kBFloat16)) : at::Tensor();
  check(hb::launch_layer_norm_bwd(dy.data_ptr(), dy.scalar_type() == at::kBFloat16, x.data_ptr<float>(),
                                  gamma.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                  has_dres ? dres->data_ptr<float>() : nullptr, dx.data_ptr<float>(),
                                  dx_bf16 ? dx16.data_ptr() : nullptr, dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), partial.data_ptr<float>(), n_cta, rows,
                                  (int)D, at::cuda::getCurrentCUDAStream()), "layer_norm_bwd launch");
  if (dx_bf16) return {dx, dgamma, dbeta, dx16};
  return {dx, dgamma, dbeta};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("tf32x3_matmul", &tf32x3_matmul);
  m.def("tf32_split", &tf32_split);
  m.def("tf32_gemm", &tf32_gemm);
  m.def("colsum_bf16", &colsum_bf16);
  m.def("colsum_bf16_batch", &colsum_bf16_batch);
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("tall_t_mul", &tall_t_mul);
  m.def("tri_inv_blocks", &tri_inv_blocks);
  m.def("layer_norm_fwd", &layer_norm_fwd);
  m.def("layer_norm_bwd", &layer_norm_bwd);
  m.def("layer_norm_supported", &hb::layer_norm_supported);
  m.def("cross_entropy_", &cross_entropy_);
  m.def("peer_signal", &peer_signal);
  m.def("peer_wait", &peer_wait);
  m.attr("MAX_WORLD") = hb::kMaxWorld;
  m.def("fused_chain", &fused_chain);
  m.def("sumsq", &sumsq);
  m.def("segmented_reduce", &segmented_reduce);
  m.def("ns_prepare", &ns_prepare);
  m.def("ns_gemm", &ns_gemm);
  m.def("ns_chain", &ns_chain);
  m.def("set_ns_gemm_tile", &hb::set_ns_gemm_tile_override);
  m.def("set_tf32_gemm_tile", &hb::set_tf32_gemm_tile_override);
  m.def("chol_inv_leaf", &chol_inv_leaf);
  m.def("triu_pack", &triu_pack);
  m.def("triu_unpack", &triu_unpack);
  m.def("chunk_elems", &hb::chain_chunk_elems);
}
