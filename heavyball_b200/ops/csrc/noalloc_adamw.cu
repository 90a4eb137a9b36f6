// Implementation of the allocation-free cautious AdamW step declared in noalloc_adamw.h.
//
// The regular two-phase caution path needs three pieces of device scratch: the tensor table the
// multi-tensor kernel reads, an int counter of masked elements, and an fp32 buffer that parks the
// masked update between the phases.  Here all three live in one file-scope device array, so the call
// performs no allocation of any kind (no cudaMalloc / cudaFree, no framework allocator).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "fused_chain.h"
#include "noalloc_adamw.h"

namespace {

constexpr long long kMaxElems = HB200_NOALLOC_MAX_ELEMS;
constexpr size_t kHeaderBytes = 4096;  // [0, 2048): tensor table + chunk prefix, [2048, 2052): masked counter
constexpr size_t kCounterOffset = 2048;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle: its device address must be obtained
// with cudaGetSymbolAddress (done once per device in scratch_base()).
static __device__ __align__(256) unsigned char g_scratch[kHeaderBytes + sizeof(float) * kMaxElems];

void* g_base[kMaxDevices] = {nullptr};

int fail(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) snprintf(err, (size_t)err_len, "%s", msg);
  return code;
}

// Device address of the scratch array on the current device (looked up on first use).
cudaError_t scratch_base(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (g_base[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess) return e;
    g_base[dev] = ptr;
  }
  *out = (unsigned char*)g_base[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int hb200_cautious_adamw_step_noalloc(float* param, const float* grad, float* exp_avg, float* exp_avg_sq,
                                                 long long numel, float lr, float beta1, float beta2, float eps,
                                                 float weight_decay, void* stream_, char* err, int err_len) {
  if (param == nullptr || grad == nullptr || exp_avg == nullptr || exp_avg_sq == nullptr)
    return fail(err, err_len, -1, "hb200_cautious_adamw_step_noalloc: null buffer");
  if (numel <= 0) return fail(err, err_len, -1, "hb200_cautious_adamw_step_noalloc: numel must be positive");
  if (numel > kMaxElems) {
    char msg[192];
    snprintf(msg, sizeof(msg),
             "hb200_cautious_adamw_step_noalloc: numel %lld exceeds the fixed scratch capacity of %lld elements; "
             "split the tensor or use the allocating path",
             numel, kMaxElems);
    return fail(err, err_len, -1, msg);
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  unsigned char* base = nullptr;
  cudaError_t e = scratch_base(&base);
  if (e != cudaSuccess) return fail(err, err_len, (int)e, cudaGetErrorString(e));

  int* masked = (int*)(base + kCounterOffset);
  float* parked = (float*)(base + kHeaderBytes);

  // table for a single tensor, followed by its chunk prefix {0, n_chunks}
  struct {
    hb::TensorMeta meta;
    int prefix[2];
  } host;
  memset(&host, 0, sizeof(host));
  const int chunk = hb::chain_chunk_elems();
  const int n_chunks = (int)((numel + chunk - 1) / chunk);
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  host.meta.p = param;
  host.meta.g = (void*)grad;
  host.meta.u = parked;
  host.meta.s0 = exp_avg;
  host.meta.s1 = exp_avg_sq;
  host.meta.masked = masked;
  host.meta.numel = numel;
  host.meta.vec_ok = (aligned(param) && aligned(grad) && aligned(exp_avg) && aligned(exp_avg_sq)) ? 1 : 0;
  host.prefix[0] = 0;
  host.prefix[1] = n_chunks;
  static_assert(sizeof(host) <= kCounterOffset, "table must fit in the header");

  // the counter must start at zero on every call; the parked update is fully overwritten by phase one
  e = cudaMemsetAsync(masked, 0, sizeof(int), stream);
  if (e != cudaSuccess) return fail(err, err_len, (int)e, cudaGetErrorString(e));
  e = cudaMemcpyAsync(base, &host, sizeof(host), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return fail(err, err_len, (int)e, cudaGetErrorString(e));
  const hb::TensorMeta* metas = (const hb::TensorMeta*)base;
  const int* prefix = (const int*)(base + offsetof(decltype(host), prefix));

  hb::ChainParams P;
  memset(&P, 0, sizeof(P));
  P.n_tensors = 1;
  P.dt_p = hb::kNone; P.dt_g = hb::kF32; P.dt_u = hb::kF32; P.dt_s = hb::kF32;
  P.algo = hb::kAdam; P.n_state = 2; P.out_mode = hb::kOutUpdate;
  P.b1 = beta1; P.b2 = beta2; P.eps = eps;
  e = hb::launch_fused_chain(metas, prefix, n_chunks, P, /*count_caution=*/true, stream);  // moments, mask, count, park
  if (e != cudaSuccess) return fail(err, err_len, (int)e, cudaGetErrorString(e));

  memset(&P, 0, sizeof(P));
  P.n_tensors = 1;
  P.dt_p = hb::kF32; P.dt_g = hb::kNone; P.dt_u = hb::kF32; P.dt_s = hb::kNone;
  P.algo = hb::kIdentity; P.u_is_input = 1; P.caution_apply = 1; P.out_mode = hb::kOutParam;
  P.lr = lr; P.wd = weight_decay;
  e = hb::launch_fused_chain(metas, prefix, n_chunks, P, /*count_caution=*/false, stream);  // rescale and apply
  if (e != cudaSuccess) return fail(err, err_len, (int)e, cudaGetErrorString(e));
  return 0;
}
