// Allocation-free cautious AdamW step for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference library (heavyball); it exists for embedding
// this library's kernels where the caller owns all memory.
//
// Who needs it: code that runs the optimizer from a place where calling cudaMalloc (or anything that
// may call it, such as a framework's caching allocator) is not possible or not allowed - a real-time
// training loop with a fixed memory budget, a host process that has handed the whole device to
// another allocator, or a plain C / ctypes client with no tensor library at all.  The regular path (`heavyball_b200.ops.fused_chain`) takes its scratch
// space - the parked masked update and the per-tensor mask counter that caution needs, plus the
// tensor table - from the PyTorch allocator on every call; this variant keeps that scratch in a
// fixed array inside the loaded library instead.
//
// Semantics (identical arithmetic to the regular caution path, fp32 buffers, one tensor):
//     m <- lerp(m, g, beta1);  v <- lerp(v, g*g, beta2);  u = m / max(sqrt(v), eps)
//     u <- 0 where sign(u) != sign(g);  u <- u * numel / max(numel - #masked, 1)
//     p <- p * (1 - weight_decay * lr) - lr * u
// `beta1` / `beta2` are the coefficients actually applied this step (already debiased by the caller,
// `1 - (1 - beta) / (1 - beta^step)`).
//
// Limits and rules:
//   * at most HB200_NOALLOC_MAX_ELEMS elements per call (the scratch array is that many floats plus a
//     4 KiB header, about 16 MiB, resident on every GPU that loads the library until the process exits);
//     larger sizes are refused with a message and a non-zero return value, nothing is launched;
//   * the first call on each device looks up the device address of the scratch array
//     (cudaGetSymbolAddress) with that device current; make that first call outside any stream capture;
//   * all calls share the one array: two calls whose kernels may overlap on the GPU (different
//     streams without ordering) race on it.  Calls on one stream, or otherwise ordered, are safe; the
//     parts that must start from zero are cleared by every call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define HB200_NOALLOC_MAX_ELEMS (1LL << 22)

// All pointers are device pointers to contiguous fp32 buffers of `numel` elements on the current
// device.  `stream` is a cudaStream_t (null = default stream).  `err` (may be null) receives a
// zero-terminated message of at most `err_len` bytes when the return value is non-zero.
// Returns 0 on success, -1 for invalid arguments / size over the limit, otherwise a cudaError_t value.
int hb200_cautious_adamw_step_noalloc(float* param, const float* grad, float* exp_avg, float* exp_avg_sq,
                                      long long numel, float lr, float beta1, float beta2, float eps,
                                      float weight_decay, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
