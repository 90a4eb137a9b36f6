// Cross-GPU synchronisation for the peer-memory data-parallel step: epoch flags in symmetric memory.
//
// Every rank owns an int array `flags[slot * kMaxWorld + src_rank]` that its peers write.  A signal stores
// the current epoch into slot[my_rank] of every peer (after a system-scope fence, so everything this
// stream wrote before is visible to a peer that observes the flag); a wait spins until every entry of a
// slot has reached the epoch.  Waits are bounded by a clock budget: on expiry the kernel records the
// fact in a status word and returns, so a missing peer can never wedge the GPU.
//
// The kernels that move the data (multi-source gradient loads, multi-destination parameter stores)
// are the ordinary fused-chain kernels with peer address deltas; see fused_chain.cu.
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer_sync.h"

namespace hb {

__global__ void peer_signal_kernel(PeerPtrs flags, int slot, int rank, int world, int epoch) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    int* dst = (int*)flags.ptr[t] + slot * kMaxWorld + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
  }
}

__global__ void peer_wait_kernel(const int* my_flags, int slot, int world, int epoch, long long budget_cycles,
                                 int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    const int* src = my_flags + slot * kMaxWorld + t;
    const long long start = clock64();
    int seen;
    for (;;) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(src) : "memory");
      if (seen >= epoch) break;
      if (clock64() - start > budget_cycles) {
        atomicExch(status, 2 + t);  // 2 + rank of the peer that never arrived
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  __threadfence_system();
}

cudaError_t launch_peer_signal(const PeerPtrs& flags, int slot, int rank, int world, int epoch, cudaStream_t stream) {
  peer_signal_kernel<<<1, 32, 0, stream>>>(flags, slot, rank, world, epoch);
  return cudaGetLastError();
}

cudaError_t launch_peer_wait(const int* my_flags, int slot, int world, int epoch, double timeout_s, int* status,
                             cudaStream_t stream) {
  // the clock-rate attribute is a driver round trip of about a millisecond: ask once per device
  static int khz_of[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int khz = (dev >= 0 && dev < 64) ? khz_of[dev] : 0;
  if (khz == 0) {
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    if (khz <= 0) khz = 1500000;
    if (dev >= 0 && dev < 64) khz_of[dev] = khz;
  }
  const long long budget = (long long)(timeout_s * 1e3 * (double)khz);
  peer_wait_kernel<<<1, 32, 0, stream>>>(my_flags, slot, world, epoch, budget, status);
  return cudaGetLastError();
}

}  // namespace hb
