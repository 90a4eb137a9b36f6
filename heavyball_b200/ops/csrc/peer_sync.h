// Epoch-flag signalling between GPUs of one node (peer_sync.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

constexpr int kMaxWorld = 16;

struct PeerPtrs {
  uint64_t ptr[kMaxWorld];  // device address of the same symmetric buffer on every rank
};

cudaError_t launch_peer_signal(const PeerPtrs& flags, int slot, int rank, int world, int epoch, cudaStream_t stream);
cudaError_t launch_peer_wait(const int* my_flags, int slot, int world, int epoch, double timeout_s, int* status,
                             cudaStream_t stream);

}  // namespace hb
