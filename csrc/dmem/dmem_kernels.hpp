// Host entry points of the dmem / coherence kernels.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

#include <cstdint>

namespace mccl {

// One immediate as it sits in a receiver's ring (32 bytes; seq is written last, with release semantics).
struct ImmWire {
  uint32_t seq;
  uint32_t imm;
  uint32_t region_id;
  uint32_t src_node;
  uint64_t offset;
  uint64_t length;
};
// Writes `rec` into `slot` (a ring entry in a peer's symmetric memory) after everything the stream did before.
cudaError_t launch_dmem_post_imm(ImmWire* slot, const ImmWire& rec, cudaStream_t stream);

// SM-driven copy of n bytes; either pointer may be a peer mapping.
cudaError_t launch_dmem_copy(void* dst, const void* src, size_t n, cudaStream_t stream);
// peer_flags_dev: device array of `world` pointers, entry p = peer p's epoch pad (one word per source rank).
cudaError_t launch_coherence_release(unsigned int* const* peer_flags_dev, int world, int rank, unsigned int epoch,
                                     cudaStream_t stream);
cudaError_t launch_coherence_acquire(const unsigned int* my_flags, int world, int rank, unsigned int epoch,
                                     unsigned long long timeout_ns, int* status_dev, cudaStream_t stream);
cudaError_t launch_dmem_atomic_selftest(unsigned int* counter, unsigned long long* slot, float* sum, int adds,
                                        cudaStream_t stream);

}  // namespace mccl
