// Host entry points of the dmem / coherence kernels.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

namespace mccl {

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
