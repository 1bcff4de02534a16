// Kernels built from the device-side dmem operations: a grid-wide copy to or
// from peer memory (what host-side put / get use when the caller wants the SMs
// rather than a copy engine to move the data), the stream-ordered acquire /
// release pair of the coherence layer, and a small self-test of the atomics.
#include "../core/launch.hpp"
#include "dmem_kernels.hpp"

#include "device/dmem.cuh"

namespace mccl {

namespace {

__global__ void __launch_bounds__(512) dmem_copy_kernel(char* dst, const char* src, unsigned long long n) {
  const unsigned long long units = (n + 15) / 16;
  const unsigned long long per = (units + gridDim.x - 1) / gridDim.x * 16;
  unsigned long long b0 = blockIdx.x * per, b1 = b0 + per;
  if (b0 > n) b0 = n;
  if (b1 > n) b1 = n;
  dmem::cta_copy(dst + b0, src + b0, b1 - b0);
}

// release: everything this stream wrote before is visible to peers that observe the new epoch.
__global__ void coherence_release_kernel(unsigned int* const* peer_flags, int world, int rank, unsigned int epoch) {
  if (threadIdx.x < world && threadIdx.x != rank) {
    __threadfence_system();
    dmem::signal(peer_flags[threadIdx.x] + rank, epoch);
  }
}

// acquire: wait (bounded) until every listed peer has released `epoch`; status 0 = ok, else 1 + peer.
__global__ void coherence_acquire_kernel(const unsigned int* my_flags, int world, int rank, unsigned int epoch,
                                         unsigned long long timeout_ns, int* status) {
  if (threadIdx.x < world && threadIdx.x != rank) {
    if (!dmem::wait_until(my_flags + threadIdx.x, epoch, timeout_ns)) atomicCAS(status, 0, 1 + static_cast<int>(threadIdx.x));
  }
}

// The record's payload first, then its sequence number with a system-scope release: a receiver that
// sees the number also sees the payload and the data the stream copied before this kernel.
__global__ void dmem_post_imm_kernel(ImmWire* slot, ImmWire rec) {
  slot->imm = rec.imm;
  slot->region_id = rec.region_id;
  slot->src_node = rec.src_node;
  slot->offset = rec.offset;
  slot->length = rec.length;
  __threadfence_system();
  dmem::signal(&slot->seq, rec.seq);
}

__global__ void dmem_atomic_selftest_kernel(unsigned int* remote_counter, unsigned long long* remote_slot, float* remote_sum,
                                            int adds) {
  for (int i = threadIdx.x; i < adds; i += blockDim.x) {
    dmem::atomic_add(remote_counter, 1u);
    dmem::atomic_add(remote_sum, 0.5f);
  }
  if (threadIdx.x == 0) {
    dmem::atomic_cas(remote_slot, 0ull, 42ull);   // succeeds once
    dmem::atomic_cas(remote_slot, 0ull, 43ull);   // must fail
  }
}

}  // namespace

cudaError_t launch_dmem_copy(void* dst, const void* src, size_t n, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  size_t want = (n + (64u << 10) - 1) / (64u << 10);
  int ctas = static_cast<int>(want < 1 ? 1 : (want > 64 ? 64 : want));
  MCCL_LAUNCH(dmem_copy_kernel, ctas, 512, 0, stream, static_cast<char*>(dst), static_cast<const char*>(src), n);
  return ::mccl::launch_status();
}

cudaError_t launch_dmem_post_imm(ImmWire* slot, const ImmWire& rec, cudaStream_t stream) {
  MCCL_LAUNCH(dmem_post_imm_kernel, 1, 1, 0, stream, slot, rec);
  return ::mccl::launch_status();
}

cudaError_t launch_coherence_release(unsigned int* const* peer_flags_dev, int world, int rank, unsigned int epoch,
                                     cudaStream_t stream) {
  MCCL_LAUNCH(coherence_release_kernel, 1, 32, 0, stream, peer_flags_dev, world, rank, epoch);
  return ::mccl::launch_status();
}

cudaError_t launch_coherence_acquire(const unsigned int* my_flags, int world, int rank, unsigned int epoch,
                                     unsigned long long timeout_ns, int* status_dev, cudaStream_t stream) {
  MCCL_LAUNCH(coherence_acquire_kernel, 1, 32, 0, stream, my_flags, world, rank, epoch, timeout_ns, status_dev);
  return ::mccl::launch_status();
}

cudaError_t launch_dmem_atomic_selftest(unsigned int* counter, unsigned long long* slot, float* sum, int adds,
                                        cudaStream_t stream) {
  MCCL_LAUNCH(dmem_atomic_selftest_kernel, 1, 256, 0, stream, counter, slot, sum, adds);
  return ::mccl::launch_status();
}

}  // namespace mccl
