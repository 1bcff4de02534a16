// Device-side one-sided operations on peer-mapped memory (NVLink).
//
// A remote address is an ordinary pointer: the mapping of the peer's symmetric
// heap block in this process (SymmAlloc::ptrs[peer] + offset).  These are the
// in-kernel counterparts of the host-side put / get / put_with_imm / fence of
// the reference's DistributedMemoryManager (csrc/dmem/DistributedMemoryManager.cpp:215-300),
// which the reference can only issue from the host through a NIC.
//
//   dmem::put / dmem::get           CTA-cooperative copies, 16 bytes per access
//   dmem::atomic_add / cas / exch   system-scope atomics on a peer's words
//   dmem::signal / wait_until       release store to a peer's flag, bounded
//                                   acquire spin on an own flag
//   dmem::fence                     orders this thread's earlier remote writes
//                                   before its later ones (system scope)
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace mccl {
namespace dmem {

__device__ __forceinline__ void fence() { __threadfence_system(); }

// Copies n bytes with all threads of the CTA.  Pointers may be local or peer-mapped, any alignment.
__device__ __forceinline__ void cta_copy(void* dst, const void* src, unsigned long long n) {
  char* d = static_cast<char*>(dst);
  const char* s = static_cast<const char*>(src);
  if (((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(s)) & 15u) == 0) {
    const unsigned long long vecs = n / 16;
    for (unsigned long long i = threadIdx.x; i < vecs; i += blockDim.x)
      reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
    for (unsigned long long b = vecs * 16 + threadIdx.x; b < n; b += blockDim.x) d[b] = s[b];
  } else {
    for (unsigned long long b = threadIdx.x; b < n; b += blockDim.x) d[b] = s[b];
  }
}
__device__ __forceinline__ void put(void* remote_dst, const void* local_src, unsigned long long n) { cta_copy(remote_dst, local_src, n); }
__device__ __forceinline__ void get(void* local_dst, const void* remote_src, unsigned long long n) { cta_copy(local_dst, remote_src, n); }

__device__ __forceinline__ unsigned int atomic_add(unsigned int* remote, unsigned int v) { return atomicAdd_system(remote, v); }
__device__ __forceinline__ unsigned long long atomic_add(unsigned long long* remote, unsigned long long v) { return atomicAdd_system(remote, v); }
__device__ __forceinline__ float atomic_add(float* remote, float v) { return atomicAdd_system(remote, v); }
__device__ __forceinline__ unsigned int atomic_cas(unsigned int* remote, unsigned int expect, unsigned int desired) {
  return atomicCAS_system(remote, expect, desired);
}
__device__ __forceinline__ unsigned long long atomic_cas(unsigned long long* remote, unsigned long long expect, unsigned long long desired) {
  return atomicCAS_system(remote, expect, desired);
}
__device__ __forceinline__ unsigned int atomic_exch(unsigned int* remote, unsigned int v) { return atomicExch_system(remote, v); }

// Publishes `value` to a peer's flag after this thread's earlier writes (call after a
// __syncthreads() when the whole CTA wrote the data).
__device__ __forceinline__ void signal(unsigned int* remote_flag, unsigned int value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote_flag), "r"(value) : "memory");
}
// Spins until *flag >= value (wrap-safe).  Returns false when timeout_ns elapsed first.
__device__ __forceinline__ bool wait_until(const unsigned int* flag, unsigned int value, unsigned long long timeout_ns) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned spins = 0;; ++spins) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - value) >= 0) return true;
    if ((spins & 63u) == 63u) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > timeout_ns) return false;
    }
  }
}

}  // namespace dmem
}  // namespace mccl
