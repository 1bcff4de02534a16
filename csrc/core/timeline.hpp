// Device-side timeline: kernels stamp %globaltimer at entry and exit into a
// record buffer, so the overlap of collective kernels with compute kernels
// inside a replayed CUDA graph can be read without a profiler attached.
//
// Off by default (kernels receive a null buffer and skip one branch).  Enabled
// per device with timeline_enable(); the buffer pointer is a kernel argument,
// so a CUDA graph must be captured after the timeline was enabled for its
// kernels to record.  The reference traces its Metal command-buffer commits
// on the host (csrc/metal/CommitTrace.hpp:15-26); here the interesting events
// are on the device, so that is where they are stamped.
#pragma once

#include <cstdint>
#include <vector>

namespace mccl {

struct TimelineRec {
  unsigned long long t0;   // %globaltimer at entry (ns)
  unsigned long long t1;   // %globaltimer at exit (ns)
  uint32_t kind;           // TimelineKind
  uint32_t tag;            // kernel-specific (GEMM: m tiles << 16 | n tiles; collective: CTAs in the grid)
  uint32_t sm;             // %smid of the recording CTA
  uint32_t cta;            // blockIdx.x
};

struct TimelineBuf {
  uint32_t cap;
  uint32_t count;          // records requested so far (may exceed cap; the excess is dropped)
  uint32_t every;          // a CTA records when blockIdx.x % every == 0
  uint32_t detail;         // non-zero: kernels that have them also record their inner phases (TL_GEMM_PHASE)
  TimelineRec rec[1];      // cap entries follow
};

enum TimelineKind : uint32_t {
  TL_GEMM = 1,
  TL_ALLREDUCE = 2,
  TL_OTHER_COLL = 3,
  TL_OP = 4,
  TL_GEMM_PHASE = 5,       // tag: phase << 24 | tile ordinal of the CTA; phases: 0 set-up, 1 wait for the accumulator, 2 epilogue
};

// Host side (timeline.cu).  All functions act on the current CUDA device.
// Allocates (once) a buffer of `capacity` records; `every` selects which CTAs record.
void timeline_enable(int capacity, int every, int detail = 0);
void timeline_disable();
// Device pointer kernels should receive, or nullptr while disabled.
TimelineBuf* timeline_device_ptr();
// Synchronises the device, copies the records out and rewinds the buffer.
std::vector<TimelineRec> timeline_drain();

#if defined(__CUDACC__)
__device__ __forceinline__ unsigned long long tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Entry stamp: 0 when this CTA does not record.
__device__ __forceinline__ unsigned long long tl_begin(const TimelineBuf* tl) {
  if (tl == nullptr) return 0ull;
  if (threadIdx.x != 0 || (blockIdx.x % tl->every) != 0) return 0ull;
  return tl_now();
}
__device__ __forceinline__ void tl_end(TimelineBuf* tl, unsigned long long t0, uint32_t kind, uint32_t tag) {
  if (tl == nullptr || t0 == 0ull) return;
  const uint32_t i = atomicAdd(&tl->count, 1u);
  if (i >= tl->cap) return;
  uint32_t sm;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  TimelineRec r;
  r.t0 = t0;
  r.t1 = tl_now();
  r.kind = kind;
  r.tag = tag;
  r.sm = sm;
  r.cta = blockIdx.x;
  tl->rec[i] = r;
}
// A record of an inner phase [t0, t1), written by one thread of a CTA that records.
__device__ __forceinline__ bool tl_detail(const TimelineBuf* tl) {
  return tl != nullptr && tl->detail != 0 && (blockIdx.x % tl->every) == 0;
}
__device__ __forceinline__ void tl_mark(TimelineBuf* tl, unsigned long long t0, unsigned long long t1, uint32_t kind, uint32_t tag) {
  const uint32_t i = atomicAdd(&tl->count, 1u);
  if (i >= tl->cap) return;
  uint32_t sm;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  TimelineRec r;
  r.t0 = t0;
  r.t1 = t1;
  r.kind = kind;
  r.tag = tag;
  r.sm = sm;
  r.cta = blockIdx.x;
  tl->rec[i] = r;
}
#endif

}  // namespace mccl
