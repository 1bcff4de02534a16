// Device-side building blocks of the collective kernels: the communicator
// view a kernel receives, per-CTA cross-GPU barriers with bounded waits,
// 16-byte vector access, wire-dtype conversion and the reduction operators.
//
// Synchronisation scheme.  Every rank owns a signal pad in peer-mapped
// memory: flags[cta][src] is written by CTA `cta` of rank `src` and read only
// by CTA `cta` of the owner.  Values are monotonically increasing epochs, so
// flags are never reset; each CTA keeps its epoch in RankState between
// launches, which makes every kernel replayable inside a CUDA graph.  A CTA
// only ever consumes data produced by the same CTA index on its peers, so no
// grid-wide synchronisation is needed.  All waits are bounded by a
// globaltimer deadline; when one runs out the kernel writes a status word
// the host reads, and returns.  (The reference bounds its event waits the same
// way on the host: csrc/metal/EventSync.mm:36-63.)
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../core/timeline.hpp"
#include "coll_args.hpp"

namespace mccl {
namespace dev {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 128;
constexpr int kThreads = 512;
constexpr int kFlagWordsPerChannel = kMaxCtas * kMaxRanks;
constexpr int kChannels = 4;  // independent flag sets so kernels on different streams never share flags

// Persistent per-(rank, channel) words the kernels keep between launches.
struct RankState {
  uint32_t seq;           // collectives finished on this channel; parity picks the arena half
  uint32_t done_ctas;     // CTAs of the running kernel that have finished
  uint32_t skip_signals;  // host-made fault for tests: signal rounds this rank must skip
  uint32_t reserved;
  uint32_t epoch[kMaxCtas];
};

struct DevComm {
  int world;
  int rank_base;                 // global rank of virtual rank 0 (virtual ranks only exist in 1-GPU emulation)
  char* arena[kMaxRanks];        // every rank's staging arena as mapped here
  uint32_t* flags[kMaxRanks];    // every rank's signal pad (already offset to the channel)
  char* mc_arena;                // NVLS multicast mapping of the arenas, or nullptr
  RankState* state[kMaxRanks];   // indexed by virtual rank
  int* status[kMaxRanks];        // indexed by virtual rank; 0 = healthy
  unsigned long long half_bytes; // size of one arena half
  unsigned long long timeout_ns;
  TimelineBuf* tl;               // device timeline, or nullptr (off)
  unsigned long long arena_limit; // MCCL_DEBUG_BOUNDS: usable bytes of an arena (canaries start here); 0 = checks off
};

// ---- point-to-point (send / recv) ----
// Every rank owns an inbound region in peer-mapped memory with two buffers of slot_bytes per source
// rank.  The sender writes chunk number `seq` of the pair's stream into buffer seq & 1 of the
// receiver's region and raises ready[cta][src] = seq on the receiver's pad; the receiver copies the
// chunk out and raises free[cta][dst] = seq on the sender's pad, which lets chunk seq + 2 be written.
// Sequence numbers live in device memory per (rank, peer, direction), so the n-th send to a peer
// pairs with the n-th receive from it and the kernels can be replayed from a CUDA graph.
struct P2PState {
  uint32_t send_seq[kMaxRanks];
  uint32_t recv_seq[kMaxRanks];
  uint32_t send_done[kMaxRanks];   // CTAs of the running send kernel that have finished, per peer
  uint32_t recv_done[kMaxRanks];
};
struct P2PComm {
  int world;
  int rank_base;
  char* region[kMaxRanks];       // rank r's inbound region as mapped here: [src][2][slot_bytes]
  uint32_t* ready[kMaxRanks];    // rank r's pad, "chunk written" flags: [cta][src]
  uint32_t* free_[kMaxRanks];    // rank r's pad, "chunk consumed" flags: [cta][dst]
  P2PState* state[kMaxRanks];    // indexed by virtual rank
  int* status[kMaxRanks];        // indexed by virtual rank
  unsigned long long slot_bytes;
  unsigned long long timeout_ns;
};
constexpr int kP2PMaxCtas = 16;

enum Phase : int { PH_BARRIER = 1, PH_PUSH = 2, PH_REDUCE = 3, PH_GATHER = 4, PH_RING = 5, PH_TREE = 6, PH_NVLS = 7, PH_SEND = 8, PH_RECV = 9, PH_BOUNDS = 10 };

__host__ __device__ inline int encode_status(int phase, int peer) { return (1 << 30) | (phase << 8) | (peer & 0xff); }

// ------------------------------------------------------------------ memory --
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Plain 16-byte accesses (no volatile): the barriers' asm statements carry the
// memory clobbers that keep data accesses on the right side of each meeting, and
// between meetings the compiler is free to keep several loads in flight.
__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// --------------------------------------------------------------- CTA state --
struct CtaSync {
  uint32_t epoch;
  uint32_t half;   // which arena half this launch uses
  bool skip;       // host-made fault: do not signal
  unsigned long long tl_t0;  // timeline entry stamp (0: this CTA does not record)
};

// Called by every thread at kernel start.
__device__ __forceinline__ CtaSync cta_begin(const DevComm& c, int vr) {
  CtaSync s;
  RankState* st = c.state[vr];
  s.epoch = st->epoch[blockIdx.x];
  s.half = st->seq & 1u;
  s.skip = st->skip_signals != 0;
  s.tl_t0 = tl_begin(c.tl);
  return s;
}

// Called by every thread at kernel end (also on the failure path).  The last
// CTA to finish advances the sequence number, which flips the arena half for
// the next launch; all CTAs of this launch have read it by then.
__device__ __forceinline__ void cta_end(const DevComm& c, int vr, const CtaSync& s, uint32_t tl_kind = TL_OTHER_COLL) {
  __syncthreads();
  if (threadIdx.x == 0) {
    tl_end(c.tl, s.tl_t0, tl_kind, gridDim.x);
    RankState* st = c.state[vr];
    st->epoch[blockIdx.x] = s.epoch;
    __threadfence();
    uint32_t prev = atomicAdd(&st->done_ctas, 1u);
    if (prev + 1 == gridDim.x) {
      st->done_ctas = 0;
      st->seq = st->seq + 1;
      if (st->skip_signals) st->skip_signals = st->skip_signals - 1;
      __threadfence();
    }
  }
}

__device__ __forceinline__ void report_timeout(const DevComm& c, int vr, int phase, int peer) {
  volatile int* s = c.status[vr];
  if (*s == 0) *s = encode_status(phase, peer);
  __threadfence_system();
}

// MCCL_DEBUG_BOUNDS: every kernel states, before its first access, the last arena byte (exclusive) it will
// touch on any rank.  When that lies beyond the arena the kernel records a violation in the status word
// (phase "bounds", peer field = this rank) and returns without dereferencing anything, instead of writing
// into whatever follows the arena in the peers' address spaces.
__device__ __forceinline__ bool bounds_violation(const DevComm& c, int vr, unsigned long long arena_end) {
  if (c.arena_limit == 0) return false;
  // the launch works inside one half: [half * half_bytes, (half + 1) * half_bytes)
  const unsigned long long half_begin = (c.state[vr]->seq & 1u) * c.half_bytes;
  if (arena_end <= half_begin + c.half_bytes && arena_end <= c.arena_limit) return false;
  if (threadIdx.x == 0) report_timeout(c, vr, PH_BOUNDS, c.rank_base + vr);
  return true;
}

// Signals `peer` (its flag for this CTA and this source rank becomes `value`).
// Call from one thread after a __syncthreads() that follows the data writes.
__device__ __forceinline__ void signal_peer(const DevComm& c, int rank, int peer, uint32_t value) {
  st_release_sys(c.flags[peer] + blockIdx.x * kMaxRanks + rank, value);
}

// Spins until `peer` has signalled at least `value`.  Returns false on timeout.
__device__ __forceinline__ bool wait_peer(const DevComm& c, int vr, int rank, int peer, uint32_t value, int phase) {
  const uint32_t* src = c.flags[rank] + blockIdx.x * kMaxRanks + peer;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    uint32_t v = ld_acquire_sys(src);
    if (static_cast<int32_t>(v - value) >= 0) return true;
    if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > c.timeout_ns) {
      report_timeout(c, vr, phase, peer);
      return false;
    }
  }
}

// Barrier between CTA `blockIdx.x` of every rank.  Orders all global writes
// made by this CTA before the barrier ahead of all reads made by the peers'
// CTAs after it.  Returns true when a wait ran out (the caller must then skip
// the rest of its work and go to cta_end).
__device__ __forceinline__ bool barrier_all(const DevComm& c, int vr, int rank, CtaSync& s, int phase) {
  __syncthreads();
  s.epoch += 1;
  bool bad = false;
  const int t = threadIdx.x;
  if (t < c.world) {
    if (!s.skip) signal_peer(c, rank, t, s.epoch);
    bad = !wait_peer(c, vr, rank, t, s.epoch, phase);
  }
  return __syncthreads_or(bad ? 1 : 0) != 0;
}

// Point-to-point forms used by ring and tree (one signalling thread).
__device__ __forceinline__ void signal_one(const DevComm& c, int rank, int peer, uint32_t value, const CtaSync& s) {
  __syncthreads();
  if (threadIdx.x == 0 && !s.skip) signal_peer(c, rank, peer, value);
}
__device__ __forceinline__ bool wait_one(const DevComm& c, int vr, int rank, int peer, uint32_t value, int phase) {
  bool bad = false;
  if (threadIdx.x == 0) bad = !wait_peer(c, vr, rank, peer, value, phase);
  return __syncthreads_or(bad ? 1 : 0) != 0;
}

// --------------------------------------------------------------- elements --

template <typename T> struct Elem;
template <> struct Elem<float> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(float v) { return v; }
  static __device__ __forceinline__ float down(Acc v) { return v; }
};
template <> struct Elem<double> {
  using Acc = double;
  static __device__ __forceinline__ Acc up(double v) { return v; }
  static __device__ __forceinline__ double down(Acc v) { return v; }
};
template <> struct Elem<__half> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(Acc v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(Acc v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<int32_t> {
  using Acc = int32_t;
  static __device__ __forceinline__ Acc up(int32_t v) { return v; }
  static __device__ __forceinline__ int32_t down(Acc v) { return v; }
};
template <> struct Elem<int64_t> {
  using Acc = long long;
  static __device__ __forceinline__ Acc up(int64_t v) { return v; }
  static __device__ __forceinline__ int64_t down(Acc v) { return v; }
};

template <typename A> struct IsIntegral { static constexpr bool value = false; };
template <> struct IsIntegral<int32_t> { static constexpr bool value = true; };
template <> struct IsIntegral<long long> { static constexpr bool value = true; };

template <typename A>
__device__ __forceinline__ A apply_op(int op, A a, A b) {
  switch (op) {
    case OP_SUM: case OP_AVG: return a + b;
    case OP_MIN: return b < a ? b : a;
    case OP_MAX: return b > a ? b : a;
    case OP_PROD: return a * b;
    default: break;
  }
  if constexpr (IsIntegral<A>::value) {
    switch (op) {
      case OP_BAND: return a & b;
      case OP_BOR: return a | b;
      case OP_BXOR: return a ^ b;
      default: break;
    }
  }
  return a;
}

// AVG finalisation: floats multiply by 1/world, integers divide by world.
template <typename A>
__device__ __forceinline__ A finish_avg(A v, int world, float inv_world) {
  if constexpr (IsIntegral<A>::value) return v / static_cast<A>(world);
  else return v * static_cast<A>(inv_world);
}

// A "pack" is the unit every thread moves: 16 bytes of the narrower of the
// data type T and the wire type W.
template <typename T, typename W> struct Pack {
  static constexpr int kElems = 16 / (sizeof(W) < sizeof(T) ? sizeof(W) : sizeof(T));
  using Acc = typename Elem<T>::Acc;
};

// Loads n_valid (≤ kElems) elements of type X starting at p into acc[].
// The vector path needs p 16-byte aligned and a full pack.
template <typename X, int kElems, typename Acc>
__device__ __forceinline__ void load_pack(const X* p, Acc (&acc)[kElems], int n_valid, bool aligned) {
  constexpr int kPerVec = 16 / sizeof(X);
  if (aligned && n_valid == kElems) {
#pragma unroll
    for (int v = 0; v < kElems / kPerVec; ++v) {
      uint4 raw = ld16(p + v * kPerVec);
      const X* e = reinterpret_cast<const X*>(&raw);
#pragma unroll
      for (int i = 0; i < kPerVec; ++i) acc[v * kPerVec + i] = static_cast<Acc>(Elem<X>::up(e[i]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < kElems; ++i) acc[i] = i < n_valid ? static_cast<Acc>(Elem<X>::up(p[i])) : Acc(0);
  }
}

template <typename X, int kElems, typename Acc>
__device__ __forceinline__ void store_pack(X* p, const Acc (&acc)[kElems], int n_valid, bool aligned) {
  constexpr int kPerVec = 16 / sizeof(X);
  if (aligned && n_valid == kElems) {
#pragma unroll
    for (int v = 0; v < kElems / kPerVec; ++v) {
      uint4 raw;
      X* e = reinterpret_cast<X*>(&raw);
#pragma unroll
      for (int i = 0; i < kPerVec; ++i) e[i] = Elem<X>::down(static_cast<typename Elem<X>::Acc>(acc[v * kPerVec + i]));
      st16(p + v * kPerVec, raw);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kElems; ++i)
      if (i < n_valid) p[i] = Elem<X>::down(static_cast<typename Elem<X>::Acc>(acc[i]));
  }
}

// Rounds accumulator values through the wire type so that the rank that
// reduced a chunk keeps exactly the bits its peers will receive.
template <typename T, typename W, int kElems, typename Acc>
__device__ __forceinline__ void round_through_wire(Acc (&acc)[kElems]) {
  if constexpr (sizeof(W) < sizeof(T)) {
#pragma unroll
    for (int i = 0; i < kElems; ++i)
      acc[i] = static_cast<Acc>(Elem<W>::up(Elem<W>::down(static_cast<typename Elem<W>::Acc>(acc[i]))));
  }
}

// Contiguous share of `packs` work units owned by this CTA.
__device__ __forceinline__ void cta_span(long long packs, long long& begin, long long& end) {
  long long per = (packs + gridDim.x - 1) / gridDim.x;
  begin = static_cast<long long>(blockIdx.x) * per;
  end = begin + per;
  if (begin > packs) begin = packs;
  if (end > packs) end = packs;
}

}  // namespace dev
}  // namespace mccl
