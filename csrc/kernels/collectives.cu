// Collective kernels over peer-mapped memory (NVLink 5 / NVSwitch), sm_100a.
//
// Each kernel is the whole collective: it stages or pushes data into the
// peers' arenas with 16-byte stores, meets the peers on the signal pad, and
// reduces / pulls with 16-byte loads, applying the wire cast (fp32 → bf16 on
// the wire, fp32 accumulation) and the AVG scale in registers.  These replace
// the reference's host loops of socket send/recv plus Metal reduce kernels
// (csrc/backend/AllreduceAlgos.cpp:52-206, ProcessGroupMCCL.cpp:188-601,
// csrc/metal/shaders.metal:196-552); schedule names follow the reference:
//   twoshot  = "butterfly": direct reduce-scatter + direct allgather
//   oneshot  = latency path used where the reference picks "tree" under auto
//   ring, tree = same step structure as the reference, flags instead of sockets
//   nvls     = in-switch reduction with multimem.ld_reduce / multimem.st
//
// blockIdx.y is the virtual rank and is non-zero only in single-GPU
// emulation, where all ranks' CTAs run as one cooperative launch so that the
// index arithmetic and the flag protocol can be tested on one device.
#include "collectives.hpp"

#include <cstdlib>

#include <cstdio>
#include <type_traits>

#include "../core/launch.hpp"
#include "comm_device.cuh"

namespace mccl {
namespace dev {

namespace {

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ int valid_in_pack(long long first, long long limit, int pack) {
  long long left = limit - first;
  return left >= pack ? pack : (left > 0 ? static_cast<int>(left) : 0);
}

// Copies n bytes; both pointers may have any alignment.  Work is split over
// the threads of this CTA only (the caller has already picked the CTA's byte
// range when more than one CTA shares a copy).
__device__ __forceinline__ void cta_copy_bytes(char* dst, const char* src, unsigned long long n) {
  if (n == 0) return;
  if (aligned16(dst) && aligned16(src)) {
    unsigned long long vecs = n / 16;
    unsigned long long i = threadIdx.x;
    // four independent 16-byte transfers in flight per thread
    for (; i + 3ull * blockDim.x < vecs; i += 4ull * blockDim.x) {
      uint4 a = reinterpret_cast<const uint4*>(src)[i];
      uint4 b = reinterpret_cast<const uint4*>(src)[i + blockDim.x];
      uint4 c = reinterpret_cast<const uint4*>(src)[i + 2ull * blockDim.x];
      uint4 d = reinterpret_cast<const uint4*>(src)[i + 3ull * blockDim.x];
      reinterpret_cast<uint4*>(dst)[i] = a;
      reinterpret_cast<uint4*>(dst)[i + blockDim.x] = b;
      reinterpret_cast<uint4*>(dst)[i + 2ull * blockDim.x] = c;
      reinterpret_cast<uint4*>(dst)[i + 3ull * blockDim.x] = d;
    }
    for (; i < vecs; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (unsigned long long b = vecs * 16 + threadIdx.x; b < n; b += blockDim.x) dst[b] = src[b];
  } else if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 3u) == 0) {
    unsigned long long words = n / 4;
    for (unsigned long long i = threadIdx.x; i < words; i += blockDim.x)
      reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
    for (unsigned long long b = words * 4 + threadIdx.x; b < n; b += blockDim.x) dst[b] = src[b];
  } else {
    for (unsigned long long b = threadIdx.x; b < n; b += blockDim.x) dst[b] = src[b];
  }
}

// Same copy, for sources that a peer rewrites while this kernel runs (staging slots that are reused round after
// round inside one launch): the loads go to L2 (ld.global.cg), so a line that this SM cached in an earlier round
// cannot be served again from L1.
__device__ __forceinline__ void cta_copy_bytes_uncached(char* dst, const char* src, unsigned long long n) {
  if (n == 0) return;
  if (aligned16(dst) && aligned16(src)) {
    unsigned long long vecs = n / 16;
    unsigned long long i = threadIdx.x;
    for (; i + 3ull * blockDim.x < vecs; i += 4ull * blockDim.x) {
      uint4 a = __ldcg(reinterpret_cast<const uint4*>(src) + i);
      uint4 b = __ldcg(reinterpret_cast<const uint4*>(src) + i + blockDim.x);
      uint4 c = __ldcg(reinterpret_cast<const uint4*>(src) + i + 2ull * blockDim.x);
      uint4 d = __ldcg(reinterpret_cast<const uint4*>(src) + i + 3ull * blockDim.x);
      reinterpret_cast<uint4*>(dst)[i] = a;
      reinterpret_cast<uint4*>(dst)[i + blockDim.x] = b;
      reinterpret_cast<uint4*>(dst)[i + 2ull * blockDim.x] = c;
      reinterpret_cast<uint4*>(dst)[i + 3ull * blockDim.x] = d;
    }
    for (; i < vecs; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = __ldcg(reinterpret_cast<const uint4*>(src) + i);
    for (unsigned long long b = vecs * 16 + threadIdx.x; b < n; b += blockDim.x) dst[b] = __ldcg(src + b);
  } else if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 3u) == 0) {
    unsigned long long words = n / 4;
    for (unsigned long long i = threadIdx.x; i < words; i += blockDim.x)
      reinterpret_cast<uint32_t*>(dst)[i] = __ldcg(reinterpret_cast<const uint32_t*>(src) + i);
    for (unsigned long long b = words * 4 + threadIdx.x; b < n; b += blockDim.x) dst[b] = __ldcg(src + b);
  } else {
    for (unsigned long long b = threadIdx.x; b < n; b += blockDim.x) dst[b] = __ldcg(src + b);
  }
}

// Copies n bytes from src to up to kMaxRanks destinations (peers' memory): every 16-byte unit is loaded once and
// stored to each destination, several units in flight per thread.  Stores to peers are posted, so this is the fast
// direction over NVLink.  Destinations must be 16-byte aligned; an unaligned source takes the per-destination path.
__device__ __forceinline__ void cta_push_bytes(char* const* dsts, int ndst, const char* src, unsigned long long n) {
  if (n == 0 || ndst == 0) return;
  if (!aligned16(src)) {
    for (int d = 0; d < ndst; ++d) cta_copy_bytes(dsts[d], src, n);
    return;
  }
  const unsigned long long vecs = n / 16;
  constexpr int U = 4;
  for (unsigned long long i0 = threadIdx.x; i0 < vecs; i0 += static_cast<unsigned long long>(blockDim.x) * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned long long i = i0 + static_cast<unsigned long long>(u) * blockDim.x;
      if (i < vecs) v[u] = reinterpret_cast<const uint4*>(src)[i];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned long long i = i0 + static_cast<unsigned long long>(u) * blockDim.x;
      if (i >= vecs) continue;
      for (int d = 0; d < ndst; ++d) reinterpret_cast<uint4*>(dsts[d])[i] = v[u];
    }
  }
  for (unsigned long long b = vecs * 16 + threadIdx.x; b < n; b += blockDim.x) {
    const char c = src[b];
    for (int d = 0; d < ndst; ++d) dsts[d][b] = c;
  }
}

// Byte range [begin, end) of an n-byte segment owned by this CTA, in 16-byte units.
__device__ __forceinline__ void cta_byte_span(unsigned long long n, unsigned long long& begin, unsigned long long& end) {
  unsigned long long units = (n + 15) / 16;
  unsigned long long per = (units + gridDim.x - 1) / gridDim.x;
  begin = blockIdx.x * per * 16;
  end = begin + per * 16;
  if (begin > n) begin = n;
  if (end > n) end = n;
}

}  // namespace

// ============================================================== two-shot ==
// kScatter = false: allreduce.  kScatter = true: reduce-scatter (input holds
// world chunks of exactly a.numel elements; output is this rank's chunk).
template <typename T, typename W, bool kScatter>
__global__ void __launch_bounds__(kThreads) twoshot_kernel(DevComm c, CollArgs a) {
  using PK = Pack<T, W>;
  constexpr int E = PK::kElems;
  using Acc = typename PK::Acc;
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const T* in = static_cast<const T*>(a.in[vr]);
  T* out = static_cast<T*>(a.out[vr]);
  const long long per = a.per;                         // arena slot length (elements, padded)
  const long long stride = kScatter ? a.stride : per;  // distance between chunks in the input
  const long long total = kScatter ? a.stride * (N - 1) + a.numel : a.numel;
  const size_t slot_bytes = static_cast<size_t>(per) * sizeof(W);
  const size_t recv_off = static_cast<size_t>(s.half) * c.half_bytes;
  const size_t red_off = recv_off + static_cast<size_t>(N) * slot_bytes;
  if (bounds_violation(c, vr, red_off + slot_bytes)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  long long pb, pe;
  cta_span(per / E, pb, pe);
  auto chunk_limit = [&](int p) -> long long {  // one past the last valid element of chunk p
    long long lim = static_cast<long long>(p) * stride + (kScatter ? a.numel : per);
    return lim < total ? lim : total;
  };

  // Phase 1: push my copy of chunk p to rank p.  Four packs per thread are loaded
  // before any is stored so that several local reads are in flight per thread.
  constexpr int U = 4;
  for (long long i0 = pb + threadIdx.x; i0 < pe; i0 += static_cast<long long>(blockDim.x) * U) {
#pragma unroll 1
    for (int k = 1; k < N; ++k) {
      const int p = (rank + k) % N;
      Acc v[U][E];
      int nv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * blockDim.x;
        const long long e0 = static_cast<long long>(p) * stride + i * E;
        nv[u] = i < pe ? valid_in_pack(e0, chunk_limit(p), E) : 0;
        if (nv[u] > 0) load_pack<T, E, Acc>(in + e0, v[u], nv[u], aligned16(in + e0));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (nv[u] <= 0) continue;
        const long long i = i0 + static_cast<long long>(u) * blockDim.x;
        W* dst = reinterpret_cast<W*>(c.arena[p] + recv_off + static_cast<size_t>(rank) * slot_bytes) + i * E;
        store_pack<W, E, Acc>(dst, v[u], E, true);
      }
    }
  }
  if (barrier_all(c, vr, rank, s, PH_PUSH)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }

  // Phase 2: reduce chunk `rank` (own copy in full precision, peers' from the arena).
  for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
    const long long e0 = static_cast<long long>(rank) * stride + i * E;
    const int nv = valid_in_pack(e0, chunk_limit(rank), E);
    if (nv <= 0) continue;
    Acc acc[E];
    load_pack<T, E, Acc>(in + e0, acc, nv, aligned16(in + e0));
    uint4 slots[kMaxRanks];
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src)
      if (src < N && src != rank)
        slots[src] = ld16(c.arena[rank] + recv_off + static_cast<size_t>(src) * slot_bytes + static_cast<size_t>(i) * 16);
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src) {
      if (src < N && src != rank) {
        const W* w = reinterpret_cast<const W*>(&slots[src]);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = apply_op<Acc>(a.op, acc[e], static_cast<Acc>(Elem<W>::up(w[e])));
      }
    }
    if (a.op == OP_AVG) {
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = finish_avg<Acc>(acc[e], N, a.inv_world);
    }
    if constexpr (kScatter) {
      T* op = out + i * E;
      store_pack<T, E, Acc>(op, acc, nv, aligned16(op));
    } else {
      round_through_wire<T, W, E, Acc>(acc);
      store_pack<W, E, Acc>(reinterpret_cast<W*>(c.arena[rank] + red_off) + i * E, acc, E, true);
      store_pack<T, E, Acc>(out + e0, acc, nv, aligned16(out + e0));
    }
  }
  if constexpr (kScatter) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  } else {
    if (barrier_all(c, vr, rank, s, PH_REDUCE)) {
      cta_end(c, vr, s, TL_ALLREDUCE);
      return;
    }
    // Phase 3: pull every other rank's reduced chunk.  All loads of a batch are
    // issued before its stores; small worlds batch several packs per peer so that
    // about eight remote reads are in flight per thread whatever N is.
    auto pull = [&](auto u_tag, auto p_tag) {
      constexpr int PU = decltype(u_tag)::value, PP = decltype(p_tag)::value;
      for (long long i0 = pb + threadIdx.x; i0 < pe; i0 += static_cast<long long>(blockDim.x) * PU) {
        uint4 raw[PU][PP];
#pragma unroll
        for (int u = 0; u < PU; ++u) {
          const long long i = i0 + static_cast<long long>(u) * blockDim.x;
#pragma unroll
          for (int k = 1; k <= PP; ++k)
            if (k < N && i < pe) raw[u][k - 1] = ld16(c.arena[(rank + k) % N] + red_off + static_cast<size_t>(i) * 16);
        }
#pragma unroll
        for (int u = 0; u < PU; ++u) {
          const long long i = i0 + static_cast<long long>(u) * blockDim.x;
#pragma unroll
          for (int k = 1; k <= PP; ++k) {
            if (k < N && i < pe) {
              const int p = (rank + k) % N;
              const long long e0 = static_cast<long long>(p) * per + i * E;
              const int nv = valid_in_pack(e0, chunk_limit(p), E);
              if (nv > 0) {
                Acc v[E];
                const W* w = reinterpret_cast<const W*>(&raw[u][k - 1]);
#pragma unroll
                for (int e = 0; e < E; ++e) v[e] = static_cast<Acc>(Elem<W>::up(w[e]));
                store_pack<T, E, Acc>(out + e0, v, nv, aligned16(out + e0));
              }
            }
          }
        }
      }
    };
    if (N <= 2) pull(std::integral_constant<int, 8>{}, std::integral_constant<int, 1>{});
    else if (N <= 4) pull(std::integral_constant<int, 3>{}, std::integral_constant<int, 3>{});
    else pull(std::integral_constant<int, 1>{}, std::integral_constant<int, kMaxRanks - 1>{});
    cta_end(c, vr, s, TL_ALLREDUCE);
  }
}

// ======================================================== two-shot, pushed ==
// Same reduce-scatter as above, but the all-gather half is pushed too: the owner of a chunk stores the reduced
// (wire-typed) chunk into every peer's arena and each rank then unpacks from its own arena.  Nothing is ever
// loaded from a peer, and loads are the slow direction over NVLink (a load's round trip bounds how much a
// thread can keep in flight, a store is posted).  Costs one more local pass and N instead of one result slots.
template <typename T, typename W>
__global__ void __launch_bounds__(kThreads) twoshot_push_kernel(DevComm c, CollArgs a) {
  using PK = Pack<T, W>;
  constexpr int E = PK::kElems;
  using Acc = typename PK::Acc;
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const T* in = static_cast<const T*>(a.in[vr]);
  T* out = static_cast<T*>(a.out[vr]);
  const long long per = a.per;
  const long long total = a.numel;
  const size_t slot_bytes = static_cast<size_t>(per) * sizeof(W);
  const size_t recv_off = static_cast<size_t>(s.half) * c.half_bytes;
  const size_t gath_off = recv_off + static_cast<size_t>(N) * slot_bytes;
  if (bounds_violation(c, vr, gath_off + static_cast<size_t>(N) * slot_bytes)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  long long pb, pe;
  cta_span(per / E, pb, pe);
  auto chunk_limit = [&](int p) -> long long {
    long long lim = static_cast<long long>(p + 1) * per;
    return lim < total ? lim : total;
  };
  // Phase 1: push my copy of chunk p to rank p.
  constexpr int U = 4;
  for (long long i0 = pb + threadIdx.x; i0 < pe; i0 += static_cast<long long>(blockDim.x) * U) {
#pragma unroll 1
    for (int k = 1; k < N; ++k) {
      const int p = (rank + k) % N;
      Acc v[U][E];
      int nv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * blockDim.x;
        const long long e0 = static_cast<long long>(p) * per + i * E;
        nv[u] = i < pe ? valid_in_pack(e0, chunk_limit(p), E) : 0;
        if (nv[u] > 0) load_pack<T, E, Acc>(in + e0, v[u], nv[u], aligned16(in + e0));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (nv[u] <= 0) continue;
        const long long i = i0 + static_cast<long long>(u) * blockDim.x;
        W* dst = reinterpret_cast<W*>(c.arena[p] + recv_off + static_cast<size_t>(rank) * slot_bytes) + i * E;
        store_pack<W, E, Acc>(dst, v[u], E, true);
      }
    }
  }
  if (barrier_all(c, vr, rank, s, PH_PUSH)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  // Phase 2: reduce chunk `rank`, keep it, and push the wire-typed result to every peer.
  for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
    const long long e0 = static_cast<long long>(rank) * per + i * E;
    const int nv = valid_in_pack(e0, chunk_limit(rank), E);
    if (nv <= 0) continue;
    Acc acc[E];
    load_pack<T, E, Acc>(in + e0, acc, nv, aligned16(in + e0));
    uint4 slots[kMaxRanks];
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src)
      if (src < N && src != rank)
        slots[src] = ld16(c.arena[rank] + recv_off + static_cast<size_t>(src) * slot_bytes + static_cast<size_t>(i) * 16);
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src) {
      if (src < N && src != rank) {
        const W* w = reinterpret_cast<const W*>(&slots[src]);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = apply_op<Acc>(a.op, acc[e], static_cast<Acc>(Elem<W>::up(w[e])));
      }
    }
    if (a.op == OP_AVG) {
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = finish_avg<Acc>(acc[e], N, a.inv_world);
    }
    round_through_wire<T, W, E, Acc>(acc);
    uint4 raw;
    {
      W* w = reinterpret_cast<W*>(&raw);
#pragma unroll
      for (int e = 0; e < E; ++e) w[e] = Elem<W>::down(static_cast<typename Elem<W>::Acc>(acc[e]));
    }
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k) {
      if (k < N) {
        const int p = (rank + k) % N;
        st16(c.arena[p] + gath_off + static_cast<size_t>(rank) * slot_bytes + static_cast<size_t>(i) * 16, raw);
      }
    }
    store_pack<T, E, Acc>(out + e0, acc, nv, aligned16(out + e0));
  }
  if (barrier_all(c, vr, rank, s, PH_REDUCE)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  // Phase 3: unpack the other ranks' chunks from my own arena.
  for (int k = 1; k < N; ++k) {
    const int p = (rank + k) % N;
    const char* src = c.arena[rank] + gath_off + static_cast<size_t>(p) * slot_bytes;
    for (long long i0 = pb + threadIdx.x; i0 < pe; i0 += static_cast<long long>(blockDim.x) * U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * blockDim.x;
        if (i < pe) raw[u] = ld16(src + static_cast<size_t>(i) * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * blockDim.x;
        if (i >= pe) continue;
        const long long e0 = static_cast<long long>(p) * per + i * E;
        const int nv = valid_in_pack(e0, chunk_limit(p), E);
        if (nv <= 0) continue;
        Acc v[E];
        const W* w = reinterpret_cast<const W*>(&raw[u]);
#pragma unroll
        for (int e = 0; e < E; ++e) v[e] = static_cast<Acc>(Elem<W>::up(w[e]));
        store_pack<T, E, Acc>(out + e0, v, nv, aligned16(out + e0));
      }
    }
  }
  cta_end(c, vr, s, TL_ALLREDUCE);
}

// =============================================================== one-shot ==
template <typename T, typename W>
__global__ void __launch_bounds__(kThreads) oneshot_kernel(DevComm c, CollArgs a) {
  using PK = Pack<T, W>;
  constexpr int E = PK::kElems;
  using Acc = typename PK::Acc;
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const T* in = static_cast<const T*>(a.in[vr]);
  T* out = static_cast<T*>(a.out[vr]);
  const long long padded = (a.numel + 15) / 16 * 16;
  const size_t slot_bytes = static_cast<size_t>(padded) * sizeof(W);
  const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
  if (bounds_violation(c, vr, base + static_cast<size_t>(N) * slot_bytes)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  long long pb, pe;
  cta_span(padded / E, pb, pe);
  const bool al_in = aligned16(in), al_out = aligned16(out);

  // Phase 1: every rank gets my whole (wire-cast) input, my own arena included,
  // so that all ranks later add the same N values in the same order.
  for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
    const long long e0 = i * E;
    const int nv = valid_in_pack(e0, a.numel, E);
    Acc v[E];
    load_pack<T, E, Acc>(in + e0, v, nv, al_in);
    uint4 raw;
    {
      W* w = reinterpret_cast<W*>(&raw);
#pragma unroll
      for (int e = 0; e < E; ++e) w[e] = Elem<W>::down(static_cast<typename Elem<W>::Acc>(v[e]));
    }
#pragma unroll
    for (int k = 0; k < kMaxRanks; ++k) {
      if (k < N) {
        const int p = (rank + k) % N;
        *reinterpret_cast<uint4*>(c.arena[p] + base + static_cast<size_t>(rank) * slot_bytes + static_cast<size_t>(i) * 16) = raw;
      }
    }
  }
  if (barrier_all(c, vr, rank, s, PH_PUSH)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  // Phase 2: reduce the N slots in rank order.
  for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
    const long long e0 = i * E;
    const int nv = valid_in_pack(e0, a.numel, E);
    if (nv <= 0) continue;
    uint4 raw[kMaxRanks];
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src)
      if (src < N)
        raw[src] = *reinterpret_cast<const uint4*>(c.arena[rank] + base + static_cast<size_t>(src) * slot_bytes + static_cast<size_t>(i) * 16);
    Acc acc[E];
    {
      const W* w = reinterpret_cast<const W*>(&raw[0]);
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = static_cast<Acc>(Elem<W>::up(w[e]));
    }
#pragma unroll
    for (int src = 1; src < kMaxRanks; ++src) {
      if (src < N) {
        const W* w = reinterpret_cast<const W*>(&raw[src]);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = apply_op<Acc>(a.op, acc[e], static_cast<Acc>(Elem<W>::up(w[e])));
      }
    }
    if (a.op == OP_AVG) {
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = finish_avg<Acc>(acc[e], N, a.inv_world);
    }
    store_pack<T, E, Acc>(out + e0, acc, nv, al_out);
  }
  cta_end(c, vr, s, TL_ALLREDUCE);
}

// =================================================================== ring ==
template <typename T, typename W>
__global__ void __launch_bounds__(kThreads) ring_kernel(DevComm c, CollArgs a) {
  using PK = Pack<T, W>;
  constexpr int E = PK::kElems;
  using Acc = typename PK::Acc;
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const T* in = static_cast<const T*>(a.in[vr]);
  T* out = static_cast<T*>(a.out[vr]);
  const long long per = a.per;
  const size_t slot_bytes = static_cast<size_t>(per) * sizeof(W);
  const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
  auto rs_buf = [&](int r, int k) { return reinterpret_cast<W*>(c.arena[r] + base + static_cast<size_t>(k) * slot_bytes); };
  auto ag_buf = [&](int r, int k) { return reinterpret_cast<W*>(c.arena[r] + base + static_cast<size_t>(N - 1 + k) * slot_bytes); };
  const int next = (rank + 1) % N, prev = (rank + N - 1) % N;
  if (bounds_violation(c, vr, base + static_cast<size_t>(2 * (N - 1)) * slot_bytes)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  long long pb, pe;
  cta_span(per / E, pb, pe);
  auto chunk_limit = [&](int p) -> long long {
    long long lim = static_cast<long long>(p + 1) * per;
    return lim < a.numel ? lim : a.numel;
  };
  const uint32_t e0v = s.epoch;
  bool failed = false;

  // Reduce-scatter: N-1 steps.
  for (int k = 0; k < N - 1 && !failed; ++k) {
    const int sc = ((rank - k) % N + N) % N;
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      const long long el = static_cast<long long>(sc) * per + i * E;
      const int nv = valid_in_pack(el, chunk_limit(sc), E);
      Acc acc[E];
      load_pack<T, E, Acc>(in + el, acc, nv, aligned16(in + el));
      if (k > 0) {
        Acc v[E];
        load_pack<W, E, Acc>(rs_buf(rank, k - 1) + i * E, v, E, true);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = apply_op<Acc>(a.op, acc[e], v[e]);
      }
      store_pack<W, E, Acc>(rs_buf(next, k) + i * E, acc, E, true);
    }
    signal_one(c, rank, next, e0v + k + 1, s);
    failed = wait_one(c, vr, rank, prev, e0v + k + 1, PH_RING);
  }
  s.epoch = e0v + 2 * (N - 1);
  if (failed) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  // Finish the chunk this rank owns and start the allgather with it.
  const int fc = (rank + 1) % N;
  for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
    const long long el = static_cast<long long>(fc) * per + i * E;
    const int nv = valid_in_pack(el, chunk_limit(fc), E);
    Acc acc[E], v[E];
    load_pack<T, E, Acc>(in + el, acc, nv, aligned16(in + el));
    load_pack<W, E, Acc>(rs_buf(rank, N - 2) + i * E, v, E, true);
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = apply_op<Acc>(a.op, acc[e], v[e]);
    if (a.op == OP_AVG) {
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = finish_avg<Acc>(acc[e], N, a.inv_world);
    }
    round_through_wire<T, W, E, Acc>(acc);
    store_pack<W, E, Acc>(ag_buf(next, 0) + i * E, acc, E, true);
    if (nv > 0) store_pack<T, E, Acc>(out + el, acc, nv, aligned16(out + el));
  }
  // Allgather: N-1 steps, forwarding what arrives.
  for (int k = 0; k < N - 1 && !failed; ++k) {
    signal_one(c, rank, next, e0v + (N - 1) + k + 1, s);
    failed = wait_one(c, vr, rank, prev, e0v + (N - 1) + k + 1, PH_RING);
    if (failed) break;
    const int rc = ((rank - k) % N + N) % N;
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      const long long el = static_cast<long long>(rc) * per + i * E;
      const int nv = valid_in_pack(el, chunk_limit(rc), E);
      Acc v[E];
      load_pack<W, E, Acc>(ag_buf(rank, k) + i * E, v, E, true);
      if (k < N - 2) store_pack<W, E, Acc>(ag_buf(next, k + 1) + i * E, v, E, true);
      if (nv > 0) store_pack<T, E, Acc>(out + el, v, nv, aligned16(out + el));
    }
  }
  cta_end(c, vr, s, TL_ALLREDUCE);
}

// =================================================================== tree ==
template <typename T, typename W>
__global__ void __launch_bounds__(kThreads) tree_kernel(DevComm c, CollArgs a) {
  using PK = Pack<T, W>;
  constexpr int E = PK::kElems;
  using Acc = typename PK::Acc;
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const T* in = static_cast<const T*>(a.in[vr]);
  T* out = static_cast<T*>(a.out[vr]);
  const long long padded = (a.numel + 15) / 16 * 16;
  const size_t slot_bytes = static_cast<size_t>(padded) * sizeof(W);
  const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
  int R = 0;
  while ((1 << R) < N) ++R;
  auto tbuf = [&](int r, int j) { return reinterpret_cast<W*>(c.arena[r] + base + static_cast<size_t>(j) * slot_bytes); };
  auto bbuf = [&](int r) { return reinterpret_cast<W*>(c.arena[r] + base + static_cast<size_t>(R) * slot_bytes); };
  if (bounds_violation(c, vr, base + static_cast<size_t>(R + 1) * slot_bytes)) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  long long pb, pe;
  cta_span(padded / E, pb, pe);
  const bool al_in = aligned16(in), al_out = aligned16(out);
  const uint32_t e0v = s.epoch;
  s.epoch = e0v + R + 1;
  bool failed = false;

  // The running partial lives in `out`.
  if (out != in) {
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      const int nv = valid_in_pack(i * E, a.numel, E);
      if (nv <= 0) continue;
      Acc v[E];
      load_pack<T, E, Acc>(in + i * E, v, nv, al_in);
      store_pack<T, E, Acc>(out + i * E, v, nv, al_out);
    }
  }
  // Binomial reduce towards rank 0.
  for (int j = 0; j < R && !failed; ++j) {
    const int mask = 1 << j;
    if (rank & mask) {
      const int parent = rank - mask;
      for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
        const int nv = valid_in_pack(i * E, a.numel, E);
        Acc v[E];
        load_pack<T, E, Acc>(out + i * E, v, nv, al_out);
        store_pack<W, E, Acc>(tbuf(parent, j) + i * E, v, E, true);
      }
      signal_one(c, rank, parent, e0v + 1 + j, s);
      break;
    }
    if (rank + mask < N) {
      failed = wait_one(c, vr, rank, rank + mask, e0v + 1 + j, PH_TREE);
      if (failed) break;
      for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
        const int nv = valid_in_pack(i * E, a.numel, E);
        if (nv <= 0) continue;
        Acc acc[E], v[E];
        load_pack<T, E, Acc>(out + i * E, acc, nv, al_out);
        load_pack<W, E, Acc>(tbuf(rank, j) + i * E, v, E, true);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = apply_op<Acc>(a.op, acc[e], v[e]);
        store_pack<T, E, Acc>(out + i * E, acc, nv, al_out);
      }
      __syncthreads();
    }
  }
  if (failed) {
    cta_end(c, vr, s, TL_ALLREDUCE);
    return;
  }
  // Binomial broadcast from rank 0.
  int low = 1;
  if (rank == 0) {
    while (low < N) low <<= 1;
    // Root finalises: AVG scale, round through the wire type, keep a wire copy to forward.
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      const int nv = valid_in_pack(i * E, a.numel, E);
      Acc acc[E];
      load_pack<T, E, Acc>(out + i * E, acc, nv, al_out);
      if (a.op == OP_AVG) {
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = finish_avg<Acc>(acc[e], N, a.inv_world);
      }
      round_through_wire<T, W, E, Acc>(acc);
      store_pack<W, E, Acc>(bbuf(rank) + i * E, acc, E, true);
      if (nv > 0) store_pack<T, E, Acc>(out + i * E, acc, nv, al_out);
    }
  } else {
    while (!(rank & low)) low <<= 1;  // lowest set bit: parent = rank - low
    failed = wait_one(c, vr, rank, rank - low, e0v + R + 1, PH_TREE);
    if (failed) {
      cta_end(c, vr, s, TL_ALLREDUCE);
      return;
    }
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      const int nv = valid_in_pack(i * E, a.numel, E);
      if (nv <= 0) continue;
      Acc v[E];
      load_pack<W, E, Acc>(bbuf(rank) + i * E, v, E, true);
      store_pack<T, E, Acc>(out + i * E, v, nv, al_out);
    }
  }
  for (int mask = low >> 1; mask > 0; mask >>= 1) {
    const int child = rank + mask;
    if (child >= N) continue;
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x)
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(bbuf(child)) + static_cast<size_t>(i) * 16) =
          *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(bbuf(rank)) + static_cast<size_t>(i) * 16);
    signal_one(c, rank, child, e0v + R + 1, s);
  }
  cta_end(c, vr, s, TL_ALLREDUCE);
}

// =================================================================== NVLS ==
// In-switch reduction.  `local` is this rank's mapping of a symmetric buffer
// holding the (wire-typed) input, `mc` the multicast mapping of the same
// buffer; the reduced values are written back through the multicast mapping,
// so afterwards every rank's copy holds the result.  When kStage is set the
// kernel first copies `in` into the arena and afterwards copies the result to
// `out`; otherwise the caller's buffer already lives in symmetric memory.
template <typename W> struct Multimem;
template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

template <typename T, typename W, bool kStage>
__global__ void __launch_bounds__(kThreads) nvls_kernel(DevComm c, CollArgs a, char* local_sym, char* mc_sym) {
  using PK = Pack<T, W>;
  constexpr int E = PK::kElems;
  using Acc = typename PK::Acc;
  constexpr int WE = 16 / sizeof(W);  // wire elements per 16 bytes
  const int rank = c.rank_base, N = c.world;
  CtaSync s = cta_begin(c, 0);
  const long long per = a.per;
  long long pb, pe;
  char* stage_local;
  char* stage_mc;
  char* result_local;
  char* result_mc;
  if constexpr (kStage) {
    const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
    const size_t region = static_cast<size_t>(N) * per * sizeof(W);
    if (bounds_violation(c, 0, base + 2 * region)) {
      cta_end(c, 0, s, TL_ALLREDUCE);
      return;
    }
    stage_local = c.arena[rank] + base;
    stage_mc = c.mc_arena + base;
    result_local = stage_local + region;
    result_mc = stage_mc + region;
    // Phase 0: wire-cast copy of the whole input into my arena.  The work is
    // split per chunk so that CTA b stages exactly the part of every chunk
    // that CTA b of the chunk's owner will reduce.
    const T* in = static_cast<const T*>(a.in[0]);
    cta_span(per / E, pb, pe);
    for (int p = 0; p < N; ++p) {
      for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
        const long long el = static_cast<long long>(p) * per + i * E;
        const int nv = valid_in_pack(el, a.numel, E);
        Acc v[E];
        load_pack<T, E, Acc>(in + el, v, nv, aligned16(in + el));
        store_pack<W, E, Acc>(reinterpret_cast<W*>(stage_local) + el, v, E, true);
      }
    }
  } else {
    stage_local = result_local = local_sym;
    stage_mc = result_mc = mc_sym;
  }
  if (barrier_all(c, 0, rank, s, PH_NVLS)) {
    cta_end(c, 0, s, TL_ALLREDUCE);
    return;
  }
  // Phase 1: reduce chunk `rank` in the switch and broadcast it back.
  cta_span(per / WE, pb, pe);
  const size_t chunk_byte0 = static_cast<size_t>(rank) * per * sizeof(W);
  constexpr int NU = 4;  // in-switch reductions in flight per thread
  for (long long i0 = pb + threadIdx.x; i0 < pe; i0 += static_cast<long long>(blockDim.x) * NU) {
    uint4 v[NU];
#pragma unroll
    for (int u = 0; u < NU; ++u) {
      const long long i = i0 + static_cast<long long>(u) * blockDim.x;
      if (i < pe) v[u] = Multimem<W>::ld_reduce(stage_mc + chunk_byte0 + static_cast<size_t>(i) * 16);
    }
#pragma unroll
    for (int u = 0; u < NU; ++u) {
      const long long i = i0 + static_cast<long long>(u) * blockDim.x;
      if (i >= pe) continue;
      if (a.op == OP_AVG) {
        W* w = reinterpret_cast<W*>(&v[u]);
#pragma unroll
        for (int e = 0; e < WE; ++e) w[e] = Elem<W>::down(Elem<W>::up(w[e]) * a.inv_world);
      }
      multimem_st16(result_mc + chunk_byte0 + static_cast<size_t>(i) * 16, v[u]);
    }
  }
  if (barrier_all(c, 0, rank, s, PH_NVLS)) {
    cta_end(c, 0, s, TL_ALLREDUCE);
    return;
  }
  if constexpr (kStage) {
    // Phase 2: copy the result out of my arena (same per-chunk split).
    T* out = static_cast<T*>(a.out[0]);
    cta_span(per / E, pb, pe);
    for (int p = 0; p < N; ++p) {
      for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
        const long long el = static_cast<long long>(p) * per + i * E;
        const int nv = valid_in_pack(el, a.numel, E);
        if (nv <= 0) continue;
        Acc v[E];
        load_pack<W, E, Acc>(reinterpret_cast<const W*>(result_local) + el, v, E, true);
        store_pack<T, E, Acc>(out + el, v, nv, aligned16(out + el));
      }
    }
  }
  cta_end(c, 0, s, TL_ALLREDUCE);
}

// ====================================================== symmetric in-place ==
// Allreduce of a buffer that every rank allocated in the symmetric heap, so
// peers' copies are directly addressable: a.in[r] is rank r's copy as mapped
// here.  No staging: rank r reads chunk r of every copy, reduces, writes its
// own copy, and after a meeting everyone pulls the other chunks.  A third
// meeting keeps a fast rank from overwriting its copy while peers still read it.
template <typename T>
__global__ void __launch_bounds__(kThreads) symm_allreduce_kernel(DevComm c, CollArgs a) {
  using Acc = typename Elem<T>::Acc;
  constexpr int E = 16 / sizeof(T);
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const long long per = a.per;
  long long pb, pe;
  cta_span(per / E, pb, pe);
  T* mine = static_cast<T*>(const_cast<void*>(a.in[rank]));
  bool failed = barrier_all(c, vr, rank, s, PH_PUSH);
  if (!failed) {
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      const long long el = static_cast<long long>(rank) * per + i * E;
      const int nv = valid_in_pack(el, a.numel, E);
      if (nv <= 0) continue;
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int src = 0; src < kMaxRanks; ++src)
        if (src < N) raw[src] = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.in[src]) + el);
      Acc acc[E];
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = static_cast<Acc>(Elem<T>::up(reinterpret_cast<const T*>(&raw[0])[e]));
#pragma unroll
      for (int src = 1; src < kMaxRanks; ++src) {
        if (src < N) {
#pragma unroll
          for (int e = 0; e < E; ++e)
            acc[e] = apply_op<Acc>(a.op, acc[e], static_cast<Acc>(Elem<T>::up(reinterpret_cast<const T*>(&raw[src])[e])));
        }
      }
      if (a.op == OP_AVG) {
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = finish_avg<Acc>(acc[e], N, a.inv_world);
      }
      store_pack<T, E, Acc>(mine + el, acc, E, true);
    }
    failed = barrier_all(c, vr, rank, s, PH_REDUCE);
  }
  if (!failed) {
    for (long long i = pb + threadIdx.x; i < pe; i += blockDim.x) {
      uint4 raw[kMaxRanks - 1];
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k) {
        if (k < N) {
          const int p = (rank + k) % N;
          raw[k - 1] = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.in[p]) + static_cast<long long>(p) * per + i * E);
        }
      }
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k) {
        if (k < N) {
          const int p = (rank + k) % N;
          *reinterpret_cast<uint4*>(mine + static_cast<long long>(p) * per + i * E) = raw[k - 1];
        }
      }
    }
    barrier_all(c, vr, rank, s, PH_GATHER);
  }
  cta_end(c, vr, s, TL_ALLREDUCE);
}

// ============================================================== allgather ==
// Bytes, any alignment.  Every rank pushes its block into slot `rank` of every peer's arena (posted stores to
// all peers at once), the ranks meet, and each one unpacks the N - 1 foreign slots from its own arena.
__global__ void __launch_bounds__(kThreads) allgather_kernel(DevComm c, CollArgs a) {
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const unsigned long long nbytes = static_cast<unsigned long long>(a.numel);
  const unsigned long long stride = static_cast<unsigned long long>(a.stride);
  const unsigned long long slot = (nbytes + 15) / 16 * 16;
  const char* in = static_cast<const char*>(a.in[vr]);
  char* out = static_cast<char*>(a.out[vr]);
  const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
  if (bounds_violation(c, vr, base + static_cast<size_t>(N) * slot)) {
    cta_end(c, vr, s);
    return;
  }
  unsigned long long b0, b1;
  cta_byte_span(nbytes, b0, b1);
  if (a.reserved != 0 && c.mc_arena != nullptr && aligned16(in)) {
    // In-switch replication: one store through the multicast mapping lands in slot `rank` of every arena, so this
    // GPU's links carry the block once instead of N - 1 times.
    char* mc = c.mc_arena + base + static_cast<size_t>(rank) * slot;
    const unsigned long long v0 = b0 / 16, v1 = (b1 - b0) / 16 + v0;
    constexpr int U = 4;
    for (unsigned long long i0 = v0 + threadIdx.x; i0 < v1; i0 += static_cast<unsigned long long>(blockDim.x) * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + static_cast<unsigned long long>(u) * blockDim.x;
        if (i < v1) v[u] = reinterpret_cast<const uint4*>(in)[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned long long i = i0 + static_cast<unsigned long long>(u) * blockDim.x;
        if (i < v1) multimem_st16(mc + i * 16, v[u]);
      }
    }
    // ragged tail of the block (fewer than 16 bytes): plain stores to every peer
    const unsigned long long tail0 = v1 * 16;
    if (tail0 < b1) {
      for (int k = 1; k < N; ++k) {
        const int p = (rank + k) % N;
        cta_copy_bytes(c.arena[p] + base + static_cast<size_t>(rank) * slot + tail0, in + tail0, b1 - tail0);
      }
    }
  } else {
    char* dsts[kMaxRanks];
    int nd = 0;
    for (int k = 1; k < N; ++k) {
      const int p = (rank + k) % N;
      dsts[nd++] = c.arena[p] + base + static_cast<size_t>(rank) * slot + b0;
    }
    cta_push_bytes(dsts, nd, in + b0, b1 - b0);
  }
  if (out + static_cast<size_t>(rank) * stride != in) cta_copy_bytes(out + static_cast<size_t>(rank) * stride + b0, in + b0, b1 - b0);
  if (barrier_all(c, vr, rank, s, PH_GATHER)) {
    cta_end(c, vr, s);
    return;
  }
  for (int k = 1; k < N; ++k) {
    const int p = (rank + k) % N;
    cta_copy_bytes(out + static_cast<size_t>(p) * stride + b0, c.arena[rank] + base + static_cast<size_t>(p) * slot + b0, b1 - b0);
  }
  cta_end(c, vr, s);
}

// ============================================================== broadcast ==
// Scatter + allgather: the root pushes slice p of its buffer into rank p's
// arena, then every rank pulls the other slices from their holders, so the
// root's links carry the message once instead of N-1 times.
__global__ void __launch_bounds__(kThreads) broadcast_kernel(DevComm c, CollArgs a) {
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world, root = a.root;
  CtaSync s = cta_begin(c, vr);
  const unsigned long long nbytes = static_cast<unsigned long long>(a.numel);
  char* data = static_cast<char*>(a.out[vr]);
  const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
  const unsigned long long slice = (nbytes + N - 1) / N;
  const unsigned long long slice16 = (slice + 15) / 16 * 16;  // slices start on 16-byte boundaries
  auto slice_len = [&](int p) -> unsigned long long {
    unsigned long long lo = p * slice16;
    if (lo >= nbytes) return 0ull;
    unsigned long long hi = lo + slice16;
    return (hi < nbytes ? hi : nbytes) - lo;
  };
  if (bounds_violation(c, vr, base + slice16)) {
    cta_end(c, vr, s);
    return;
  }
  if (rank == root) {
    for (int k = 0; k < N; ++k) {
      const int p = (rank + k) % N;
      unsigned long long b0, b1;
      cta_byte_span(slice_len(p), b0, b1);
      cta_copy_bytes(c.arena[p] + base + b0, data + p * slice16 + b0, b1 - b0);
    }
  }
  if (barrier_all(c, vr, rank, s, PH_GATHER)) {
    cta_end(c, vr, s);
    return;
  }
  if (rank != root) {
    for (int k = 0; k < N; ++k) {
      const int p = (rank + k) % N;
      unsigned long long b0, b1;
      cta_byte_span(slice_len(p), b0, b1);
      cta_copy_bytes(data + p * slice16 + b0, c.arena[p] + base + b0, b1 - b0);
    }
  }
  cta_end(c, vr, s);
}

// =============================================================== alltoall ==
// P2P dispatch: rank r pushes the segment meant for rank q straight into slot r of q's arena (posted stores); after
// the meeting every rank unpacks its N - 1 slots into its output at the senders' offsets.  Segment sizes may differ
// per pair, and a rank only knows its own, so the number of rounds (a round moves at most slot_bytes per pair) is
// agreed on the device: every CTA first tells every peer its rank's longest segment through a word behind the
// slots, and all take the largest.  Segments of any length therefore go through one launch.
__global__ void __launch_bounds__(kThreads) alltoall_kernel(DevComm c, A2AArgs a) {
  const int vr = blockIdx.y, rank = c.rank_base + vr, N = c.world;
  CtaSync s = cta_begin(c, vr);
  const char* in = static_cast<const char*>(a.in[vr]);
  char* out = static_cast<char*>(a.out[vr]);
  const size_t base = static_cast<size_t>(s.half) * c.half_bytes;
  const unsigned long long slot = a.slot_bytes;
  // control words: [cta][source rank] behind the N data slots of this half
  const size_t ctl_off = base + static_cast<size_t>(N) * slot;
  if (bounds_violation(c, vr, ctl_off + static_cast<size_t>(gridDim.x) * kMaxRanks * sizeof(unsigned long long))) {
    cta_end(c, vr, s);
    return;
  }
  unsigned long long longest = 0;
  for (int q = 0; q < N; ++q) {
    longest = a.in_len[vr][q] > longest ? a.in_len[vr][q] : longest;
    longest = a.out_len[vr][q] > longest ? a.out_len[vr][q] : longest;
  }
  if (threadIdx.x < N)
    reinterpret_cast<unsigned long long*>(c.arena[threadIdx.x] + ctl_off)[blockIdx.x * kMaxRanks + rank] = longest;
  if (barrier_all(c, vr, rank, s, PH_GATHER)) {
    cta_end(c, vr, s);
    return;
  }
  for (int q = 0; q < N; ++q) {
    const unsigned long long v = reinterpret_cast<const unsigned long long*>(c.arena[rank] + ctl_off)[blockIdx.x * kMaxRanks + q];
    longest = v > longest ? v : longest;
  }
  const unsigned long long rounds = longest == 0 ? 0 : (longest + slot - 1) / slot;
  for (unsigned long long r = 0; r < rounds; ++r) {
    const unsigned long long lo = r * slot;
    for (int k = 0; k < N; ++k) {
      const int q = (rank + k) % N;
      const unsigned long long len = a.in_len[vr][q] > lo ? (a.in_len[vr][q] - lo < slot ? a.in_len[vr][q] - lo : slot) : 0;
      // The slot is cut among the CTAs once per pair, whatever the round's length: a byte of the slot then belongs to
      // the same CTA index in every round, and the per-CTA meetings below are all the ordering a slot byte needs.
      // A segment shorter than the slot has one round and is cut by its own length, so that every CTA moves a share
      // (both sides know the length: what this rank sends to q is what q receives from this rank).
      unsigned long long b0, b1;
      cta_byte_span(a.in_len[vr][q] < slot ? a.in_len[vr][q] : slot, b0, b1);
      b0 = b0 < len ? b0 : len;
      b1 = b1 < len ? b1 : len;
      if (q == rank)
        cta_copy_bytes(out + a.out_off[vr][q] + lo + b0, in + a.in_off[vr][q] + lo + b0, b1 - b0);
      else
        cta_copy_bytes(c.arena[q] + base + static_cast<size_t>(rank) * slot + b0, in + a.in_off[vr][q] + lo + b0, b1 - b0);
    }
    if (barrier_all(c, vr, rank, s, PH_GATHER)) break;
    for (int k = 1; k < N; ++k) {
      const int p = (rank + k) % N;
      const unsigned long long len = a.out_len[vr][p] > lo ? (a.out_len[vr][p] - lo < slot ? a.out_len[vr][p] - lo : slot) : 0;
      unsigned long long b0, b1;
      cta_byte_span(a.out_len[vr][p] < slot ? a.out_len[vr][p] : slot, b0, b1);
      b0 = b0 < len ? b0 : len;
      b1 = b1 < len ? b1 : len;
      cta_copy_bytes_uncached(out + a.out_off[vr][p] + lo + b0, c.arena[rank] + base + static_cast<size_t>(p) * slot + b0, b1 - b0);
    }
    // the slots are overwritten in the next round: everybody must have unpacked first
    if (r + 1 < rounds && barrier_all(c, vr, rank, s, PH_GATHER)) break;
  }
  cta_end(c, vr, s);
}

// ============================================================= send / recv ==
// One launch moves one message between a pair of ranks: blockIdx.y selects the virtual rank
// (single-GPU emulation runs a sender and a receiver as one cooperative launch), each CTA moves
// its own byte range of every chunk and talks only to the CTA of the same index on the other side.
__global__ void __launch_bounds__(kThreads) p2p_kernel(P2PComm c, P2PArgs a) {
  const int vr = blockIdx.y, rank = c.rank_base + vr, peer = a.peer[vr];
  if (peer < 0) return;
  const bool sending = a.is_send[vr] != 0;
  P2PState* st = c.state[vr];
  const uint32_t base = sending ? st->send_seq[peer] : st->recv_seq[peer];
  const unsigned long long slot = c.slot_bytes;
  const unsigned long long chunks = (a.nbytes + slot - 1) / slot;
  char* user = static_cast<char*>(a.buf[vr]);
  bool failed = false;
  auto wait_flag = [&](const uint32_t* flag, uint32_t value, int phase) -> bool {
    bool bad = false;
    if (threadIdx.x == 0) {
      const unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      for (;;) {
        if (static_cast<int32_t>(ld_acquire_sys(flag) - value) >= 0) break;
        if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > c.timeout_ns) {
          volatile int* sw = c.status[vr];
          if (*sw == 0) *sw = encode_status(phase, peer);
          __threadfence_system();
          bad = true;
          break;
        }
      }
    }
    return __syncthreads_or(bad ? 1 : 0) != 0;
  };
  for (unsigned long long k = 0; k < chunks && !failed; ++k) {
    const uint32_t seq = base + static_cast<uint32_t>(k) + 1u;
    const unsigned long long off = k * slot;
    const unsigned long long len = a.nbytes - off < slot ? a.nbytes - off : slot;
    // fixed partition of the slot among the CTAs (clipped to this chunk): a slot byte has one owner in every chunk
    unsigned long long b0, b1;
    cta_byte_span(slot, b0, b1);
    b0 = b0 < len ? b0 : len;
    b1 = b1 < len ? b1 : len;
    if (sending) {
      // buffer seq & 1 last held chunk seq - 2: the receiver must have copied that one out
      failed = wait_flag(c.free_[rank] + blockIdx.x * kMaxRanks + peer, seq - 2u, PH_SEND);
      if (failed) break;
      char* dst = c.region[peer] + (static_cast<size_t>(rank) * 2 + (seq & 1u)) * slot;
      cta_copy_bytes(dst + b0, user + off + b0, b1 - b0);
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        st_release_sys(c.ready[peer] + blockIdx.x * kMaxRanks + rank, seq);
      }
    } else {
      failed = wait_flag(c.ready[rank] + blockIdx.x * kMaxRanks + peer, seq, PH_RECV);
      if (failed) break;
      const char* src = c.region[rank] + (static_cast<size_t>(peer) * 2 + (seq & 1u)) * slot;
      cta_copy_bytes_uncached(user + off + b0, src + b0, b1 - b0);   // the two buffers are reused chunk after chunk
      __syncthreads();
      if (threadIdx.x == 0) st_release_sys(c.free_[peer] + blockIdx.x * kMaxRanks + rank, seq);
    }
  }
  // The last CTA to finish advances the pair's sequence number (also after a timeout, so that both
  // sides keep counting the same messages).
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = sending ? &st->send_done[peer] : &st->recv_done[peer];
    __threadfence();
    if (atomicAdd(done, 1u) + 1u == gridDim.x) {
      *done = 0;
      if (sending) st->send_seq[peer] = base + static_cast<uint32_t>(chunks);
      else st->recv_seq[peer] = base + static_cast<uint32_t>(chunks);
      __threadfence();
    }
  }
}

// ================================================================ barrier ==
__global__ void __launch_bounds__(32) barrier_kernel(DevComm c) {
  const int vr = blockIdx.y, rank = c.rank_base + vr;
  CtaSync s = cta_begin(c, vr);
  barrier_all(c, vr, rank, s, PH_BARRIER);
  cta_end(c, vr, s);
}

// ============================================================== launchers ==
namespace {

template <typename... KArgs, typename... Args>
cudaError_t launch(const char* name, void (*kernel)(KArgs...), const LaunchCfg& cfg, int threads, Args... args) {
  // Threads per CTA: cfg.threads when the caller chose (128..512), else MCCL_COMM_THREADS, else 256.  A
  // 256-thread collective CTA needs half a register file, so it can share an SM with a persistent GEMM CTA; a
  // 512-thread CTA needs a whole one and therefore only lands on an SM no GEMM CTA occupies, which is what a
  // trainer wants when it keeps a few SMs free of GEMM work for the gradient collectives.
  static const int env_threads = [] {
    const char* v = std::getenv("MCCL_COMM_THREADS");
    const int t = v && *v ? std::atoi(v) : 256;
    return t >= 128 && t <= kThreads ? (t / 32) * 32 : 256;
  }();
  if (threads == kThreads) {
    const int want = cfg.threads > 0 ? cfg.threads : env_threads;
    threads = want >= 128 && want <= kThreads ? (want / 32) * 32 : 256;
  }
  dim3 grid(cfg.ctas, cfg.nlocal > 1 ? cfg.nlocal : 1);
  if (cfg.nlocal > 1) {
    void* params[] = {static_cast<void*>(&args)...};
    cudaError_t rc = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, dim3(threads), params, 0, cfg.stream);
    const cudaError_t seen = launch_record(name, __FILE__, __LINE__, grid, dim3(threads), 0, cfg.stream);
    return rc != cudaSuccess ? rc : seen;
  }
  kernel<<<grid, threads, 0, cfg.stream>>>(args...);   // the one launch statement of this file: every collective goes through here
  return launch_record(name, __FILE__, __LINE__, grid, dim3(threads), 0, cfg.stream);
}

enum class Sched { TWOSHOT, TWOSHOT_PUSH, SCATTER, ONESHOT, RING, TREE };

template <typename T, typename W>
cudaError_t launch_typed(Sched k, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  switch (k) {
    case Sched::TWOSHOT: return launch("twoshot_kernel", twoshot_kernel<T, W, false>, cfg, kThreads, c, a);
    case Sched::TWOSHOT_PUSH: return launch("twoshot_push_kernel", twoshot_push_kernel<T, W>, cfg, kThreads, c, a);
    case Sched::SCATTER: return launch("twoshot_kernel", twoshot_kernel<T, W, true>, cfg, kThreads, c, a);
    case Sched::ONESHOT: return launch("oneshot_kernel", oneshot_kernel<T, W>, cfg, kThreads, c, a);
    case Sched::RING: return launch("ring_kernel", ring_kernel<T, W>, cfg, kThreads, c, a);
    case Sched::TREE: return launch("tree_kernel", tree_kernel<T, W>, cfg, kThreads, c, a);
  }
  return cudaErrorInvalidValue;
}

cudaError_t dispatch(Sched k, ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  switch (t) {
    case ElemType::F32:
      return bf16_wire ? launch_typed<float, __nv_bfloat16>(k, c, a, cfg) : launch_typed<float, float>(k, c, a, cfg);
    case ElemType::F16: return launch_typed<__half, __half>(k, c, a, cfg);
    case ElemType::BF16: return launch_typed<__nv_bfloat16, __nv_bfloat16>(k, c, a, cfg);
    case ElemType::F64: return launch_typed<double, double>(k, c, a, cfg);
    case ElemType::I32: return launch_typed<int32_t, int32_t>(k, c, a, cfg);
    case ElemType::I64: return launch_typed<int64_t, int64_t>(k, c, a, cfg);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_allreduce_twoshot(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return dispatch(Sched::TWOSHOT, t, bf16_wire, c, a, cfg);
}
cudaError_t launch_allreduce_twoshot_push(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return dispatch(Sched::TWOSHOT_PUSH, t, bf16_wire, c, a, cfg);
}
cudaError_t launch_reduce_scatter(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return dispatch(Sched::SCATTER, t, bf16_wire, c, a, cfg);
}
cudaError_t launch_allreduce_oneshot(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return dispatch(Sched::ONESHOT, t, bf16_wire, c, a, cfg);
}
cudaError_t launch_allreduce_ring(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return dispatch(Sched::RING, t, bf16_wire, c, a, cfg);
}
cudaError_t launch_allreduce_tree(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return dispatch(Sched::TREE, t, bf16_wire, c, a, cfg);
}

cudaError_t launch_allreduce_nvls(ElemType t, bool bf16_wire, bool staged, const DevComm& c, const CollArgs& a,
                                  char* local_sym, char* mc_sym, const LaunchCfg& cfg) {
  if (cfg.nlocal > 1) return cudaErrorNotSupported;  // no multicast object inside one GPU
#define MCCL_NVLS(T, W)                                                                       \
  (staged ? launch("nvls_kernel", nvls_kernel<T, W, true>, cfg, kThreads, c, a, local_sym, mc_sym)           \
          : launch("nvls_kernel", nvls_kernel<T, W, false>, cfg, kThreads, c, a, local_sym, mc_sym))
  switch (t) {
    case ElemType::F32: return bf16_wire ? MCCL_NVLS(float, __nv_bfloat16) : MCCL_NVLS(float, float);
    case ElemType::F16: return MCCL_NVLS(__half, __half);
    case ElemType::BF16: return MCCL_NVLS(__nv_bfloat16, __nv_bfloat16);
    default: return cudaErrorNotSupported;
  }
#undef MCCL_NVLS
}

cudaError_t launch_allreduce_symm(ElemType t, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  switch (t) {
    case ElemType::F32: return launch("symm_allreduce_kernel", symm_allreduce_kernel<float>, cfg, kThreads, c, a);
    case ElemType::F16: return launch("symm_allreduce_kernel", symm_allreduce_kernel<__half>, cfg, kThreads, c, a);
    case ElemType::BF16: return launch("symm_allreduce_kernel", symm_allreduce_kernel<__nv_bfloat16>, cfg, kThreads, c, a);
    case ElemType::F64: return launch("symm_allreduce_kernel", symm_allreduce_kernel<double>, cfg, kThreads, c, a);
    case ElemType::I32: return launch("symm_allreduce_kernel", symm_allreduce_kernel<int32_t>, cfg, kThreads, c, a);
    case ElemType::I64: return launch("symm_allreduce_kernel", symm_allreduce_kernel<int64_t>, cfg, kThreads, c, a);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_allgather(const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return launch("allgather_kernel", allgather_kernel, cfg, kThreads, c, a);
}
cudaError_t launch_broadcast(const DevComm& c, const CollArgs& a, const LaunchCfg& cfg) {
  return launch("broadcast_kernel", broadcast_kernel, cfg, kThreads, c, a);
}
cudaError_t launch_alltoall(const DevComm& c, const A2AArgs& a, const LaunchCfg& cfg) {
  return launch("alltoall_kernel", alltoall_kernel, cfg, kThreads, c, a);
}
cudaError_t launch_p2p(const P2PComm& c, const P2PArgs& a, const LaunchCfg& cfg) {
  return launch("p2p_kernel", p2p_kernel, cfg, kThreads, c, a);
}
cudaError_t launch_barrier(const DevComm& c, const LaunchCfg& cfg) {
  LaunchCfg one = cfg;
  one.ctas = 1;
  return launch("barrier_kernel", barrier_kernel, one, 32, c);
}

}  // namespace dev
}  // namespace mccl
