// Persistent bf16 GEMM for sm_100a: one CTA per SM walks a list of 128 x BN
// output tiles.  The accumulator is double-buffered in tensor memory, so the
// epilogue of tile i (tcgen05.ld, bias / activation, stores) runs while the
// tensor cores already work on tile i+1, and the barrier / TMEM set-up cost is
// paid once per SM instead of once per tile.
//
//   warp 0      TMA producer (one thread): A / B k-blocks into a ring of stages
//   warp 1      TMEM owner and tcgen05.mma issuer (one thread)
//   warps 2-9   epilogue: two warps per TMEM lane quarter, each finishing half of the tile's columns
//
// The same kernel carries the tensor-parallel fusions (see tp_gemm.cu):
//   all-gather → GEMM   the A operand arrives in row chunks; the producer waits
//                       for a chunk's flag before it loads tiles of that chunk
//   GEMM → reduce-scatter  output row chunks belong to different ranks; the
//                       epilogue stores each tile into its owner's staging slot
// Tiles are visited chunk by chunk starting with this rank's own chunk, so
// compute on data that is already local overlaps the NVLink transfers.
#include "../core/launch.hpp"
#include "gemm_common.cuh"
#include "gemm_persistent.cuh"

#include <atomic>
#include <cstdlib>

namespace mccl {
namespace ops {

namespace {

template <int BN, int STAGES>
struct PLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTiles = STAGES * kStageBytes;
  static constexpr int kGemmBarriers = (2 * STAGES + 4) * 8 + 16;
  static constexpr int kReduceBarriers = 64;             // the reduce-scatter reducers' barriers and ring
  static constexpr int kSchedBytes = 4 * 8 * 2 + 4 * 4;  // tile scheduler: full / empty barriers and tile ring
  static constexpr int kBarriers = kGemmBarriers + kReduceBarriers + kSchedBytes;
  // behind the barriers: one 4 KB staging buffer per epilogue warp (output rows are transposed through it so that
  // global stores cover whole 128-byte lines)
  static constexpr int kStagingOff = kTiles + 512;
  static constexpr int kStagingPerWarp = 4096;
  static constexpr int kTotal = kStagingOff + 8 * kStagingPerWarp + 1024;
  static_assert(kBarriers <= 512, "barriers overlap the epilogue staging");
  static_assert(kTotal <= 227 * 1024, "shared memory of one CTA");
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait that also gives up when another role of this CTA has failed.  The limit is a
// time (the fused roles legitimately wait for other GPUs), read only once the fast path missed.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned long long limit_ns) {
  for (int i = 0; i < 64; ++i)
    if (tc::mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  for (uint32_t i = 0;; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u) {
      if (*abort_flag) return false;
      if (now_ns() - t0 > limit_ns) return false;
    }
  }
}

// Spin on a flag word in global memory written by another CTA of this GPU (chunk
// arrival in the all-gather fusion).  Bounded; false on timeout.
__device__ __forceinline__ bool wait_flag_geq(const uint32_t* flag, uint32_t value, volatile int* abort_flag, unsigned long long limit_ns) {
  const unsigned long long t0 = now_ns();
  for (uint32_t i = 0;; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - value) >= 0) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
      if (now_ns() - t0 > limit_ns) return false;
    }
    __nanosleep(64);
  }
}


// ---- cross-GPU signalling for the fused roles (bounded waits, status word on timeout) ----
__device__ __forceinline__ void sig_store(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool sig_wait(const uint32_t* p, uint32_t v, unsigned long long timeout_ns) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned spins = 0;; ++spins) {
    uint32_t cur;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(cur) : "l"(p) : "memory");
    if (static_cast<int32_t>(cur - v) >= 0) return true;
    if ((spins & 63u) == 63u) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > timeout_ns) return false;
    }
  }
}
// Meeting of copy CTA `cta` of every rank.  Returns false when a peer did not arrive in time.
__device__ __forceinline__ bool copy_cta_meet(const FusedDev& f, int cta, uint32_t value) {
  __syncthreads();
  bool bad = false;
  const int t = threadIdx.x;
  if (t < f.world) {
    __threadfence_system();
    sig_store(f.sig[t] + kFuseSigAg + 8 * cta + f.rank, value);
    bad = !sig_wait(f.sig[f.rank] + kFuseSigAg + 8 * cta + t, value, f.timeout_ns);
    if (bad) atomicCAS(f.status, 0, 0x100 + t);
  }
  return __syncthreads_or(bad ? 1 : 0) == 0;
}
// Bulk (TMA, untiled, no multicast) copy engine of a copy CTA: one thread streams [b0, b1) of
// `src` (possibly a peer's memory) to `dst` (local) through `stages` shared-memory buffers of
// `piece` bytes, so that (stages - 1) * piece bytes are in flight per CTA with a single thread
// issuing.  Addresses and sizes are multiples of 16 bytes.  Returns false when a load never landed.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(tc::smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(tc::smem_u32(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
constexpr int kCopyStages = 4;
constexpr uint32_t kCopyPiece = 48 * 1024;

struct CopyEngine {
  uint8_t* buf;       // kCopyStages * kCopyPiece bytes of shared memory, 128-byte aligned
  uint64_t* full;     // kCopyStages barriers
  uint32_t issued;    // loads issued so far (all chunks)
  uint32_t drained;   // pieces stored so far
};

// Streams one byte range and returns when its last piece has been handed to a store.
__device__ bool copy_range(CopyEngine& e, char* dst, const char* src, unsigned long long b0, unsigned long long b1,
                           unsigned long long limit_ns) {
  const unsigned long long total = b1 - b0;
  const uint32_t pieces = static_cast<uint32_t>((total + kCopyPiece - 1) / kCopyPiece);
  uint32_t loaded = 0;
  auto issue = [&](uint32_t j) {
    const unsigned long long off = static_cast<unsigned long long>(j) * kCopyPiece;
    const uint32_t n = static_cast<uint32_t>(total - off < kCopyPiece ? total - off : kCopyPiece);
    const uint32_t s = e.issued % kCopyStages;
    tc::mbar_expect_tx(&e.full[s], n);
    bulk_load(e.buf + static_cast<size_t>(s) * kCopyPiece, src + b0 + off, n, &e.full[s]);
    ++e.issued;
  };
  // a stage may be refilled once the store that read it has finished reading: keep one stage for that
  while (loaded < pieces && e.issued - e.drained < kCopyStages - 1) issue(loaded++);
  for (uint32_t j = 0; j < pieces; ++j) {
    const uint32_t s = e.drained % kCopyStages;
    const unsigned long long t0 = now_ns();
    while (!tc::mbar_try_wait(&e.full[s], (e.drained / kCopyStages) & 1u))
      if (now_ns() - t0 > limit_ns) return false;
    const unsigned long long off = static_cast<unsigned long long>(j) * kCopyPiece;
    const uint32_t n = static_cast<uint32_t>(total - off < kCopyPiece ? total - off : kCopyPiece);
    bulk_store(dst + b0 + off, e.buf + static_cast<size_t>(s) * kCopyPiece, n);
    ++e.drained;
    if (loaded < pieces) {
      // the stage to refill is the one stored in the previous iteration: wait until at most the newest
      // store is still reading shared memory
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue(loaded++);
    }
  }
  return true;
}

// Role of CTAs [0, copy_ctas) in the all-gather fusion: meet the peers (their shards are
// complete), pull the shards chunk by chunk starting with the own one, raise a chunk's flag
// when every copy CTA has finished it, meet again (nobody reads my shard any more).
__device__ void allgather_copy_role(const FusedDev& f, uint32_t epoch, uint8_t* smem) {
  const int cta = blockIdx.x;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kCopyStages * kCopyPiece);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kCopyStages; ++s) tc::mbar_init(&full[s], 1);
    tc::mbar_init_fence();
  }
  if (!copy_cta_meet(f, cta, 2 * epoch - 1)) return;
  const unsigned long long units = f.chunk_bytes / 16;
  const unsigned long long per = (units + f.copy_ctas - 1) / f.copy_ctas;
  unsigned long long b0 = cta * per * 16, b1 = b0 + per * 16;
  if (b0 > f.chunk_bytes) b0 = f.chunk_bytes;
  if (b1 > f.chunk_bytes) b1 = f.chunk_bytes;
  if (threadIdx.x == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");   // the shards were written with ordinary stores
    CopyEngine e{smem, full, 0u, 0u};
    bool ok = true;
    for (int k = 0; k < f.world && ok; ++k) {
      const int c = (f.rank + k) % f.world;
      if (b1 > b0)
        ok = copy_range(e, static_cast<char*>(f.a_gathered) + static_cast<size_t>(c) * f.chunk_bytes,
                        static_cast<const char*>(f.a_peer[c]), b0, b1, f.timeout_ns);
      if (!ok) break;
      // the chunk's bytes must be in global memory before its flag can rise
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      const uint32_t arrived = atomicAdd(f.chunk_counters + c, 1u) + 1u;
      if (arrived == static_cast<uint32_t>(f.copy_ctas) * epoch)
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(f.chunk_flags + c), "r"(epoch) : "memory");
    }
    if (!ok) {
      atomicCAS(f.status, 0, 0x100 + f.rank);
      // queued stores must have read shared memory, and loads in flight must land, before the CTA retires
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      for (uint32_t j = e.drained; j < e.issued; ++j) tc::mbar_wait(&full[j % kCopyStages], (j / kCopyStages) & 1u, 1u << 22);
    }
  }
  copy_cta_meet(f, cta, 2 * epoch);
}

// Reduction side of the reduce-scatter fusion.  The chunk this rank owns is cut into `rs_phases`
// row groups and every group into pieces; a piece is pulled from all partial products (bulk loads
// into shared memory, `world` buffers per stage), added in fp32 in rank order and written as bf16.
// Pieces are handed out through a device-wide counter: the dedicated CTAs [0, copy_ctas) take
// pieces of a group as soon as every rank has flagged it, while the GEMM CTAs still work on the
// next group, and the GEMM CTAs join in when they have run out of tiles.
constexpr int kReduceStages = 3;
constexpr uint32_t kReduceStageBytes = 64 * 1024;
constexpr uint32_t kNoPiece = 0xffffffffu;

struct ReduceShared {           // lives behind the GEMM roles' barriers in shared memory
  uint64_t full[kReduceStages];
  uint32_t piece[kReduceStages];
  int bad;
};

__device__ void reduce_scatter_role(const FusedDev& f, const GemmDev& g, uint32_t epoch, uint8_t* smem, ReduceShared* sh) {
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < kReduceStages; ++s) tc::mbar_init(&sh->full[s], 1);
    sh->bad = 0;
    tc::mbar_init_fence();
  }
  __syncthreads();
  const uint32_t piece = (kReduceStageBytes / static_cast<uint32_t>(f.world)) & ~127u;   // bytes per rank per stage
  const unsigned long long chunk_bytes = static_cast<unsigned long long>(f.chunk_rows) * g.n * 2ull;
  const unsigned long long phase_bytes = chunk_bytes / f.rs_phases;
  const uint32_t pieces_per_phase = static_cast<uint32_t>((phase_bytes + piece - 1) / piece);
  const uint32_t total = pieces_per_phase * static_cast<uint32_t>(f.rs_phases);
  const unsigned long long my_base = static_cast<unsigned long long>(f.rank) * chunk_bytes;   // my rows inside a partial product
  volatile int* bad_flag = &sh->bad;

  auto piece_range = [&](uint32_t p, unsigned long long& off, uint32_t& n) {
    const uint32_t ph = p / pieces_per_phase, q = p % pieces_per_phase;
    const unsigned long long o = static_cast<unsigned long long>(q) * piece;
    n = static_cast<uint32_t>(phase_bytes - o < piece ? phase_bytes - o : piece);
    off = static_cast<unsigned long long>(ph) * phase_bytes + o;   // byte offset inside my chunk
  };
  uint32_t issued = 0;
  int ready_phase = -1;
  bool exhausted = false;
  // thread 0 only: takes the next piece, waits for its group's flags when needed, queues the loads
  auto issue = [&]() -> bool {
    const uint32_t s = issued % kReduceStages;
    const uint32_t p = exhausted ? total : atomicAdd(f.work_counter, 1u);
    ++issued;
    if (p >= total) {
      exhausted = true;
      sh->piece[s] = kNoPiece;
      return true;
    }
    const int ph = static_cast<int>(p / pieces_per_phase);
    while (ready_phase < ph) {
      for (int r = 0; r < f.world; ++r) {
        if (!sig_wait(f.sig[f.rank] + kFuseSigRs + 4 * r + (ready_phase + 1), epoch, f.timeout_ns)) {
          atomicCAS(f.status, 0, 0x200 + r);
          sh->piece[s] = kNoPiece;
          return false;
        }
      }
      ++ready_phase;
      asm volatile("fence.proxy.async;" ::: "memory");   // the partial products were written with ordinary stores
    }
    unsigned long long off;
    uint32_t n;
    piece_range(p, off, n);
    sh->piece[s] = p;
    tc::mbar_expect_tx(&sh->full[s], n * static_cast<uint32_t>(f.world));
    for (int r = 0; r < f.world; ++r)
      bulk_load(smem + static_cast<size_t>(s) * kReduceStageBytes + static_cast<size_t>(r) * piece,
                static_cast<const char*>(f.rs_partial[epoch & 1u][r]) + my_base + off, n, &sh->full[s]);
    return true;
  };
  uint32_t j = 0;
  for (;; ++j) {
    const uint32_t s = j % kReduceStages;
    // thread 0 keeps the ring full: the stage refilled here was released at the end of iteration j - 1
    if (tid == 0) {
      while (!*bad_flag && issued < j + kReduceStages) {
        if (!issue()) *bad_flag = 1;
      }
    }
    __syncthreads();
    const uint32_t p = sh->piece[s];
    if (p == kNoPiece || *bad_flag) break;   // uniform: both were written before the barrier above
    bool landed = false;
    {
      const unsigned long long t0 = now_ns();
      for (uint32_t i = 0;; ++i) {
        if (tc::mbar_try_wait(&sh->full[s], (j / kReduceStages) & 1u)) {
          landed = true;
          break;
        }
        if ((i & 255u) == 255u && now_ns() - t0 > f.timeout_ns + 2000000000ull) break;
      }
    }
    if (__syncthreads_or(landed ? 0 : 1)) {
      if (tid == 0) {
        *bad_flag = 1;
        atomicCAS(f.status, 0, 0x200 + f.rank);
      }
      break;
    }
    unsigned long long off;
    uint32_t n;
    piece_range(p, off, n);
    const uint8_t* st = smem + static_cast<size_t>(s) * kReduceStageBytes;
    uint4* out = reinterpret_cast<uint4*>(static_cast<char*>(f.rs_out) + off);
    for (uint32_t v = tid; v < n / 16; v += blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kFuseMaxRanks; ++r) {
        if (r < f.world) {
          const uint4 raw = reinterpret_cast<const uint4*>(st + static_cast<size_t>(r) * piece)[v];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 t = __bfloat1622float2(h[q]);
            acc[2 * q] += t.x;
            acc[2 * q + 1] += t.y;
          }
        }
      }
      uint4 pk;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      out[v] = pk;
    }
    __syncthreads();   // stage s may be refilled
  }
  __syncthreads();
  if (tid == 0 && *bad_flag) {
    // loads already queued must land before the CTA retires (stages whose entry is a real piece)
    for (uint32_t q = j; q < issued; ++q)
      if (sh->piece[q % kReduceStages] != kNoPiece) tc::mbar_wait(&sh->full[q % kReduceStages], (q / kReduceStages) & 1u, 1u << 22);
  }
}

// ++*epoch and, when given, *zeroed = 0 (the reduce-scatter fusion's piece counter).
__global__ void bump_epoch_kernel(uint32_t* epoch, uint32_t* zeroed) {
  *epoch = *epoch + 1;
  if (zeroed) *zeroed = 0;
}

constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);

template <int BN, int STAGES, bool kAMn, bool kBMn>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_persistent_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                 const __grid_constant__ CUtensorMap tma_b, GemmDev g,
                                                                 FusedDev f) {
  using L = PLayout<BN, STAGES>;
  static_assert(L::kTiles >= kCopyStages * static_cast<int>(kCopyPiece), "copy CTAs stage through the tile ring");
  static_assert(L::kTiles >= kReduceStages * static_cast<int>(kReduceStageBytes), "reducer CTAs stage through the tile ring");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* tiles = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kTiles);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // Tile ring: the producer publishes the tiles of this CTA (static round-robin order) to the MMA and epilogue
  // warps through a ring of four entries.  (A device-wide tile counter was tried in its place, so that a CTA
  // sharing its SM with a collective kernel would take fewer tiles: neutral on one GPU, 0.1-0.3 ms slower per
  // step on two, so it is gone; the collectives get SMs of their own instead.)
  uint64_t* sched_full = reinterpret_cast<uint64_t*>(smem + L::kTiles + L::kGemmBarriers + L::kReduceBarriers);
  uint64_t* sched_empty = sched_full + 4;
  volatile int* sched_tile = reinterpret_cast<volatile int*>(sched_empty + 4);

  // Dependent launch: this CTA may be resident while the previous kernel of the stream is still draining.  Barrier
  // init, tensor-memory allocation and descriptor prefetch below touch no global data; pdl_wait() comes before the
  // first access that does (at once for the fused roles, which read their call number from global memory).
  pdl_trigger();
  if (f.mode != FUSE_NONE) pdl_wait();
  const unsigned long long tl_t0 = tl_begin(g.tl);
  const uint32_t epoch = f.mode != FUSE_NONE ? *f.epoch_ptr : 0u;
  if (f.mode != FUSE_NONE && static_cast<int>(blockIdx.x) < f.copy_ctas) {
    // these CTAs move data; the others compute
    if (f.mode == FUSE_ALLGATHER_A) allgather_copy_role(f, epoch, smem);
    else reduce_scatter_role(f, g, epoch, smem, reinterpret_cast<ReduceShared*>(smem + L::kTiles + L::kGemmBarriers));
    return;
  }
  // in-CTA waits: two seconds alone, the cross-GPU limit plus two seconds when a role waits for peers
  const unsigned long long wait_ns = 2000000000ull + (f.mode != FUSE_NONE ? f.timeout_ns : 0ull);
  const int gcta = static_cast<int>(blockIdx.x) - f.copy_ctas, gctas = static_cast<int>(gridDim.x) - f.copy_ctas;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (g.m + BM - 1) / BM, n_tiles = (g.n + BN - 1) / BN;
  // Split-K: a work item is (tile, k-slice); slices of one tile run on different SMs
  // at the same time and add their partial sums into the fp32 output.
  const int splits = f.k_splits > 1 ? f.k_splits : 1;
  const int total_tiles = m_tiles * n_tiles * splits;
  const int num_kb = (g.k / BK) / splits;
  // Row-chunk rotation: tile order starts at this rank's own chunk (fusions only).
  const int m_rot = f.mode != FUSE_NONE ? (f.rank * (f.chunk_rows / BM)) % m_tiles : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], kEpiWarps);
    }
    for (int b = 0; b < 4; ++b) {
      tc::mbar_init(&sched_full[b], 1);
      tc::mbar_init(&sched_empty[b], 1 + kEpiWarps);   // the MMA thread and the epilogue warps
    }
    *abort_flag = 0;
    tc::mbar_init_fence();
    tc::tma_prefetch_desc(&tma_a);
    tc::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, 2 * BN);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (tl_t0 != 0ull && tl_detail(g.tl)) tl_mark(g.tl, tl_t0, tl_now(), TL_GEMM_PHASE, 0u);
  if (f.mode == FUSE_NONE) pdl_wait();   // set-up done: from here on operands are read and outputs written

  // Reduce-scatter fusion: phase-major order; inside a phase the chunks of the other ranks come first
  // (rank + 1, rank + 2, ...) and this rank's own chunk last, so what peers wait for is ready earliest.
  const int chunk_mt = f.mode == FUSE_REDUCE_SCATTER_D ? f.chunk_rows / BM : 1;
  const int phase_mt = f.mode == FUSE_REDUCE_SCATTER_D ? chunk_mt / f.rs_phases : 1;
  const int per_chunk_phase = phase_mt * n_tiles, per_phase = per_chunk_phase * f.world;
  auto tile_coords = [&](int w, int& m_blk, int& n_blk, int& kb0) -> int {
    if (f.mode == FUSE_REDUCE_SCATTER_D) {
      const int ph = w / per_phase, rem = w % per_phase;
      const int c = (f.rank + 1 + rem / per_chunk_phase) % f.world, rem2 = rem % per_chunk_phase;
      kb0 = 0;
      n_blk = rem2 % n_tiles;
      m_blk = c * chunk_mt + ph * phase_mt + rem2 / n_tiles;
      return ph;
    }
    const int t = w / splits;
    kb0 = (w % splits) * num_kb;
    n_blk = t % n_tiles;
    m_blk = (t / n_tiles + m_rot) % m_tiles;
    return 0;
  };

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;
      for (int i = 0; ok; ++i) {
        // draw and publish tile i of this CTA (-1: no more)
        const int slot = i & 3;
        if (i >= 4) {
          ok = wait_or_abort(&sched_empty[slot], ((i >> 2) - 1) & 1, abort_flag, wait_ns);
          if (!ok) break;
        }
        int t = gcta + i * gctas;   // static round-robin over the CTAs
        if (t >= total_tiles) t = -1;
        sched_tile[slot] = t;
        tc::mbar_arrive(&sched_full[slot]);
        if (t < 0) break;
        int m_blk, n_blk, kb0;
        tile_coords(t, m_blk, n_blk, kb0);
        if (f.mode == FUSE_ALLGATHER_A) {
          const int chunk = (m_blk * BM) / f.chunk_rows;
          ok = wait_flag_geq(f.chunk_flags + chunk, epoch, abort_flag, wait_ns);
          if (!ok) break;
          // the chunk was written with ordinary stores by other CTAs; TMA reads it through the async proxy
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES) ok = wait_or_abort(&empty[s], ((it / STAGES) - 1) & 1, abort_flag, wait_ns);
          if (!ok) break;
          tc::mbar_expect_tx(&full[s], L::kStageBytes);
          uint8_t* a_dst = tiles + s * L::kStageBytes;
          if (kAMn) {
#pragma unroll
            for (int gq = 0; gq < BM / 64; ++gq)
              tc::tma_load_2d(a_dst + gq * (BK * 128), &tma_a, &full[s], m_blk * BM + gq * 64, (kb0 + kb) * BK);
          } else {
            tc::tma_load_2d(a_dst, &tma_a, &full[s], (kb0 + kb) * BK, m_blk * BM);
          }
          if (kBMn) {
#pragma unroll
            for (int gq = 0; gq < BN / 64; ++gq)
              tc::tma_load_2d(a_dst + L::kABytes + gq * (BK * 128), &tma_b, &full[s], n_blk * BN + gq * 64, (kb0 + kb) * BK);
          } else {
            tc::tma_load_2d(a_dst + L::kABytes, &tma_b, &full[s], (kb0 + kb) * BK, n_blk * BN);
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(g.err, 1);
        // copies already issued must land before the CTA retires
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j) tc::mbar_wait(&full[j % STAGES], (j / STAGES) & 1, 1u << 20);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16(BM, BN, kAMn, kBMn);
      constexpr uint64_t a_step = kAMn ? (16 * 128) >> 4 : 2, b_step = kBMn ? (16 * 128) >> 4 : 2;
      bool ok = true;
      uint32_t it = 0;
      int i = 0;
      for (;; ++i) {
        const int slot = i & 3;
        ok = wait_or_abort(&sched_full[slot], (i >> 2) & 1, abort_flag, wait_ns);
        if (!ok) break;
        const int t = sched_tile[slot];
        tc::mbar_arrive(&sched_empty[slot]);
        if (t < 0) break;
        const int buf = i & 1;
        if (i >= 2) {
          ok = wait_or_abort(&acc_empty[buf], ((i >> 1) - 1) & 1, abort_flag, wait_ns);
          if (!ok) break;
          tc::fence_after_sync();
        }
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = wait_or_abort(&full[s], (it / STAGES) & 1, abort_flag, wait_ns);
          if (!ok) break;
          tc::fence_after_sync();
          const uint8_t* a_tile = tiles + s * L::kStageBytes;
          const uint64_t da = kAMn ? tc::smem_desc_mn_sw128(a_tile, BK * 128) : tc::smem_desc_k_sw128(a_tile);
          const uint64_t db = kBMn ? tc::smem_desc_mn_sw128(a_tile + L::kABytes, BK * 128) : tc::smem_desc_k_sw128(a_tile + L::kABytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4)
            tc::mma_bf16(tmem_d, da + a_step * k4, db + b_step * k4, idesc, (kb | k4) != 0);
          tc::mma_commit(&empty[s]);
        }
        if (!ok) break;
        tc::mma_commit(&acc_full[buf]);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(g.err, 2);
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue --
    // a warp may read only the 32 tensor-memory lanes of its index modulo four; the two warps of a quarter split the columns
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    constexpr int kHalfCols = BN / 2;
    bool ok = true;
    int i = 0;
    for (;; ++i) {
      const int slot = i & 3;
      ok = wait_or_abort(&sched_full[slot], (i >> 2) & 1, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int t = sched_tile[slot];
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sched_empty[slot]);
      if (t < 0) break;
      int m_blk, n_blk, kb0;
      const int phase = tile_coords(t, m_blk, n_blk, kb0);
      const int buf = i & 1;
      const bool stamp = warp == 2 && lane == 0 && tl_detail(g.tl);
      const unsigned long long ts0 = stamp ? tl_now() : 0ull;
      ok = wait_or_abort(&acc_full[buf], (i >> 1) & 1, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc::fence_after_sync();
      const unsigned long long ts1 = stamp ? tl_now() : 0ull;
      GemmDev gt = g;
      if (f.mode == FUSE_REDUCE_SCATTER_D) gt.d = f.rs_partial[epoch & 1u][f.rank];   // my partial product; the owners pull from it
      const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BN + half * kHalfCols) + (static_cast<uint32_t>(quarter * 32) << 16);
      const int col_base = n_blk * BN + half * kHalfCols;
      uint8_t* stage = smem + L::kStagingOff + (warp - 2) * L::kStagingPerWarp;
      const int row0 = m_blk * BM + quarter * 32;
      auto last_read = [&]() {
        // every column of this warp's part is in registers: hand the buffer back to the MMA warp
        tc::fence_before_sync();
        if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
      };
      epilogue_tile(gt, stage, tmem_d, row0, col_base, kHalfCols, lane, last_read);
      if (stamp) {
        const unsigned long long ts2 = tl_now();   // before the records below: their atomics take a microsecond
        tl_mark(g.tl, ts0, ts1, TL_GEMM_PHASE, (1u << 24) | static_cast<uint32_t>(i));
        tl_mark(g.tl, ts1, ts2, TL_GEMM_PHASE, (2u << 24) | static_cast<uint32_t>(i));
      }
      if (f.mode == FUSE_REDUCE_SCATTER_D) {
        // count this warp's part of the tile; the warp that completes a phase tells every rank
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          const uint32_t target = static_cast<uint32_t>(per_phase) * static_cast<uint32_t>(kEpiWarps);
          if (atomicAdd(f.phase_counters + phase, 1u) + 1u == target) {
            atomicExch(f.phase_counters + phase, 0u);
            __threadfence_system();
            for (int p = 0; p < f.world; ++p) sig_store(f.sig[p] + kFuseSigRs + 4 * f.rank + phase, epoch);
          }
        }
      }
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicExch(g.err, 3);
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, 2 * BN);
  }
  tl_end(g.tl, tl_t0, TL_GEMM, (static_cast<uint32_t>(m_tiles) << 16) | static_cast<uint32_t>(n_tiles * splits));
  // out of tiles: help with the reduction (the tile ring is idle now)
  if (f.mode == FUSE_REDUCE_SCATTER_D && *abort_flag == 0)
    reduce_scatter_role(f, g, epoch, smem, reinterpret_cast<ReduceShared*>(smem + L::kTiles + L::kGemmBarriers));
}

// Process-wide cap on the CTAs of plain GEMM launches (0 = one per SM); see set_gemm_cta_limit().
std::atomic<int> g_gemm_cta_limit{0};

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Number of k-slices that minimises ceil(items / SMs) * (k-blocks per item + fixed
// per-item cost).  Only fp32 outputs can be split (partial sums are added atomically).
int choose_splits(int tiles, int num_kb, int sms) {
  auto cost = [&](int s) {
    const long long rounds = (static_cast<long long>(tiles) * s + sms - 1) / sms;
    return rounds * (num_kb / s + 8 + (s > 1 ? 8 : 0));  // atomics make a split item's epilogue dearer
  };
  int best = 1;
  long long best_cost = cost(1);
  for (int s = 2; s <= 16; s *= 2) {
    if (num_kb % s != 0 || num_kb / s < 4) break;
    const long long c = cost(s);
    if (c * 5 < best_cost * 4 && c < (best == 1 ? best_cost : best_cost)) {  // at least 20 % better than no split
      if (best == 1 || c < best_cost) {
        best = s;
        best_cost = c;
      }
    }
  }
  return best;
}

template <int BN, int STAGES, bool kAMn, bool kBMn>
cudaError_t launch_persistent_cfg(const GemmArgs& a, const FusedDev& f_in, int max_ctas, cudaStream_t stream) {
  FusedDev f = f_in;
  using L = PLayout<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t rc = cudaFuncSetAttribute(gemm_persistent_kernel<BN, STAGES, kAMn, kBMn>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (rc != cudaSuccess) return rc;
    configured = true;
  }
  CUtensorMap ma, mb;
  const bool oka = kAMn ? encode_map(&ma, a.a, a.k, a.m, a.lda, BK) : encode_map(&ma, a.a, a.m, a.k, a.lda, BM);
  const bool okb = kBMn ? encode_map(&mb, a.b, a.k, a.n, a.ldb, BK) : encode_map(&mb, a.b, a.n, a.k, a.ldb, BN);
  if (!oka || !okb) return cudaErrorNotSupported;
  (void)cudaGetLastError();
  GemmDev g;
  g.d = a.d;
  g.aux = a.aux;
  g.bias = a.bias;
  g.residual = a.residual;
  g.mul = a.mul;
  g.m = a.m;
  g.n = a.n;
  g.k = a.k;
  g.ldd = a.ldd;
  g.d_fp32 = a.d_fp32 ? 1 : 0;
  g.accumulate = a.accumulate ? 1 : 0;
  g.epilogue = a.epilogue;
  g.atomic_add = 0;
  g.err = gemm_error_device_ptr();
  if (!g.err) return cudaErrorNotSupported;
  g.tl = timeline_device_ptr();
  int tiles = ((a.m + BM - 1) / BM) * ((a.n + BN - 1) / BN);
  f.k_splits = 1;
  static const bool allow_split = [] {
    const char* v = std::getenv("MCCL_GEMM_SPLITK");
    return !(v && v[0] == '0');
  }();
  if (allow_split && a.d_fp32 && a.epilogue == EPI_NONE && !a.residual && !a.mul && f.mode == FUSE_NONE) {
    const int splits = choose_splits(tiles, a.k / BK, sm_count());
    if (splits > 1) {
      if (!a.accumulate) {
        // partial sums are added into the output: start from zero
        if (a.ldd != a.n) goto no_split;
        cudaMemsetAsync(a.d, 0, static_cast<size_t>(a.m) * a.n * sizeof(float), stream);
      }
      f.k_splits = splits;
      g.atomic_add = 1;
      tiles *= splits;
    }
  }
no_split:
  int ctas = sm_count();
  if (max_ctas <= 0) max_ctas = g_gemm_cta_limit.load(std::memory_order_relaxed);
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  // fused roles wait on one another inside the kernel: every CTA must be resident (one per SM)
  int gemm_ctas = ctas - f.copy_ctas;
  if (gemm_ctas < 1) return cudaErrorInvalidValue;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  MCCL_LAUNCH_PDL((gemm_persistent_kernel<BN, STAGES, kAMn, kBMn>), gemm_ctas + f.copy_ctas, kGemmThreads, L::kTotal, stream, ma, mb, g, f);
  count_launch();
  return ::mccl::launch_status();
}

}  // namespace

int gemm_choose_splits(int tiles, int num_kb, int workers) { return choose_splits(tiles, num_kb, workers); }
void set_gemm_cta_limit(int ctas) { g_gemm_cta_limit.store(ctas > 0 ? ctas : 0, std::memory_order_relaxed); }
int gemm_cta_limit() { return g_gemm_cta_limit.load(std::memory_order_relaxed); }
int gemm_sm_count() { return sm_count(); }

cudaError_t launch_bump_epoch(uint32_t* epoch, uint32_t* zeroed, cudaStream_t stream) {
  MCCL_LAUNCH(bump_epoch_kernel, 1, 1, 0, stream, epoch, zeroed);
  return ::mccl::launch_status();
}

cudaError_t launch_gemm_persistent(const GemmArgs& a, const FusedDev& f, int max_ctas, cudaStream_t stream) {
  // Wide tiles when they still give every SM work; otherwise 128 x 128.
  const long long tiles256 = static_cast<long long>((a.m + BM - 1) / BM) * ((a.n + 255) / 256);
  const bool wide = a.n % 256 == 0 && tiles256 >= sm_count();
#define MCCL_PGEMM(BN, ST)                                                                                      \
  (a.a_mn_major ? (a.b_mn_major ? launch_persistent_cfg<BN, ST, true, true>(a, f, max_ctas, stream)             \
                                : launch_persistent_cfg<BN, ST, true, false>(a, f, max_ctas, stream))           \
                : (a.b_mn_major ? launch_persistent_cfg<BN, ST, false, true>(a, f, max_ctas, stream)            \
                                : launch_persistent_cfg<BN, ST, false, false>(a, f, max_ctas, stream)))
  return wide ? MCCL_PGEMM(256, 4) : MCCL_PGEMM(128, 6);
#undef MCCL_PGEMM
}

}  // namespace ops
}  // namespace mccl
