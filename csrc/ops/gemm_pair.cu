// bf16 GEMM on CTA pairs: D[M, N] = A[M, K] * B[N, K]^T with tcgen05.mma.cta_group::2.
//
// Why pairs.  The one-CTA kernel (gemm_persistent.cu) is bound by the operand bytes an SM can pull from L2: measured,
// its main loop moves about 54 bytes per clock per SM whatever the shape, while a 128 x 128 x 64 step needs 32 KB per
// 256 tensor-core clocks (128 B / clk) and a 128 x 256 x 64 step 48 KB per 512 (96 B / clk).  Two CTAs of a cluster
// that share one 256 x BN tile each load their own 128 rows of A but only HALF of the B tile; the MMA, issued by the
// even CTA for both, reads B from both shared memories.  Per 128 x BN output block that is 16 KB + BN/2 x 128 B per
// k-block instead of 16 KB + BN x 128 B: a quarter (BN = 128) or a third (BN = 256) fewer bytes through the same pipe.
// No load here uses cluster multicast: every CTA issues plain TMA tile loads into its own shared memory.
//
//   CTA r of the pair (r = %cluster_ctarank)
//     warp 0, lane 0   producer: TMA loads of A rows [256 i + 128 r, +128) and B rows [BN j + BN/2 r, +BN/2);
//                      the bytes of BOTH CTAs complete on the even CTA's `full` barrier
//     warp 1, lane 0   even CTA only: waits `full`, issues the MMAs for both CTAs, commits (multicast commit, which
//                      is an mbarrier arrive, not a load) to `empty` and `acc_full` of both CTAs
//     warps 2-9        epilogue of the CTA's own 128 accumulator rows (tensor memory of its own SM); when a buffer
//                      has been read, each warp arrives on the even CTA's `acc_empty`
//
// Every wait is bounded (two seconds); a wait that runs out sets the error word the host checks, the roles leave
// their loops, and both CTAs still meet at the cluster barrier before tensor memory is freed.
#include "gemm_common.cuh"
#include "gemm_persistent.cuh"

#include "../core/launch.hpp"

#include <cstdlib>

namespace mccl {
namespace ops {

int gemm_choose_splits(int tiles, int num_kb, int workers);   // gemm_persistent.cu

namespace {

// Epilogue warps per CTA: two per tensor-memory lane quarter; the GELU instantiation, whose epilogue is 25 instructions
// of arithmetic per value, takes four per quarter (each a quarter of the tile's columns) so that twice as many
// dependent chains are in flight per scheduler.
// (Wide tiles only: a warp finishes 64-column groups, and a 128-wide tile has just two of them per lane quarter.)
constexpr int pair_epi_warps(bool gelu, int bn) { return gelu && bn == 256 ? 16 : 8; }
constexpr int pair_threads(bool gelu, int bn) { return 32 * (2 + pair_epi_warps(gelu, bn)); }

template <int BN, int STAGES, bool kGelu = false>
struct PairLayout {
  static constexpr int kABytes = BM * BK * 2;             // this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * BK * 2;       // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTiles = STAGES * kStageBytes;
  static constexpr int kBarriers = (2 * STAGES + 4) * 8 + 16;
  static constexpr int kStagingOff = kTiles + 1024;      // 1024-byte aligned: TMA stores read it with the 128-byte swizzle
  static constexpr int kStagingPerWarp = 4096;
  static constexpr int kTotal = kStagingOff + pair_epi_warps(kGelu, BN) * kStagingPerWarp + 1024;
  static_assert(kBarriers <= 1024, "barriers overlap the epilogue staging");
  static_assert(kTotal <= 227 * 1024, "shared memory of one CTA");
};

__device__ __forceinline__ unsigned long long pair_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool pair_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < 64; ++i)
    if (tc::mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = pair_now_ns();
  for (uint32_t i = 0;; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u) {
      if (*abort_flag) return false;
      if (pair_now_ns() - t0 > 2000000000ull) return false;
    }
  }
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address, in the cluster's shared window, of the even CTA's copy of a shared-memory object of this CTA.
__device__ __forceinline__ uint32_t leader_addr(const void* p) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(tc::smem_u32(p)), "r"(0));
  return a;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile load of a CTA pair: the bytes land in this CTA's shared memory and complete on `bar_cluster_addr`
// (an address in the cluster window: the even CTA's barrier).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(tc::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs once every MMA issued so far has finished.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(tc::smem_u32(bar)), "h"(mask)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(smem_slot)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- epilogue by TMA store ---------------------------------------------------------------------------------------------
// Measured on a 4096 x 32000 x 512 product, an epilogue that moved every 4 output values with a handful of ordinary
// instructions (shared-memory transpose, address arithmetic, 8-byte stores) executed 19 000 warp instructions per
// 128 x 256 block and took 7.8 us of it, twice the time of the block's MMAs: the kernel was bound by instruction
// issue.  Here a thread converts its row, writes it to the warp's staging buffer (eight 16-byte stores, laid out as
// the 128-byte swizzle wants) and one lane hands the 32 x 128-byte box to the TMA unit, which clips it at the edges
// of the matrix.  fp32 partial sums (split-K, accumulation into a gradient) go out as TMA reductions (add).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(tc::smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(tc::smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the stores committed so far have read their shared-memory source (it may be overwritten)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 pk;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return pk;
}

// `ncols` (a multiple of 64) accumulator columns of this warp's 32 rows; the thread's row is row0 + lane.
template <bool kGelu, typename F>
__device__ __forceinline__ void epilogue_tma(const GemmDev& g, const CUtensorMap* map_d, const CUtensorMap* map_aux, uint8_t* stage, uint32_t taddr,
                                             int row0, int col0, int ncols, int lane, const float4& bias4, F&& last_read) {
  const int row = row0 + lane;
  const bool has_bias = g.epilogue == EPI_BIAS || g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_BIAS_GELU_D;
  const bool gelu_d = kGelu && (g.epilogue == EPI_BIAS_GELU_D || g.epilogue == EPI_GELU_D);
  const bool gelu_z = kGelu && (g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_GELU);
  // one input with the layout of the output is prefetched (the GELU instantiation takes none: its launcher refuses them)
  const __nv_bfloat16* extra_in = kGelu ? nullptr : (g.mul ? g.mul : g.residual);
  const bool both_in = !kGelu && g.mul != nullptr && g.residual != nullptr;
  if (g.d_fp32) {
    const bool add = g.atomic_add || g.accumulate;
#pragma unroll 1
    for (int c = 0; c < ncols; c += 32) {
      uint32_t r[32];
      tc::tmem_ld_32x32(taddr + static_cast<uint32_t>(c), r);
      tc::tmem_ld_wait();
      if (c + 32 >= ncols) last_read();
      const int cg = col0 + c;
      if (row0 >= g.m || cg >= g.n) continue;   // uniform over the warp
      if (has_bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (cg + j < g.n) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(g.bias + cg + j));
      }
      if (lane == 0) bulk_wait_read();
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) *stage_unit(stage, lane, j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (add) tma_reduce_add_2d(map_d, stage, cg, row0);
        else tma_store_2d(map_d, stage, cg, row0);
        bulk_commit();
      }
    }
    return;
  }
  if constexpr (kGelu) {
    // 32 columns at a time (one tensor-memory read, 32 live accumulators): this instantiation runs 576 threads and
    // has 112 registers per thread.  D goes to the staging buffer as it is produced, the second output waits packed
    // in registers until D's store has read the buffer.
#pragma unroll 1
    for (int c = 0; c < ncols; c += 64) {
      const int cg = col0 + c;
      const bool active = row0 < g.m && cg < g.n;   // uniform over the warp
      uint4 aux_out[8];
      if (lane == 0) bulk_wait_read();
      __syncwarp();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + static_cast<uint32_t>(c + 32 * h), r);
        tc::tmem_ld_wait();
        if (h == 1 && c + 64 >= ncols) last_read();
        if (!active) continue;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = 4 * h + jj;
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[jj * 8 + e]);
          if (has_bias) {
            const int src = (c >> 2) + 2 * j;
            v[0] += __shfl_sync(0xffffffffu, bias4.x, src);
            v[1] += __shfl_sync(0xffffffffu, bias4.y, src);
            v[2] += __shfl_sync(0xffffffffu, bias4.z, src);
            v[3] += __shfl_sync(0xffffffffu, bias4.w, src);
            v[4] += __shfl_sync(0xffffffffu, bias4.x, src + 1);
            v[5] += __shfl_sync(0xffffffffu, bias4.y, src + 1);
            v[6] += __shfl_sync(0xffffffffu, bias4.z, src + 1);
            v[7] += __shfl_sync(0xffffffffu, bias4.w, src + 1);
          }
          if (gelu_d) {
            // value and derivative share one exponential; the derivative is what backward needs, so it is saved instead of z
            float dv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) gelu_value_grad(v[e], v[e], dv[e]);
            aux_out[j] = pack8(dv);
          } else {
            aux_out[j] = pack8(v);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = gelu_erf(v[e]);
          }
          *stage_unit(stage, lane, j) = pack8(v);
        }
      }
      if (!active) continue;
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map_d, stage, cg, row0);
        bulk_commit();
        bulk_wait_read();
      }
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) *stage_unit(stage, lane, j) = aux_out[j];
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map_aux, stage, cg, row0);
        bulk_commit();
      }
    }
    return;
  }
#pragma unroll 1
  for (int c = 0; c < ncols; c += 64) {
    uint32_t ra[32], rb[32];
    tc::tmem_ld_32x32(taddr + static_cast<uint32_t>(c), ra);
    tc::tmem_ld_32x32(taddr + static_cast<uint32_t>(c + 32), rb);
    const int cg = col0 + c;
    // the thread's 64 values of the multiplier (or residual): eight independent loads in flight during the wait below
    uint4 extra[8];
    if (extra_in && row < g.m) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (cg + j * 8 < g.n) extra[j] = __ldg(reinterpret_cast<const uint4*>(extra_in + static_cast<size_t>(row) * g.ldd + cg + j * 8));
    }
    tc::tmem_ld_wait();
    if (c + 64 >= ncols) last_read();
    if (row0 >= g.m || cg >= g.n) continue;   // uniform over the warp
    uint4 out[8], aux_out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(j < 4 ? ra[j * 8 + e] : rb[(j - 4) * 8 + e]);
      const int col = cg + j * 8;
      const bool inside = col < g.n;   // N is a multiple of 8
      if (has_bias) {
        // lane l holds the bias of columns [col0 + 4 l, col0 + 4 l + 4) of this warp's span (zero outside the matrix)
        const int src = (c >> 2) + 2 * j;
        v[0] += __shfl_sync(0xffffffffu, bias4.x, src);
        v[1] += __shfl_sync(0xffffffffu, bias4.y, src);
        v[2] += __shfl_sync(0xffffffffu, bias4.z, src);
        v[3] += __shfl_sync(0xffffffffu, bias4.w, src);
        v[4] += __shfl_sync(0xffffffffu, bias4.x, src + 1);
        v[5] += __shfl_sync(0xffffffffu, bias4.y, src + 1);
        v[6] += __shfl_sync(0xffffffffu, bias4.z, src + 1);
        v[7] += __shfl_sync(0xffffffffu, bias4.w, src + 1);
      }
      if (kGelu && gelu_d) {
        // value and derivative share one exponential; the derivative is what backward needs, so it is saved instead of z
        float dv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) gelu_value_grad(v[e], v[e], dv[e]);
        aux_out[j] = pack8(dv);
      } else if (kGelu && gelu_z) {
        aux_out[j] = pack8(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = gelu_erf(v[e]);
      }
      if (extra_in && inside && row < g.m) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&extra[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __bfloat1622float2(h[e]);
          if (g.mul) {
            v[2 * e] *= t.x;
            v[2 * e + 1] *= t.y;
          } else {
            v[2 * e] += t.x;
            v[2 * e + 1] += t.y;
          }
        }
      }
      if (both_in && inside && row < g.m) {
        const uint4 pk = *reinterpret_cast<const uint4*>(g.residual + static_cast<size_t>(row) * g.ldd + col);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __bfloat1622float2(h[e]);
          v[2 * e] += t.x;
          v[2 * e + 1] += t.y;
        }
      }
      out[j] = pack8(v);
    }
    if (lane == 0) bulk_wait_read();
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) *stage_unit(stage, lane, j) = out[j];
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_d, stage, cg, row0);
      bulk_commit();
    }
    if (kGelu && (gelu_d || gelu_z)) {
      if (lane == 0) bulk_wait_read();
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) *stage_unit(stage, lane, j) = aux_out[j];
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map_aux, stage, cg, row0);
        bulk_commit();
      }
    }
  }
}

// kGelu: the instantiation for GELU epilogues (two outputs, 25 instructions of arithmetic per value).  It is a kernel of
// its own so that every other product runs without that code in its instruction stream.
template <int BN, int STAGES, bool kAMn, bool kBMn, bool kGelu>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads(kGelu, BN), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_d, const __grid_constant__ CUtensorMap tma_aux, GemmDev g, int k_splits) {
  using L = PairLayout<BN, STAGES, kGelu>;
  constexpr int BNH = BN / 2;
  extern __shared__ uint8_t smem_raw[];
  // the same offset in both CTAs: the MMA addresses the peer's operands by this CTA's offsets
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* tiles = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kTiles);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // Dependent launch (only with MCCL_PDL=1): the kernel after this one may become resident as SMs free up; this
  // kernel's own set-up below touches no global data and runs while the kernel before it drains.
  pdl_trigger();
  const unsigned long long tl_t0 = tl_begin(g.tl);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = static_cast<int>(blockIdx.x >> 1), pairs = static_cast<int>(gridDim.x >> 1);
  const int m_tiles = (g.m + 2 * BM - 1) / (2 * BM), n_tiles = (g.n + BN - 1) / BN;
  const int splits = k_splits > 1 ? k_splits : 1;
  const int total = m_tiles * n_tiles * splits;
  const int num_kb = (g.k / BK) / splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full[s], 1);     // the even CTA's producer arrives once and expects the bytes of both CTAs
      tc::mbar_init(&empty[s], 1);    // one commit per use, delivered to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 2 * pair_epi_warps(kGelu, BN));   // the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    tc::mbar_init_fence();
    tc::tma_prefetch_desc(&tma_a);
    tc::tma_prefetch_desc(&tma_b);
    tc::tma_prefetch_desc(&tma_d);
    if (g.aux) tc::tma_prefetch_desc(&tma_aux);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 2 * BN);
  tc::fence_before_sync();
  __syncthreads();
  // the peer's barriers exist and its tensor memory is allocated before anything is sent its way
  cluster_sync_all();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // set-up done: from here on operands are read and outputs written
  if (tl_t0 != 0ull && tl_detail(g.tl)) tl_mark(g.tl, tl_t0, tl_now(), TL_GEMM_PHASE, 0u);

  auto tile_coords = [&](int w, int& m_blk, int& n_blk, int& kb0) {
    const int t = w / splits;
    kb0 = (w % splits) * num_kb;
    n_blk = t % n_tiles;
    m_blk = t / n_tiles;
  };

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;
      for (int w = pair; w < total && ok; w += pairs) {
        int m_blk, n_blk, kb0;
        tile_coords(w, m_blk, n_blk, kb0);
        const int a_row = m_blk * 2 * BM + static_cast<int>(rank) * BM;
        const int b_row = n_blk * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES) ok = pair_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag);
          if (!ok) break;
          if (rank == 0) tc::mbar_expect_tx(&full[s], 2 * L::kStageBytes);
          const uint32_t bar = leader_addr(&full[s]);
          uint8_t* a_dst = tiles + s * L::kStageBytes;
          if (kAMn) {
#pragma unroll
            for (int gq = 0; gq < BM / 64; ++gq) tma_load_2d_pair(a_dst + gq * (BK * 128), &tma_a, bar, a_row + gq * 64, (kb0 + kb) * BK);
          } else {
            tma_load_2d_pair(a_dst, &tma_a, bar, (kb0 + kb) * BK, a_row);
          }
          if (kBMn) {
#pragma unroll
            for (int gq = 0; gq < BNH / 64; ++gq)
              tma_load_2d_pair(a_dst + L::kABytes + gq * (BK * 128), &tma_b, bar, b_row + gq * 64, (kb0 + kb) * BK);
          } else {
            tma_load_2d_pair(a_dst + L::kABytes, &tma_b, bar, (kb0 + kb) * BK, b_row);
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(g.err, 11);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16(2 * BM, BN, kAMn, kBMn);
      constexpr uint64_t a_step = kAMn ? (16 * 128) >> 4 : 2, b_step = kBMn ? (16 * 128) >> 4 : 2;
      bool ok = true;
      uint32_t it = 0;
      int i = 0;
      for (int w = pair; w < total; w += pairs, ++i) {
        const int buf = i & 1;
        if (i >= 2) {
          ok = pair_wait(&acc_empty[buf], ((i >> 1) - 1) & 1, abort_flag);
          if (!ok) break;
          tc::fence_after_sync();
        }
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = pair_wait(&full[s], (it / STAGES) & 1, abort_flag);
          if (!ok) break;
          tc::fence_after_sync();
          const uint8_t* a_tile = tiles + s * L::kStageBytes;
          const uint64_t da = kAMn ? tc::smem_desc_mn_sw128(a_tile, BK * 128) : tc::smem_desc_k_sw128(a_tile);
          const uint64_t db = kBMn ? tc::smem_desc_mn_sw128(a_tile + L::kABytes, BK * 128) : tc::smem_desc_k_sw128(a_tile + L::kABytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4) mma_bf16_pair(tmem_d, da + a_step * k4, db + b_step * k4, idesc, (kb | k4) != 0);
          mma_commit_pair(&empty[s]);
        }
        if (!ok) break;
        mma_commit_pair(&acc_full[buf]);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(g.err, 12);
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue --
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    constexpr int kHalfCols = BN / (pair_epi_warps(kGelu, BN) / 4);   // columns per epilogue warp
    uint8_t* stage = smem + L::kStagingOff + (warp - 2) * L::kStagingPerWarp;
    const bool has_bias = g.epilogue == EPI_BIAS || g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_BIAS_GELU_D;
    bool ok = true;
    int i = 0;
    for (int w = pair; w < total; w += pairs, ++i) {
      int m_blk, n_blk, kb0;
      tile_coords(w, m_blk, n_blk, kb0);
      const int buf = i & 1;
      const bool stamp = warp == 2 && lane == 0 && tl_detail(g.tl);
      const unsigned long long ts0 = stamp ? tl_now() : 0ull;
      // this warp's bias values, one float4 per lane, fetched while the MMAs of the tile still run
      float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (has_bias) {
        const int bc = n_blk * BN + half * kHalfCols + 4 * lane;
        if (4 * lane < kHalfCols && bc < g.n) {   // N is a multiple of 8: four columns are inside or outside together
          if ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0) bias4 = __ldg(reinterpret_cast<const float4*>(g.bias + bc));
          else bias4 = make_float4(__ldg(g.bias + bc), __ldg(g.bias + bc + 1), __ldg(g.bias + bc + 2), __ldg(g.bias + bc + 3));
        }
      }
      ok = pair_wait(&acc_full[buf], (i >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc::fence_after_sync();
      const unsigned long long ts1 = stamp ? tl_now() : 0ull;
      const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BN + half * kHalfCols) + (static_cast<uint32_t>(quarter * 32) << 16);
      const int col_base = n_blk * BN + half * kHalfCols;
      const int row0 = m_blk * 2 * BM + static_cast<int>(rank) * BM + quarter * 32;
      const uint32_t acc_empty_leader = leader_addr(&acc_empty[buf]);
      auto last_read = [&]() {
        // every column of this warp's part is in registers: hand the buffer back to the MMA thread of the even CTA
        tc::fence_before_sync();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      };
      epilogue_tma<kGelu>(g, &tma_d, &tma_aux, stage, tmem_d, row0, col_base, kHalfCols, lane, bias4, last_read);
      if (stamp) {
        const unsigned long long ts2 = tl_now();   // before the records below: their atomics take a microsecond
        tl_mark(g.tl, ts0, ts1, TL_GEMM_PHASE, (1u << 24) | static_cast<uint32_t>(i));
        tl_mark(g.tl, ts1, ts2, TL_GEMM_PHASE, (2u << 24) | static_cast<uint32_t>(i));
      }
    }
    if (lane == 0) bulk_wait_read();   // the stores have read this warp's staging buffer; kernel completion publishes them
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicExch(g.err, 13);
    }
  }
  if (*abort_flag) {
    // a wait ran out somewhere: loads this pair still has in flight get time to land before shared memory is given up
    const unsigned long long t0 = pair_now_ns();
    while (pair_now_ns() - t0 < 50000ull) __nanosleep(1000);
  }
  tc::fence_before_sync();
  __syncthreads();
  // nothing of the peer is touched after this: its shared memory (operands the MMAs read) and barriers (remote arrives)
  cluster_sync_all();
  if (warp == 1) {
    tc::fence_after_sync();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
  tl_end(g.tl, tl_t0, TL_GEMM, (static_cast<uint32_t>(m_tiles * 2) << 16) | static_cast<uint32_t>(n_tiles * splits));
}

// Clusters of two that can be resident at once (GPCs with an odd number of free SMs leave one SM out).
template <int BN, int STAGES, bool kAMn, bool kBMn, bool kGelu>
int max_pairs() {
  using L = PairLayout<BN, STAGES, kGelu>;
  static int cached = 0;
  if (cached > 0) return cached;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 74);
  cfg.blockDim = dim3(pair_threads(kGelu, BN));
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.numAttrs = 0;   // the cluster shape is part of the kernel (__cluster_dims__)
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<BN, STAGES, kAMn, kBMn, kGelu>, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = gemm_sm_count() / 2 - 2;
  }
  cached = n;
  return n;
}

template <int BN, int STAGES, bool kAMn, bool kBMn, bool kGelu = false>
cudaError_t launch_pair_cfg(const GemmArgs& a, cudaStream_t stream) {
  using L = PairLayout<BN, STAGES, kGelu>;
  static bool configured = false;
  if (!configured) {
    cudaError_t rc = cudaFuncSetAttribute(gemm_pair_kernel<BN, STAGES, kAMn, kBMn, kGelu>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (rc != cudaSuccess) return rc;
    configured = true;
  }
  CUtensorMap ma, mb;
  const bool oka = kAMn ? encode_map(&ma, a.a, a.k, a.m, a.lda, BK) : encode_map(&ma, a.a, a.m, a.k, a.lda, BM);
  const bool okb = kBMn ? encode_map(&mb, a.b, a.k, a.n, a.ldb, BK) : encode_map(&mb, a.b, a.n, a.k, a.ldb, BN / 2);
  CUtensorMap md, maux;
  if (!oka || !okb || !encode_out_map(&md, a.d, a.m, a.n, a.ldd, a.d_fp32)) return cudaErrorNotSupported;
  if (a.aux) {
    if (!encode_out_map(&maux, a.aux, a.m, a.n, a.ldd, false)) return cudaErrorNotSupported;
  } else {
    maux = md;   // never used
  }
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
  int pairs = max_pairs<BN, STAGES, kAMn, kBMn, kGelu>();
  const int limit = gemm_cta_limit();
  if (limit > 0 && limit / 2 < pairs) pairs = limit / 2;
  if (pairs < 1) return cudaErrorInvalidValue;
  int tiles = ((a.m + 2 * BM - 1) / (2 * BM)) * ((a.n + BN - 1) / BN);
  int splits = 1;
  static const bool allow_split = [] {
    const char* v = std::getenv("MCCL_GEMM_SPLITK");
    return !(v && v[0] == '0');
  }();
  if (allow_split && a.d_fp32 && a.epilogue == EPI_NONE && !a.residual && !a.mul) {
    const int s = gemm_choose_splits(tiles, a.k / BK, pairs);
    if (s > 1 && (a.accumulate || a.ldd == a.n)) {
      // partial sums are added into the output: start from zero unless the caller accumulates anyway
      if (!a.accumulate) cudaMemsetAsync(a.d, 0, static_cast<size_t>(a.m) * a.n * sizeof(float), stream);
      splits = s;
      g.atomic_add = 1;
      tiles *= s;
    }
  }
  if (tiles < pairs) pairs = tiles;
  MCCL_LAUNCH_PDL((gemm_pair_kernel<BN, STAGES, kAMn, kBMn, kGelu>), 2 * pairs, pair_threads(kGelu, BN), L::kTotal, stream, ma, mb, md, maux, g, splits);
  count_launch();
  return ::mccl::launch_status();
}

}  // namespace

cudaError_t launch_gemm_pair(const GemmArgs& a, cudaStream_t stream) {
  // Tile width by a small cost model (microseconds, fitted to device timelines of this kernel): a k-block of a
  // 256 x 256 pair tile takes 0.45 us and one of a 256 x 128 tile 0.33 us, so the wide tile does twice the work for
  // 1.4 times the time whenever it leaves no SM idle; its epilogue is about twice as long.  Split-K (fp32 outputs
  // only) multiplies the work items, which is what lets small weight-gradient products use wide tiles at all.
  int pairs = gemm_sm_count() / 2;
  const int limit = gemm_cta_limit();
  if (limit > 0 && limit / 2 < pairs) pairs = limit / 2;
  if (pairs < 1) pairs = 1;
  const int kb = a.k / BK;
  const bool splittable = a.d_fp32 && a.epilogue == EPI_NONE && !a.residual && !a.mul && (a.accumulate || a.ldd == a.n);
  auto estimate = [&](int bn) {
    const int tiles = ((a.m + 2 * BM - 1) / (2 * BM)) * ((a.n + bn - 1) / bn);
    const int s = splittable ? gemm_choose_splits(tiles, kb, pairs) : 1;
    const int rounds = (tiles * s + pairs - 1) / pairs;
    const double t_kb = bn == 256 ? 0.45 : 0.33, t_epi = bn == 256 ? 3.0 : 1.8;
    return rounds * ((kb / s) * t_kb + t_epi + (s > 1 ? 1.0 : 0.0));
  };
  const bool wide = a.n > 128 && estimate(256) < estimate(128);
#define MCCL_PAIR(BN, ST)                                                                               \
  (a.a_mn_major ? (a.b_mn_major ? launch_pair_cfg<BN, ST, true, true>(a, stream)                        \
                                : launch_pair_cfg<BN, ST, true, false>(a, stream))                      \
                : (a.b_mn_major ? launch_pair_cfg<BN, ST, false, true>(a, stream)                       \
                                : launch_pair_cfg<BN, ST, false, false>(a, stream)))
  const bool gelu = a.epilogue == EPI_BIAS_GELU || a.epilogue == EPI_GELU || a.epilogue == EPI_BIAS_GELU_D || a.epilogue == EPI_GELU_D;
  if (gelu) {
    // activations are applied in forward products only; combined with a multiplier or residual they take the one-CTA kernel
    if (a.a_mn_major || a.b_mn_major || a.mul || a.residual) return launch_gemm_persistent(a, FusedDev{}, 0, stream);
    // sixteen staging buffers in the wide instantiation: one TMA stage fewer
    return wide ? launch_pair_cfg<256, 5, false, false, true>(a, stream) : launch_pair_cfg<128, 8, false, false, true>(a, stream);
  }
  return wide ? MCCL_PAIR(256, 6) : MCCL_PAIR(128, 8);
#undef MCCL_PAIR
}

}  // namespace ops
}  // namespace mccl
