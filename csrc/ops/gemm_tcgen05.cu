// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = A[M,K] · B[N,K]^T with
// fused epilogues (bias, GELU with saved pre-activation, fp32 output with
// accumulation for weight gradients).
//
// Structure per CTA (one 128 x BN output tile):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A (128 x 64)
//               and B (BN x 64) k-blocks into a ring of swizzled smem stages
//   warp 1      allocates tensor memory, issues tcgen05.mma (one thread), and
//               releases each stage with tcgen05.commit
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator (one TMEM lane
//               quarter per warp), bias / activation, 16-byte global stores
// Shared memory per CTA is kept under half an SM so two CTAs are resident and
// one tile's epilogue overlaps the other's main loop.
//
// The reference has no GEMM of its own (no tensor-core code at all); this
// kernel exists for the model operators and as the core the fused
// all-gather→GEMM / GEMM→reduce-scatter tensor-parallel kernels build on.
#include "../core/launch.hpp"
#include "gemm_common.cuh"
#include "gemm_persistent.cuh"

#include <atomic>

#include <cstdlib>
#include <string>

namespace mccl {
namespace ops {

namespace {

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTiles = STAGES * kStageBytes;
  static constexpr int kBarriers = (2 * STAGES + 1) * 8 + 16;
  static constexpr int kTotal = kTiles + kBarriers + 1024;  // slack for 1024-byte alignment
};

// kAMn / kBMn: the operand is stored with its M (or N) index contiguous, i.e. as a
// [K, M] (or [K, N]) row-major matrix; the tile is then fetched as 64-wide column
// groups of BK rows each and described to the tensor core as MN-major.
template <int BN, int STAGES, bool kAMn, bool kBMn>
__global__ void __launch_bounds__(192) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                        const __grid_constant__ CUtensorMap tma_b, GemmDev g) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* tiles = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kTiles);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_ready = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blk = blockIdx.x, m_blk = blockIdx.y;
  const int num_kb = g.k / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 1);
    }
    tc::mbar_init(acc_ready, 1);
    tc::mbar_init_fence();
    tc::tma_prefetch_desc(&tma_a);
    tc::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, BN);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES) ok = tc::mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1);
        if (!ok) break;
        tc::mbar_expect_tx(&full[s], L::kStageBytes);
        uint8_t* a_dst = tiles + s * L::kStageBytes;
        if (kAMn) {
#pragma unroll
          for (int gq = 0; gq < BM / 64; ++gq)
            tc::tma_load_2d(a_dst + gq * (BK * 128), &tma_a, &full[s], m_blk * BM + gq * 64, kb * BK);
        } else {
          tc::tma_load_2d(a_dst, &tma_a, &full[s], kb * BK, m_blk * BM);
        }
        if (kBMn) {
#pragma unroll
          for (int gq = 0; gq < BN / 64; ++gq)
            tc::tma_load_2d(a_dst + L::kABytes + gq * (BK * 128), &tma_b, &full[s], n_blk * BN + gq * 64, kb * BK);
        } else {
          tc::tma_load_2d(a_dst + L::kABytes, &tma_b, &full[s], kb * BK, n_blk * BN);
        }
        issued = kb + 1;
      }
      if (!ok) {
        atomicExch(g.err, 1);
        // let the copies already in flight land before the CTA retires
        for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb)
          tc::mbar_wait(&full[kb % STAGES], (kb / STAGES) & 1, 1u << 20);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16(BM, BN, kAMn, kBMn);
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        ok = tc::mbar_wait(&full[s], (kb / STAGES) & 1);
        if (!ok) break;
        tc::fence_after_sync();
        const uint8_t* a_tile = tiles + s * L::kStageBytes;
        const uint64_t da = kAMn ? tc::smem_desc_mn_sw128(a_tile, BK * 128) : tc::smem_desc_k_sw128(a_tile);
        const uint64_t db = kBMn ? tc::smem_desc_mn_sw128(a_tile + L::kABytes, BK * 128) : tc::smem_desc_k_sw128(a_tile + L::kABytes);
        // Advancing K by 16 elements: K-major = 32 bytes inside the swizzled row (+2 in the
        // 16-byte address field); MN-major = 16 rows of 128 bytes (+128).
        constexpr uint64_t a_step = kAMn ? (16 * 128) >> 4 : 2, b_step = kBMn ? (16 * 128) >> 4 : 2;
#pragma unroll
        for (int k4 = 0; k4 < BK / UMMA_K; ++k4)
          tc::mma_bf16(tmem_base, da + a_step * k4, db + b_step * k4, idesc, (kb | k4) != 0);
        tc::mma_commit(&empty[s]);  // frees the stage once these MMAs have read it
      }
      if (!ok) atomicExch(g.err, 2);
      tc::mma_commit(acc_ready);    // on the failure path this still releases the epilogue warps
    }
  } else {
    // ----------------------------------------------------------- epilogue --
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const bool ok = tc::mbar_wait(acc_ready, 0);
    tc::fence_after_sync();
    const int row = m_blk * BM + quarter * 32 + lane;
    const bool failed = !ok || (*reinterpret_cast<volatile int*>(g.err) != 0);
    if (!ok && lane == 0) atomicExch(g.err, 3);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t r[32];
      tc::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c0), r);
      tc::tmem_ld_wait();
      const int col0 = n_blk * BN + c0;
      if (failed || row >= g.m || col0 >= g.n) continue;
      epilogue_store(g, row, col0, r);
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, BN);
  }
}

thread_local const char* t_reason = "";
cudaError_t unsupported(const char* why) {
  t_reason = why;
  return cudaErrorNotSupported;
}

template <int BN, int STAGES, bool kAMn, bool kBMn>
cudaError_t launch_cfg(const GemmArgs& a, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t rc = cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, kAMn, kBMn>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          L::kTotal);
    if (rc != cudaSuccess) return rc;
    configured = true;
  }
  CUtensorMap ma, mb;
  const bool oka = kAMn ? encode_map(&ma, a.a, a.k, a.m, a.lda, BK) : encode_map(&ma, a.a, a.m, a.k, a.lda, BM);
  const bool okb = kBMn ? encode_map(&mb, a.b, a.k, a.n, a.ldb, BK) : encode_map(&mb, a.b, a.n, a.k, a.ldb, BN);
  if (!oka || !okb) return unsupported("cuTensorMapEncodeTiled rejected an operand");
  (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be blamed on this launch
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
  if (!g.err) return unsupported("no device error word");
  g.tl = nullptr;
  dim3 grid((a.n + BN - 1) / BN, (a.m + BM - 1) / BM);
  MCCL_LAUNCH((gemm_bf16_kernel<BN, STAGES, kAMn, kBMn>), grid, 192, L::kTotal, stream, ma, mb, g);
  count_launch();
  return ::mccl::launch_status();
}

}  // namespace

#ifndef MCCL_GEMM_DEFAULT_KERNEL
#define MCCL_GEMM_DEFAULT_KERNEL 1
#endif

namespace {
std::atomic<int> g_gemm_kernel_override{-1};
int kernel_index(const std::string& s) {
  return s == "tile" ? 2 : (s == "pair" ? 1 : (s == "persistent" ? 0 : MCCL_GEMM_DEFAULT_KERNEL));
}
}  // namespace

// "pair", "persistent" or "tile" for the calls that follow; "" returns to MCCL_GEMM_KERNEL / the default.
void set_gemm_kernel(const std::string& name) {
  g_gemm_kernel_override.store(name.empty() ? -1 : kernel_index(name), std::memory_order_relaxed);
}

const char* gemm_last_reason() { return t_reason; }

cudaError_t gemm_bf16_tn(const GemmArgs& a, cudaStream_t stream) {
  t_reason = "";
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return cudaErrorInvalidValue;
  if (a.k % BK != 0 || a.n % 8 != 0) return unsupported("K must be a multiple of 64 and N a multiple of 8");
  if (a.lda % 8 != 0 || a.ldb % 8 != 0 || a.ldd % (a.d_fp32 ? 4 : 8) != 0)
    return unsupported("row strides must keep rows 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.d)) & 15u)
    return unsupported("operand pointers must be 16-byte aligned");
  if (a.aux && (reinterpret_cast<uintptr_t>(a.aux) & 15u)) return unsupported("aux pointer must be 16-byte aligned");
  if ((a.epilogue == EPI_BIAS || a.epilogue == EPI_BIAS_GELU || a.epilogue == EPI_BIAS_GELU_D) && !a.bias) return cudaErrorInvalidValue;
  if ((a.epilogue == EPI_BIAS_GELU || a.epilogue == EPI_GELU || a.epilogue == EPI_BIAS_GELU_D || a.epilogue == EPI_GELU_D) &&
      (!a.aux || a.d_fp32))
    return cudaErrorInvalidValue;
  if (a.accumulate && !a.d_fp32) return cudaErrorInvalidValue;
  if (a.residual && (reinterpret_cast<uintptr_t>(a.residual) & 15u)) return unsupported("residual pointer must be 16-byte aligned");
  if (a.mul && ((reinterpret_cast<uintptr_t>(a.mul) & 15u) || a.d_fp32)) return unsupported("mul must be 16-byte aligned and the output bf16");
  if (a.a_mn_major && a.m % 8 != 0) return unsupported("an MN-major A needs M to be a multiple of 8");
  // MCCL_GEMM_KERNEL: "pair" = CTA pairs (tcgen05.mma.cta_group::2), "persistent" = one CTA per SM,
  // "tile" = the one-tile-per-CTA kernel below.
  static const int env_choice = [] {
    const char* v = std::getenv("MCCL_GEMM_KERNEL");
    return kernel_index(v ? v : "");
  }();
  const int forced = g_gemm_kernel_override.load(std::memory_order_relaxed);
  const int kernel_choice = forced >= 0 ? forced : env_choice;
  if (kernel_choice != 2) {
    cudaError_t rc = kernel_choice == 1 ? launch_gemm_pair(a, stream) : launch_gemm_persistent(a, FusedDev{}, 0, stream);
    if (rc == cudaErrorNotSupported) return unsupported("cuTensorMapEncodeTiled rejected an operand");
    return rc;
  }
  // 128 x 128 tiles, 3 stages of 32 KB: two CTAs per SM.
  if (a.a_mn_major) return a.b_mn_major ? launch_cfg<128, 3, true, true>(a, stream) : launch_cfg<128, 3, true, false>(a, stream);
  return a.b_mn_major ? launch_cfg<128, 3, false, true>(a, stream) : launch_cfg<128, 3, false, false>(a, stream);
}

namespace {
__device__ int g_gemm_error = 0;
}

int* gemm_error_device_ptr() {
  static int* ptr = nullptr;
  if (!ptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_gemm_error) == cudaSuccess) ptr = static_cast<int*>(p);
  }
  return ptr;
}

int gemm_error_flag() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int));
  return v;
}

}  // namespace ops
}  // namespace mccl
