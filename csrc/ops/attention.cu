// Causal self-attention for sm_100a, head dimension 64, forward and backward, on the 5th-generation tensor cores.
//
// Operands come straight from the fused QKV projection: qkv is [B, S, 3, H, 64] bf16 (the projection's output
// viewed, not copied), so q, k and v tiles of a (batch, head) are boxes of one 2-D tensor map over the
// [B*S, 3*H*64] matrix, fetched by TMA into 128-byte-swizzled shared memory.  The output is written as
// [B, S, H, 64], which is the layout the output projection reads, and backward produces the gradient of the whole
// qkv tensor in one piece.  Nothing is transposed, sliced or concatenated around the kernels.
//
// Forward, one CTA per (batch, head, block of 128 queries), looping over the key blocks up to the diagonal:
//   S = Q K^T           tcgen05.mma, fp32 accumulator in tensor memory (128 lanes x 128 columns)
//   P = exp2(S*c - m)   tcgen05.ld, one query row per thread, running max / sum (online softmax), P written as bf16
//                       into shared memory in the layout the next MMA reads as its A operand
//   O += P V            tcgen05.mma into a second tensor-memory region, folded into registers with the rescale
// Backward, one CTA per (batch, head) for S = 256 (two blocks; dQ, dK, dV accumulate in tensor memory):
//   per block pair (i, j <= i):  S = Q_i K_j^T,  P = exp2(S*c - L_i),  dP = dO_i V_j^T,  dS = P (dP - delta_i) c,
//                                dV_j += P^T dO_i,  dK_j += dS^T Q_i,  dQ_i += dS K_j
// The transposed products read P / dS from the same shared-memory tile through an MN-major operand descriptor.
//
// The reference has no attention kernel (its models call PyTorch's); this one exists because attention and the
// copies around it are a tenth of the headline training step.  Every wait is bounded: on a timeout the kernel sets
// the GEMM error word, frees its tensor memory and returns.
#include "../core/launch.hpp"
#include "gemm_common.cuh"

namespace mccl {
namespace ops {

namespace {

constexpr int kBlk = 128;       // queries per CTA block, keys per inner block
constexpr int kHd = 64;         // head dimension
constexpr int kTile = kBlk * kHd * 2;   // bytes of a [128 x 64] bf16 tile: 16 KiB

struct AttnDev {
  __nv_bfloat16* o;        // [B, S, H, 64]
  float* lse;              // [B, H, S]  log2-domain log-sum-exp: m + log2(l)
  int S, H;
  float scale_log2;        // softmax scale * log2(e)
  int* err;
};

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a [rows x 64] bf16 tile stored the way a TMA load with
// the 128-byte swizzle stores it: rows of 128 bytes, 8-row groups of 1024 bytes, chunk index XORed with the row.
__device__ __forceinline__ uint32_t sw128_offset(int r, int c) {
  return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  tc::tmem_ld_32x32(taddr, r);
  tc::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ------------------------------------------------------------------ forward --
__global__ void __launch_bounds__(128) attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, AttnDev a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                       // 16 KiB
  uint8_t* sK = sQ + kTile;                 // 16 KiB: K_j is dead once S_j is in tensor memory, so one buffer will do
  uint8_t* sV = sK + kTile;                 // 2 x 16 KiB
  uint8_t* sP = sV + 2 * kTile;             // 32 KiB: two [128 x 64] sub-tiles
  uint64_t* q_full = reinterpret_cast<uint64_t*>(sP + 2 * kTile);
  uint64_t* k_full = q_full + 1;
  uint64_t* v_full = k_full + 1;            // [2]
  uint64_t* mma_bar = v_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 1);
  volatile int* bad = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5;
  const int nblk = a.S / kBlk;
  const int qi = nblk - 1 - static_cast<int>(blockIdx.x);   // long rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int HD = a.H * kHd;
  if (tid == 0) {
    tc::mbar_init(q_full, 1);
    tc::mbar_init(k_full, 1);
    tc::mbar_init(&v_full[0], 1);
    tc::mbar_init(&v_full[1], 1);
    tc::mbar_init(mma_bar, 1);
    *bad = 0;
    tc::mbar_init_fence();
    tc::tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 0) tc::tmem_alloc(tmem_slot, 256);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + 128;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  pdl_wait();

  const int row0 = b * a.S;
  auto load_k = [&](int j) {
    tc::mbar_expect_tx(k_full, kTile);
    tc::tma_load_2d(sK, &tm_qkv, k_full, HD + h * kHd, row0 + j * kBlk);
  };
  auto load_v = [&](int j) {
    const int st = j & 1;
    tc::mbar_expect_tx(&v_full[st], kTile);
    tc::tma_load_2d(sV + st * kTile, &tm_qkv, &v_full[st], 2 * HD + h * kHd, row0 + j * kBlk);
  };
  if (tid == 0) {
    tc::mbar_expect_tx(q_full, kTile);
    tc::tma_load_2d(sQ, &tm_qkv, q_full, h * kHd, row0 + qi * kBlk);
    load_k(0);
    load_v(0);
    if (qi >= 1) load_v(1);
  }

  float m_run = -INFINITY, l_run = 0.f;
  float o_acc[kHd];
#pragma unroll
  for (int d = 0; d < kHd; ++d) o_acc[d] = 0.f;
  uint32_t mma_phase = 0;
  const int q_row = qi * kBlk + tid;   // this thread's query index inside the sequence
  bool ok = true;

  for (int j = 0; j <= qi && ok; ++j) {
    const int st = j & 1;
    if (tid == 0) {
      bool w = true;
      if (j == 0) w = tc::mbar_wait(q_full, 0);
      w = w && tc::mbar_wait(k_full, j & 1);
      if (!w) *bad = 1;
      tc::fence_after_sync();
      if (w) {
        constexpr uint32_t idesc = tc::idesc_bf16(kBlk, kBlk, false, false);
        const uint64_t da = tc::smem_desc_k_sw128(sQ), db = tc::smem_desc_k_sw128(sK);
#pragma unroll
        for (int k4 = 0; k4 < kHd / UMMA_K; ++k4) tc::mma_bf16(tmem_s, da + 2 * k4, db + 2 * k4, idesc, k4 != 0);
      }
      tc::mma_commit(mma_bar);   // also on the failure path: releases the waiters below
    }
    ok = tc::mbar_wait(mma_bar, mma_phase) && *bad == 0;
    mma_phase ^= 1u;
    tc::fence_after_sync();
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ok = false;
      break;
    }
    if (tid == 0 && j + 1 <= qi) load_k(j + 1);   // S_j is in tensor memory: the K buffer is free again
    // pass 1: row maximum of the (masked) scores
    const bool diag = j == qi;
    float mx = -INFINITY;
#pragma unroll 1
    for (int c0 = 0; c0 < kBlk; c0 += 32) {
      float s[32];
      tmem_ld32(tmem_s + lane_base + static_cast<uint32_t>(c0), s);
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const bool masked = diag && (j * kBlk + c0 + e > q_row);
        mx = masked ? mx : fmaxf(mx, s[e]);
      }
    }
    const float m_new = fmaxf(m_run, mx * a.scale_log2);
    const float alpha = exp2f(m_run - m_new);   // 0 on the first block (m_run = -inf)
    // pass 2: probabilities, their sum, and P as the A operand of the next product
    float rs = 0.f;
#pragma unroll 1
    for (int c0 = 0; c0 < kBlk; c0 += 32) {
      float s[32];
      tmem_ld32(tmem_s + lane_base + static_cast<uint32_t>(c0), s);
      uint8_t* sub = sP + (c0 >> 6) * kTile;
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        uint4 pk;
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
          float p[2];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int e = c8 * 8 + e2 * 2 + q;
            const bool masked = diag && (j * kBlk + c0 + e > q_row);
            p[q] = masked ? 0.f : exp2f(s[e] * a.scale_log2 - m_new);
          }
          hp[e2] = __floats2bfloat162_rn(p[0], p[1]);
          // the sum uses the rounded values: they are what multiplies V
          const float2 back = __bfloat1622float2(hp[e2]);
          rs += back.x + back.y;
        }
        *reinterpret_cast<uint4*>(sub + sw128_offset(tid, ((c0 & 63) >> 3) + c8)) = pk;
      }
    }
    l_run = l_run * alpha + rs;
    m_run = m_new;
    fence_async_smem();          // the MMA reads P through the async proxy
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      const bool w = tc::mbar_wait(&v_full[st], (j >> 1) & 1);
      if (!w) *bad = 1;
      tc::fence_after_sync();
      if (w) {
        constexpr uint32_t idesc = tc::idesc_bf16(kBlk, kHd, false, true);
        const uint64_t dv = tc::smem_desc_mn_sw128(sV + st * kTile, kTile);
#pragma unroll
        for (int kk = 0; kk < kBlk / UMMA_K; ++kk) {
          const uint64_t dp = tc::smem_desc_k_sw128(sP + (kk >> 2) * kTile) + 2 * (kk & 3);
          tc::mma_bf16(tmem_o, dp, dv + 128 * kk, idesc, kk != 0);
        }
      }
      tc::mma_commit(mma_bar);
    }
    ok = tc::mbar_wait(mma_bar, mma_phase) && *bad == 0;
    mma_phase ^= 1u;
    tc::fence_after_sync();
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ok = false;
      break;
    }
    // this key block's contribution, folded into the running output
#pragma unroll
    for (int c0 = 0; c0 < kHd; c0 += 32) {
      float t[32];
      tmem_ld32(tmem_o + lane_base + static_cast<uint32_t>(c0), t);
#pragma unroll
      for (int e = 0; e < 32; ++e) o_acc[c0 + e] = o_acc[c0 + e] * alpha + t[e];
    }
    tc::fence_before_sync();
    __syncthreads();   // everybody has read S and O: the stage and both accumulators may be reused
    if (tid == 0 && j + 2 <= qi) load_v(j + 2);
  }

  if (ok) {
    const float inv = 1.f / l_run;
    __nv_bfloat16* orow = a.o + (static_cast<size_t>(row0 + q_row) * a.H + h) * kHd;
#pragma unroll
    for (int c8 = 0; c8 < kHd / 8; ++c8) {
      uint4 pk;
      __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int e2 = 0; e2 < 4; ++e2) hp[e2] = __floats2bfloat162_rn(o_acc[c8 * 8 + 2 * e2] * inv, o_acc[c8 * 8 + 2 * e2 + 1] * inv);
      reinterpret_cast<uint4*>(orow)[c8] = pk;
    }
    a.lse[(static_cast<size_t>(b) * a.H + h) * a.S + q_row] = m_run + log2f(l_run);
  } else if (tid == 0) {
    atomicExch(a.err, 11);
    // loads that were issued must land before the CTA retires
    tc::mbar_wait(q_full, 0, 1u << 20);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_s, 256);
  }
}

constexpr int kFwdSmem = 6 * kTile + 64 + 1024;   // 97 KiB: two CTAs per SM

// ----------------------------------------------------------------- backward --
struct AttnBwdDev {
  const __nv_bfloat16* o;    // [B, S, H, 64]
  const __nv_bfloat16* d_o;  // [B, S, H, 64]
  const float* lse;          // [B, H, S], log2 domain
  __nv_bfloat16* dqkv;       // [B, S, 3, H, 64]
  int S, H;
  float scale, scale_log2;
  int* err;
};

// One CTA per (batch, head); the sequence is one or two blocks of 128 (S = 128 or 256).  Tensor memory, 512 columns:
//   [0,128) dQ_0, dQ_1   [128,256) dK_0, dK_1   [256,384) dV_0, dV_1   [384,512) scratch: S, then dP
__global__ void __launch_bounds__(128) attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv,
                                                       const __grid_constant__ CUtensorMap tm_do, AttnBwdDev a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                 // [2] x 16 KiB
  uint8_t* sK = sQ + 2 * kTile;       // [2]
  uint8_t* sV = sK + 2 * kTile;       // [2]
  uint8_t* sDO = sV + 2 * kTile;      // [2]
  uint8_t* sP = sDO + 2 * kTile;      // 32 KiB
  uint8_t* sDS = sP + 2 * kTile;      // 32 KiB
  uint64_t* in_full = reinterpret_cast<uint64_t*>(sDS + 2 * kTile);
  uint64_t* mma_bar = in_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 1);
  volatile int* bad = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5;
  const int nblk = a.S / kBlk;   // 1 or 2
  const int h = blockIdx.x, b = blockIdx.y;
  const int HD = a.H * kHd;
  if (tid == 0) {
    tc::mbar_init(in_full, 1);
    tc::mbar_init(mma_bar, 1);
    *bad = 0;
    tc::mbar_init_fence();
    tc::tma_prefetch_desc(&tm_qkv);
    tc::tma_prefetch_desc(&tm_do);
  }
  if (warp == 0) tc::tmem_alloc(tmem_slot, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem0 = *tmem_slot;
  const uint32_t tm_dq = tmem0, tm_dk = tmem0 + 128, tm_dv = tmem0 + 256, tm_sc = tmem0 + 384;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  pdl_wait();

  const int row0 = b * a.S;
  if (tid == 0) {
    tc::mbar_expect_tx(in_full, static_cast<uint32_t>(4 * nblk * kTile));
    for (int i = 0; i < nblk; ++i) {
      tc::tma_load_2d(sQ + i * kTile, &tm_qkv, in_full, h * kHd, row0 + i * kBlk);
      tc::tma_load_2d(sK + i * kTile, &tm_qkv, in_full, HD + h * kHd, row0 + i * kBlk);
      tc::tma_load_2d(sV + i * kTile, &tm_qkv, in_full, 2 * HD + h * kHd, row0 + i * kBlk);
      tc::tma_load_2d(sDO + i * kTile, &tm_do, in_full, h * kHd, row0 + i * kBlk);
    }
  }
  // delta_i[row] = sum_d dO[row, d] * O[row, d] and the row's log-sum-exp, one row per thread and block
  float delta[2] = {0.f, 0.f}, lse[2] = {0.f, 0.f};
  for (int i = 0; i < nblk; ++i) {
    const size_t r = static_cast<size_t>(row0 + i * kBlk + tid);
    const uint4* po = reinterpret_cast<const uint4*>(a.o + (r * a.H + h) * kHd);
    const uint4* pd = reinterpret_cast<const uint4*>(a.d_o + (r * a.H + h) * kHd);
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < kHd / 8; ++c) {
      const uint4 vo = po[c], vd = pd[c];
      const __nv_bfloat162* ho = reinterpret_cast<const __nv_bfloat162*>(&vo);
      const __nv_bfloat162* hd = reinterpret_cast<const __nv_bfloat162*>(&vd);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __bfloat1622float2(ho[e]), y = __bfloat1622float2(hd[e]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
    delta[i] = acc;
    lse[i] = a.lse[(static_cast<size_t>(b) * a.H + h) * a.S + i * kBlk + tid];
  }

  uint32_t mma_phase = 0;
  bool ok = true;
  auto wait_mma = [&]() -> bool {
    bool w = tc::mbar_wait(mma_bar, mma_phase) && *bad == 0;
    mma_phase ^= 1u;
    tc::fence_after_sync();
    return __syncthreads_and(w ? 1 : 0) != 0;
  };
  constexpr uint32_t idesc_qk = tc::idesc_bf16(kBlk, kBlk, false, false);    // S, dP: both operands K-major
  constexpr uint32_t idesc_tt = tc::idesc_bf16(kBlk, kHd, true, true);       // dV, dK: A transposed (MN-major), B MN-major
  constexpr uint32_t idesc_nt = tc::idesc_bf16(kBlk, kHd, false, true);      // dQ: A K-major, B MN-major

  bool first = true;
  for (int i = 0; i < nblk && ok; ++i) {
    for (int j = 0; j <= i && ok; ++j) {
      const bool diag = i == j;
      // ---- S = Q_i K_j^T
      if (tid == 0) {
        bool w = true;
        if (first) w = tc::mbar_wait(in_full, 0);
        if (!w) *bad = 1;
        tc::fence_after_sync();
        if (w) {
          const uint64_t da = tc::smem_desc_k_sw128(sQ + i * kTile), db = tc::smem_desc_k_sw128(sK + j * kTile);
#pragma unroll
          for (int k4 = 0; k4 < kHd / UMMA_K; ++k4) tc::mma_bf16(tm_sc, da + 2 * k4, db + 2 * k4, idesc_qk, k4 != 0);
        }
        tc::mma_commit(mma_bar);   // completes after every earlier product too: P and dS may be overwritten below
      }
      first = false;
      if (!wait_mma()) {
        ok = false;
        break;
      }
      // ---- P = exp2(S c - L_i), written as bf16 for the products that follow
#pragma unroll 1
      for (int c0 = 0; c0 < kBlk; c0 += 32) {
        float s[32];
        tmem_ld32(tm_sc + lane_base + static_cast<uint32_t>(c0), s);
        uint8_t* sub = sP + (c0 >> 6) * kTile;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint4 pk;
          __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            float p[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int e = c8 * 8 + e2 * 2 + q;
              const bool masked = diag && (c0 + e > tid);
              p[q] = masked ? 0.f : exp2f(s[e] * a.scale_log2 - lse[i]);
            }
            hp[e2] = __floats2bfloat162_rn(p[0], p[1]);
          }
          *reinterpret_cast<uint4*>(sub + sw128_offset(tid, ((c0 & 63) >> 3) + c8)) = pk;
        }
      }
      fence_async_smem();
      tc::fence_before_sync();
      __syncthreads();   // P is complete, and nobody reads the scratch columns any more
      // ---- dP = dO_i V_j^T into the scratch columns; dV_j += P^T dO_i
      if (tid == 0) {
        tc::fence_after_sync();
        const uint64_t da = tc::smem_desc_k_sw128(sDO + i * kTile), db = tc::smem_desc_k_sw128(sV + j * kTile);
#pragma unroll
        for (int k4 = 0; k4 < kHd / UMMA_K; ++k4) tc::mma_bf16(tm_sc, da + 2 * k4, db + 2 * k4, idesc_qk, k4 != 0);
        const uint64_t dpt = tc::smem_desc_mn_sw128(sP, kTile), ddo = tc::smem_desc_mn_sw128(sDO + i * kTile, kTile);
#pragma unroll
        for (int kk = 0; kk < kBlk / UMMA_K; ++kk)
          tc::mma_bf16(tm_dv + static_cast<uint32_t>(j * kHd), dpt + 128 * kk, ddo + 128 * kk, idesc_tt, (kk != 0) || !diag);
        tc::mma_commit(mma_bar);
      }
      if (!wait_mma()) {
        ok = false;
        break;
      }
      // ---- dS = P (dP - delta_i) c
#pragma unroll 1
      for (int c0 = 0; c0 < kBlk; c0 += 32) {
        float dp[32];
        tmem_ld32(tm_sc + lane_base + static_cast<uint32_t>(c0), dp);
        const uint8_t* psub = sP + (c0 >> 6) * kTile;
        uint8_t* dsub = sDS + (c0 >> 6) * kTile;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          const uint32_t off = sw128_offset(tid, ((c0 & 63) >> 3) + c8);
          const uint4 pv = *reinterpret_cast<const uint4*>(psub + off);
          const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&pv);
          uint4 pk;
          __nv_bfloat162* hs = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            const float2 p = __bfloat1622float2(hp[e2]);
            const int e = c8 * 8 + e2 * 2;
            hs[e2] = __floats2bfloat162_rn(p.x * (dp[e] - delta[i]) * a.scale, p.y * (dp[e + 1] - delta[i]) * a.scale);
          }
          *reinterpret_cast<uint4*>(dsub + off) = pk;
        }
      }
      fence_async_smem();
      tc::fence_before_sync();
      __syncthreads();
      // ---- dK_j += dS^T Q_i ; dQ_i += dS K_j
      if (tid == 0) {
        tc::fence_after_sync();
        const uint64_t dst = tc::smem_desc_mn_sw128(sDS, kTile), dq = tc::smem_desc_mn_sw128(sQ + i * kTile, kTile);
#pragma unroll
        for (int kk = 0; kk < kBlk / UMMA_K; ++kk)
          tc::mma_bf16(tm_dk + static_cast<uint32_t>(j * kHd), dst + 128 * kk, dq + 128 * kk, idesc_tt, (kk != 0) || !diag);
        const uint64_t dk = tc::smem_desc_mn_sw128(sK + j * kTile, kTile);
#pragma unroll
        for (int kk = 0; kk < kBlk / UMMA_K; ++kk) {
          const uint64_t dsn = tc::smem_desc_k_sw128(sDS + (kk >> 2) * kTile) + 2 * (kk & 3);
          tc::mma_bf16(tm_dq + static_cast<uint32_t>(i * kHd), dsn, dk + 128 * kk, idesc_nt, (kk != 0) || (j != 0));
        }
        // no commit here: the next block pair's first commit (or the final one) covers these products
      }
    }
  }
  if (tid == 0) tc::mma_commit(mma_bar);
  ok = wait_mma() && ok;

  if (ok) {
    // gradients out of tensor memory, one row per thread, straight into the [B, S, 3, H, 64] gradient of qkv
    for (int t = 0; t < 3; ++t) {          // 0: dQ, 1: dK, 2: dV
      const uint32_t base = t == 0 ? tm_dq : (t == 1 ? tm_dk : tm_dv);
      for (int i = 0; i < nblk; ++i) {
        __nv_bfloat16* grow = a.dqkv + ((static_cast<size_t>(row0 + i * kBlk + tid) * 3 + t) * a.H + h) * kHd;
#pragma unroll
        for (int c0 = 0; c0 < kHd; c0 += 32) {
          float v[32];
          tmem_ld32(base + static_cast<uint32_t>(i * kHd) + lane_base + static_cast<uint32_t>(c0), v);
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            uint4 pk;
            __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) hp[e2] = __floats2bfloat162_rn(v[c8 * 8 + 2 * e2], v[c8 * 8 + 2 * e2 + 1]);
            reinterpret_cast<uint4*>(grow)[(c0 >> 3) + c8] = pk;
          }
        }
      }
    }
  } else if (tid == 0) {
    atomicExch(a.err, 12);
    tc::mbar_wait(in_full, 0, 1u << 20);   // the loads that were issued must land before the CTA retires
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem0, 512);
  }
}

constexpr int kBwdSmem = 12 * kTile + 64 + 1024;   // 193 KiB

}  // namespace

cudaError_t attention_bwd(const __nv_bfloat16* qkv, const __nv_bfloat16* o, const __nv_bfloat16* d_o, const float* lse,
                          __nv_bfloat16* dqkv, int B, int S, int H, float softmax_scale, cudaStream_t stream) {
  if ((S != kBlk && S != 2 * kBlk) || B <= 0 || H <= 0) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o) |
       reinterpret_cast<uintptr_t>(dqkv)) & 15u)
    return cudaErrorNotSupported;
  static bool configured = false;
  if (!configured) {
    cudaError_t rc = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (rc != cudaSuccess) return rc;
    configured = true;
  }
  CUtensorMap tq, tdo;
  if (!encode_map(&tq, qkv, B * S, 3 * H * kHd, 3 * H * kHd, kBlk)) return cudaErrorNotSupported;
  if (!encode_map(&tdo, d_o, B * S, H * kHd, H * kHd, kBlk)) return cudaErrorNotSupported;
  (void)cudaGetLastError();
  AttnBwdDev a;
  a.o = o;
  a.d_o = d_o;
  a.lse = lse;
  a.dqkv = dqkv;
  a.S = S;
  a.H = H;
  a.scale = softmax_scale;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.err = gemm_error_device_ptr();
  if (!a.err) return cudaErrorNotSupported;
  MCCL_LAUNCH_PDL(attn_bwd_kernel, dim3(H, B), 128, kBwdSmem, stream, tq, tdo, a);
  count_launch();
  return launch_status();
}

cudaError_t attention_fwd(const __nv_bfloat16* qkv, __nv_bfloat16* o, float* lse, int B, int S, int H, float softmax_scale,
                          cudaStream_t stream) {
  if (S % kBlk != 0 || S <= 0 || B <= 0 || H <= 0) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(o)) & 15u) return cudaErrorNotSupported;
  static bool configured = false;
  if (!configured) {
    cudaError_t rc = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (rc != cudaSuccess) return rc;
    configured = true;
  }
  CUtensorMap tm;
  if (!encode_map(&tm, qkv, B * S, 3 * H * kHd, 3 * H * kHd, kBlk)) return cudaErrorNotSupported;
  (void)cudaGetLastError();
  AttnDev a;
  a.o = o;
  a.lse = lse;
  a.S = S;
  a.H = H;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.err = gemm_error_device_ptr();
  if (!a.err) return cudaErrorNotSupported;
  MCCL_LAUNCH_PDL(attn_fwd_kernel, dim3(S / kBlk, H, B), 128, kFwdSmem, stream, tm, a);
  count_launch();
  return launch_status();
}

}  // namespace ops
}  // namespace mccl
