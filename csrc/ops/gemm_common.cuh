// Pieces shared by the GEMM kernels: tile constants, the device-side argument
// block, the epilogue (bias / GELU / residual / bf16 or fp32 store) and the TMA
// descriptor encoder.
#pragma once

#include "ops.hpp"
#include "tcgen05.cuh"

#include "../core/timeline.hpp"
#include "../symm/cu_driver.hpp"

namespace mccl {
namespace ops {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;      // bf16 MMA consumes 32 bytes of K per instruction

struct GemmDev {
  void* d;
  __nv_bfloat16* aux;
  const float* bias;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* mul;       // when set: D = acc * mul, e.g. the backward of a GELU (mul = saved gelu'(z)) fused into the producing GEMM
  int m, n, k;
  int ldd;
  int d_fp32;
  int accumulate;
  int epilogue;
  int atomic_add;  // fp32 output accumulated with red.global.add (split-K partial sums)
  int* err;  // device word set non-zero when a pipeline wait runs out
  TimelineBuf* tl;  // device timeline, or nullptr (off)
};

// Device address of the error word (one per process and device context).
int* gemm_error_device_ptr();


// GELU (erf form) and its derivative from one exponential.  With u = |x| / sqrt(2) and E = exp(-u^2) = exp(-x^2 / 2),
// erf(u) = 1 - (a1 t + ... + a5 t^5) E, t = 1 / (1 + p u), to 1.5e-7 absolute (Abramowitz & Stegun 7.1.26): far below
// what a bf16 output resolves, and E is the exponential the normal density of the derivative needs anyway.
__device__ __forceinline__ void gelu_value_grad(float x, float& value, float& grad) {
  const float u = fabsf(x) * 0.70710678f;
  const float e = __expf(-0.5f * x * x);
  const float t = __fdividef(1.f, fmaf(0.3275911f, u, 1.f));
  const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
  const float cdf = 0.5f * (1.f + copysignf(1.f - poly * e, x));
  value = x * cdf;
  grad = fmaf(x * 0.39894228f, e, cdf);
}

__device__ __forceinline__ float gelu_erf(float x) {
  float v, d;
  gelu_value_grad(x, v, d);
  return v;
}

// Finishes 32 consecutive accumulator columns [col0, col0 + 32) of one output
// row: r holds the raw fp32 bits read from tensor memory.
__device__ __forceinline__ void epilogue_store(const GemmDev& g, int row, int col0, const uint32_t (&r)[32]) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  const int ncols = (g.n - col0) < 32 ? (g.n - col0) : 32;  // multiple of 8
  if (g.epilogue == EPI_BIAS || g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_BIAS_GELU_D) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) v[j] += __ldg(g.bias + col0 + j);
  }
  if (g.epilogue == EPI_BIAS_GELU_D || g.epilogue == EPI_GELU_D) {
    // value and derivative share one exponential; the derivative is what backward needs, so it is saved instead of z
    float dv[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      gelu_value_grad(v[j], v[j], dv[j]);
    }
    __nv_bfloat16* arow = g.aux + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      if (j8 * 8 < ncols) {
        uint4 pk;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(dv[j8 * 8 + 2 * i], dv[j8 * 8 + 2 * i + 1]);
        *reinterpret_cast<uint4*>(arow + j8 * 8) = pk;
      }
    }
  }
  if (g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_GELU) {
    __nv_bfloat16* zrow = g.aux + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      if (j8 * 8 < ncols) {
        uint4 pk;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[j8 * 8 + 2 * i], v[j8 * 8 + 2 * i + 1]);
        *reinterpret_cast<uint4*>(zrow + j8 * 8) = pk;
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
  }
  if (g.mul) {
    const __nv_bfloat16* mrow = g.mul + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      if (j8 * 8 < ncols) {
        const uint4 pk = *reinterpret_cast<const uint4*>(mrow + j8 * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = __bfloat1622float2(h[i]);
          v[j8 * 8 + 2 * i] *= t.x;
          v[j8 * 8 + 2 * i + 1] *= t.y;
        }
      }
    }
  }
  if (g.residual) {
    const __nv_bfloat16* rrow = g.residual + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      if (j8 * 8 < ncols) {
        const uint4 pk = *reinterpret_cast<const uint4*>(rrow + j8 * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = __bfloat1622float2(h[i]);
          v[j8 * 8 + 2 * i] += t.x;
          v[j8 * 8 + 2 * i + 1] += t.y;
        }
      }
    }
  }
  if (g.d_fp32) {
    float* drow = static_cast<float*>(g.d) + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
      if (j4 * 4 < ncols) {
        float4 o = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
        if (g.atomic_add) {
          atomicAdd(reinterpret_cast<float4*>(drow + j4 * 4), o);
          continue;
        }
        if (g.accumulate) {
          const float4 old = *reinterpret_cast<const float4*>(drow + j4 * 4);
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        *reinterpret_cast<float4*>(drow + j4 * 4) = o;
      }
    }
  } else {
    __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(g.d) + static_cast<size_t>(row) * g.ldd + col0;
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      if (j8 * 8 < ncols) {
        uint4 pk;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[j8 * 8 + 2 * i], v[j8 * 8 + 2 * i + 1]);
        *reinterpret_cast<uint4*>(drow + j8 * 8) = pk;
      }
    }
  }
}

// ---- epilogue through shared memory ------------------------------------------------------------------------------------
// Two measured facts shape this code.  (1) A thread owns one accumulator row (that is how tensor memory is read), so
// storing straight from registers makes every warp-wide store touch 32 different 128-byte lines.  Each epilogue warp
// therefore owns a 4 KB staging buffer of 32 rows x 128 bytes: a thread writes its row there, and the warp then moves
// the buffer to global memory with several lanes per row, whole lines (or half lines) at a time; inputs that have the
// layout of the output (gelu' multiplier, residual) come in the same way.  16-byte units are XOR-swizzled by the row
// index so that both access patterns are free of bank conflicts.  (2) A CTA runs the epilogue of one or two tiles, so
// straight-line code is executed once and every instruction is an instruction-cache miss: with the epilogue fully
// unrolled, `no_instruction` was the top warp stall, and unrolling 32 columns per trip instead of 8 made the training
// step 5 % slower.  The loops below are kept rolled (8 columns per trip) so that their instructions are fetched once.
__device__ __forceinline__ uint4* stage_unit(uint8_t* stage, int r, int u) {
  return reinterpret_cast<uint4*>(stage + r * 128 + ((u ^ (r & 7)) << 4));
}

// Staging <-> global for `upr` (8 or 4) 16-byte units per row, starting at unit `u0` of the staging rows; the global
// side is rows [row0, row0 + 32) of a row-major matrix with `ldb` bytes per row, at byte offset `colb`.  `valid` units
// of a row lie inside the matrix.
__device__ __forceinline__ void stage_load(uint8_t* stage, const void* src, size_t ldb, size_t colb, int row0, int m, int upr, int valid, int lane) {
  __syncwarp();
  const int u = lane & (upr - 1), rsub = lane / upr, rows_per_trip = 32 / upr;
#pragma unroll 1
  for (int r = rsub; r < 32; r += rows_per_trip) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + r < m && u < valid)
      v = *reinterpret_cast<const uint4*>(static_cast<const char*>(src) + static_cast<size_t>(row0 + r) * ldb + colb + u * 16);
    *stage_unit(stage, r, u) = v;
  }
  __syncwarp();
}

__device__ __forceinline__ void stage_flush(uint8_t* stage, int u0, void* dst, size_t ldb, size_t colb, int row0, int m, int upr, int valid, int lane) {
  __syncwarp();
  const int u = lane & (upr - 1), rsub = lane / upr, rows_per_trip = 32 / upr;
#pragma unroll 1
  for (int r = rsub; r < 32; r += rows_per_trip) {
    if (row0 + r < m && u < valid)
      *reinterpret_cast<uint4*>(static_cast<char*>(dst) + static_cast<size_t>(row0 + r) * ldb + colb + u * 16) = *stage_unit(stage, r, u0 + u);
  }
  __syncwarp();
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 pk;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return pk;
}

__device__ __forceinline__ void add_bias8(const GemmDev& g, int col, float (&v)[8]) {
  if ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0) {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(g.bias + col)), b1 = __ldg(reinterpret_cast<const float4*>(g.bias + col) + 1);
    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
    v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += __ldg(g.bias + col + j);
  }
}

__device__ __forceinline__ void apply8(const uint4& pk, bool multiply, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    if (multiply) {
      v[2 * i] *= t.x;
      v[2 * i + 1] *= t.y;
    } else {
      v[2 * i] += t.x;
      v[2 * i + 1] += t.y;
    }
  }
}

// Finishes `ncols` (a multiple of 64) accumulator columns of this warp's 32 rows, bf16 output.  `taddr` is the tensor-
// memory address of the first column in this warp's lanes, `col0` its column in the matrix.  Calls last_read() right
// after the last tensor-memory read, so that the accumulator can be handed back early.
template <typename F>
__device__ __forceinline__ void epilogue_bf16(const GemmDev& g, uint8_t* stage, uint32_t taddr, int row0, int col0, int ncols, int lane, F&& last_read) {
  const bool has_bias = g.epilogue == EPI_BIAS || g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_BIAS_GELU_D;
  const bool gelu_d = g.epilogue == EPI_BIAS_GELU_D || g.epilogue == EPI_GELU_D;
  const bool gelu_z = g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_GELU;
  const bool two_out = gelu_d || gelu_z;
  // with a second output the staging row holds 32 columns of each (units 0-3: D, units 4-7: aux), otherwise 64 of D
  const int upr = two_out ? 4 : 8, gcols = upr * 8;
  const size_t ldb = static_cast<size_t>(g.ldd) * 2;
  const __nv_bfloat16* staged_in = g.mul ? g.mul : g.residual;
  const bool direct_residual = g.mul != nullptr && g.residual != nullptr;
  const int row = row0 + lane;
  const bool rows_ok = row0 < g.m;
#pragma unroll 1
  for (int c = 0; c < ncols; c += gcols) {
    const int cg = col0 + c;
    const int left = (g.n - cg) >> 3;
    const int valid = left < upr ? (left < 0 ? 0 : left) : upr;
    const bool active = rows_ok && valid > 0;
    const size_t colb = static_cast<size_t>(cg) * 2;
    if (active && staged_in) stage_load(stage, staged_in, ldb, colb, row0, g.m, upr, valid, lane);
#pragma unroll 1
    for (int u = 0; u < upr; ++u) {
      uint32_t r[8];
      tc::tmem_ld_32x8(taddr + static_cast<uint32_t>(c + u * 8), r);
      tc::tmem_ld_wait();
      if (c + gcols >= ncols && u + 1 == upr) last_read();
      if (!active || u >= valid) continue;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[j]);
      if (has_bias) add_bias8(g, cg + u * 8, v);
      if (gelu_d) {
        float dv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) gelu_value_grad(v[j], v[j], dv[j]);
        *stage_unit(stage, lane, 4 + u) = pack8(dv);
      } else if (gelu_z) {
        *stage_unit(stage, lane, 4 + u) = pack8(v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = gelu_erf(v[j]);
      }
      if (staged_in) apply8(*stage_unit(stage, lane, u), g.mul != nullptr, v);
      if (direct_residual && row < g.m)
        apply8(*reinterpret_cast<const uint4*>(g.residual + static_cast<size_t>(row) * g.ldd + cg + u * 8), false, v);
      *stage_unit(stage, lane, u) = pack8(v);   // the unit this thread has just consumed, in its own row
    }
    if (active) {
      stage_flush(stage, 0, g.d, ldb, colb, row0, g.m, upr, valid, lane);
      if (two_out) stage_flush(stage, 4, g.aux, ldb, colb, row0, g.m, upr, valid, lane);
    }
  }
}

// The same for an fp32 output (`ncols` a multiple of 32): plain store, read-add-store, or red.global.add.
template <typename F>
__device__ __forceinline__ void epilogue_fp32(const GemmDev& g, uint8_t* stage, uint32_t taddr, int row0, int col0, int ncols, int lane, F&& last_read) {
  const bool has_bias = g.epilogue == EPI_BIAS;
  const int row = row0 + lane;
  const bool rows_ok = row0 < g.m;
  float* d = static_cast<float*>(g.d);
#pragma unroll 1
  for (int c = 0; c < ncols; c += 32) {
    const int cg = col0 + c;
    const int left = (g.n - cg) >> 2;                          // 16-byte units (4 floats) inside the matrix
    const int valid = left < 8 ? (left < 0 ? 0 : left) : 8;
    const bool active = rows_ok && valid > 0;
#pragma unroll 1
    for (int u = 0; u < 8; u += 2) {
      uint32_t r[8];
      tc::tmem_ld_32x8(taddr + static_cast<uint32_t>(c + u * 4), r);
      tc::tmem_ld_wait();
      if (c + 32 >= ncols && u == 6) last_read();
      if (!active || u >= valid) continue;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[j]);
      if (has_bias) add_bias8(g, cg + u * 4, v);
      if (g.residual && row < g.m) apply8(*reinterpret_cast<const uint4*>(g.residual + static_cast<size_t>(row) * g.ldd + cg + u * 4), false, v);
      *reinterpret_cast<float4*>(stage_unit(stage, lane, u)) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(stage_unit(stage, lane, u + 1)) = make_float4(v[4], v[5], v[6], v[7]);
    }
    __syncwarp();
    if (active) {
      const int u = lane & 7;
#pragma unroll 1
      for (int rr = lane >> 3; rr < 32; rr += 4) {
        if (row0 + rr < g.m && u < valid) {
          float4 o = *reinterpret_cast<const float4*>(stage_unit(stage, rr, u));
          float4* p = reinterpret_cast<float4*>(d + static_cast<size_t>(row0 + rr) * g.ldd + cg + 4 * u);
          if (g.atomic_add) {
            atomicAdd(p, o);
          } else {
            if (g.accumulate) {
              const float4 old = *p;
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *p = o;
          }
        }
      }
    }
    __syncwarp();
  }
}

// K-major operand [rows = M or N, cols = K]: box = 64 (K) x box_rows.
// MN-major operand [rows = K, cols = M or N]: box = 64 (M/N) x 64 (K).
inline bool encode_map(CUtensorMap* map, const void* base, int rows, int cols, int ld_elems, int box_rows) {
  const CuDriver& cu = CuDriver::get();
  if (!cu.loaded || !cu.TensorMapEncodeTiled) return false;
  int device = 0;
  cudaGetDevice(&device);
  cu.ensure_context(device);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = cu.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}


}  // namespace ops
}  // namespace mccl
