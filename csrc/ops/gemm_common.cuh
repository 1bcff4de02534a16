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
// Three measured facts shape this code.
// (1) A thread owns one accumulator row (that is how tensor memory is read), so storing straight from registers makes
//     every warp-wide store touch 32 different 128-byte lines.
// (2) A CTA runs the epilogue of one or two tiles, so straight-line code is executed once and every instruction is an
//     instruction-cache miss: with the epilogue fully unrolled, `no_instruction` was the top warp stall, and unrolling
//     32 columns of epilogue math per trip instead of 8 made the training step 5 % slower.
// (3) A tensor-memory read takes about 500 clocks before tcgen05.wait::ld returns: reading 8 columns per trip of a
//     rolled loop cost 0.4 us per trip (3.4 us for a 128 x 128 tile) even with the next read in flight.
// So: each epilogue warp reads 32 columns of its 32 rows at once (the next 32 are requested before these are used),
// parks the raw fp32 values in a 4 KB staging buffer of its own (32 rows x 128 bytes, 16-byte units XOR-swizzled by
// the row so that row-wise writes and unit-wise reads are both free of bank conflicts), and then finishes them in the
// transposed assignment: lane = (row mod 4, 4 columns), 8 rolled trips over the rows.  There bias is a register, the
// multiplier / residual loads and the output stores of 8 lanes cover 64 (bf16) or 128 (fp32) contiguous bytes of a
// row, and the loop body is a few dozen instructions that are fetched once.
__device__ __forceinline__ uint4* stage_unit(uint8_t* stage, int r, int u) {
  return reinterpret_cast<uint4*>(stage + r * 128 + ((u ^ (r & 7)) << 4));
}

__device__ __forceinline__ uint2 pack4(const float4& v) {
  uint2 pk;
  *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(v.z, v.w);
  return pk;
}
__device__ __forceinline__ float4 unpack4(const uint2& pk) {
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Finishes `ncols` (a multiple of 32) accumulator columns of this warp's 32 rows [row0, row0 + 32).  `taddr` is the
// tensor-memory address of the first column in this warp's lanes, `col0` its column in the matrix.  Calls last_read()
// right after the last tensor-memory read has landed, so that the accumulator can be handed back early.
template <typename F>
__device__ __forceinline__ void epilogue_tile(const GemmDev& g, uint8_t* stage, uint32_t taddr, int row0, int col0, int ncols, int lane, F&& last_read) {
  const bool has_bias = g.epilogue == EPI_BIAS || g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_BIAS_GELU_D;
  const bool gelu_d = g.epilogue == EPI_BIAS_GELU_D || g.epilogue == EPI_GELU_D;
  const bool gelu_z = g.epilogue == EPI_BIAS_GELU || g.epilogue == EPI_GELU;
  const int u = lane & 7, rsub = lane >> 3;   // transposed assignment: columns [4u, 4u + 4) of rows rsub, rsub + 4, ...
  uint32_t acc[32];
  tc::tmem_ld_32x32(taddr, acc);
#pragma unroll 1
  for (int c = 0; c < ncols; c += 32) {
    tc::tmem_ld_wait();
    __syncwarp();   // the previous group's reads of the staging buffer are done
#pragma unroll
    for (int j = 0; j < 8; ++j) *stage_unit(stage, lane, j) = make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    if (c + 32 < ncols) tc::tmem_ld_32x32(taddr + static_cast<uint32_t>(c + 32), acc);
    else last_read();
    __syncwarp();
    const int col = col0 + c + 4 * u;
    if (row0 >= g.m || col >= g.n) continue;   // N is a multiple of 8: a unit of 4 columns is inside or outside as a whole
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_bias) {
      if ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0) b = __ldg(reinterpret_cast<const float4*>(g.bias + col));
      else b = make_float4(__ldg(g.bias + col), __ldg(g.bias + col + 1), __ldg(g.bias + col + 2), __ldg(g.bias + col + 3));
    }
#pragma unroll 2
    for (int r = rsub; r < 32; r += 4) {
      const int row = row0 + r;
      if (row >= g.m) break;
      float4 v = *reinterpret_cast<const float4*>(stage_unit(stage, r, u));
      const size_t at = static_cast<size_t>(row) * g.ldd + col;
      v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      if (gelu_d) {
        float4 d;
        gelu_value_grad(v.x, v.x, d.x);
        gelu_value_grad(v.y, v.y, d.y);
        gelu_value_grad(v.z, v.z, d.z);
        gelu_value_grad(v.w, v.w, d.w);
        *reinterpret_cast<uint2*>(g.aux + at) = pack4(d);
      } else if (gelu_z) {
        *reinterpret_cast<uint2*>(g.aux + at) = pack4(v);
        v.x = gelu_erf(v.x); v.y = gelu_erf(v.y); v.z = gelu_erf(v.z); v.w = gelu_erf(v.w);
      }
      if (g.mul) {
        const float4 t = unpack4(*reinterpret_cast<const uint2*>(g.mul + at));
        v.x *= t.x; v.y *= t.y; v.z *= t.z; v.w *= t.w;
      }
      if (g.residual) {
        const float4 t = unpack4(*reinterpret_cast<const uint2*>(g.residual + at));
        v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
      }
      if (g.d_fp32) {
        float4* p = reinterpret_cast<float4*>(static_cast<float*>(g.d) + at);
        if (g.atomic_add) {
          atomicAdd(p, v);
        } else {
          if (g.accumulate) {
            const float4 old = *p;
            v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
          }
          *p = v;
        }
      } else {
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(g.d) + at) = pack4(v);
      }
    }
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

// Output matrix [rows, cols] (bf16, or fp32 when `fp32`) as the target of TMA stores of 32-row boxes whose rows are
// 128 bytes (64 bf16 or 32 fp32 columns), 128-byte swizzle: the layout of an epilogue warp's staging buffer.
inline bool encode_out_map(CUtensorMap* map, const void* base, int rows, int cols, int ld_elems, bool fp32) {
  const CuDriver& cu = CuDriver::get();
  if (!cu.loaded || !cu.TensorMapEncodeTiled) return false;
  int device = 0;
  cudaGetDevice(&device);
  cu.ensure_context(device);
  const int es = fp32 ? 4 : 2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), 32u};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = cu.TensorMapEncodeTiled(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

}  // namespace ops
}  // namespace mccl
