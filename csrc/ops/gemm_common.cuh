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


__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678f)); }

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
    // value and derivative share the erf; the derivative is what backward needs, so it is saved instead of z
    float dv[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float x = v[j];
      const float cdf = 0.5f * (1.f + erff(x * 0.70710678f));
      dv[j] = cdf + x * 0.39894228f * __expf(-0.5f * x * x);
      v[j] = x * cdf;
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
