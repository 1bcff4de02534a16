// Stand-alone element-wise kernels: dst ∘= src, buf *= s, dst = (dst+src)*s.
//
// These are the sm_100a counterparts of the reference's 18 Metal kernels
// (accumulate_chunk_*, elementwise_min/max/product_*, scale_inplace_*,
// accumulate_scale_*: csrc/metal/shaders.metal:196-552).  Inside the
// collectives the same arithmetic is fused into the kernel that moves the
// data; the stand-alone forms exist for the kernel unit tests and for callers
// that reduce two local buffers.  Grid-stride over 16-byte packs with a scalar
// path for unaligned pointers and the tail, mirroring the reference's
// vector / scalar split (shaders.metal:159-187).
#include "../core/launch.hpp"
#include "collectives.hpp"
#include "comm_device.cuh"

namespace mccl {
namespace dev {

namespace {

constexpr int kEwThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kEwThreads) reduce2_kernel(T* dst, const T* src, long long n, int op) {
  using Acc = typename Elem<T>::Acc;
  constexpr int E = 16 / sizeof(T);
  const bool al = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const long long packs = (n + E - 1) / E;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < packs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long left = n - i * E;
    const int nv = left >= E ? E : static_cast<int>(left);
    Acc a[E], b[E];
    load_pack<T, E, Acc>(dst + i * E, a, nv, al);
    load_pack<T, E, Acc>(src + i * E, b, nv, al);
#pragma unroll
    for (int e = 0; e < E; ++e) a[e] = apply_op<Acc>(op, a[e], b[e]);
    store_pack<T, E, Acc>(dst + i * E, a, nv, al);
  }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads) scale_kernel(T* buf, long long n, float scale) {
  using Acc = typename Elem<T>::Acc;
  constexpr int E = 16 / sizeof(T);
  const bool al = (reinterpret_cast<uintptr_t>(buf) & 15u) == 0;
  const long long packs = (n + E - 1) / E;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < packs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long left = n - i * E;
    const int nv = left >= E ? E : static_cast<int>(left);
    Acc a[E];
    load_pack<T, E, Acc>(buf + i * E, a, nv, al);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if constexpr (IsIntegral<Acc>::value) a[e] = static_cast<Acc>(llrintf(static_cast<float>(a[e]) * scale));
      else a[e] = a[e] * static_cast<Acc>(scale);
    }
    store_pack<T, E, Acc>(buf + i * E, a, nv, al);
  }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads) reduce2_scale_kernel(T* dst, const T* src, long long n, float scale) {
  using Acc = typename Elem<T>::Acc;
  constexpr int E = 16 / sizeof(T);
  const bool al = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const long long packs = (n + E - 1) / E;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < packs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long left = n - i * E;
    const int nv = left >= E ? E : static_cast<int>(left);
    Acc a[E], b[E];
    load_pack<T, E, Acc>(dst + i * E, a, nv, al);
    load_pack<T, E, Acc>(src + i * E, b, nv, al);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if constexpr (IsIntegral<Acc>::value) a[e] = static_cast<Acc>(llrintf(static_cast<float>(a[e] + b[e]) * scale));
      else a[e] = (a[e] + b[e]) * static_cast<Acc>(scale);
    }
    store_pack<T, E, Acc>(dst + i * E, a, nv, al);
  }
}

int grid_for(long long n, int elems_per_pack) {
  long long packs = (n + elems_per_pack - 1) / elems_per_pack;
  long long blocks = (packs + kEwThreads - 1) / kEwThreads;
  const long long cap = 148LL * 8;  // one wave of 8 resident CTAs per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

#define MCCL_EW_DISPATCH(t, CALL)                                 \
  switch (t) {                                                    \
    case ElemType::F32: { using T = float; CALL; } break;         \
    case ElemType::F16: { using T = __half; CALL; } break;        \
    case ElemType::BF16: { using T = __nv_bfloat16; CALL; } break;\
    case ElemType::F64: { using T = double; CALL; } break;        \
    case ElemType::I32: { using T = int32_t; CALL; } break;       \
    case ElemType::I64: { using T = int64_t; CALL; } break;       \
    default: return cudaErrorInvalidValue;                        \
  }

cudaError_t launch_reduce2(ElemType t, int op, void* dst, const void* src, long long n, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  MCCL_EW_DISPATCH(t, (MCCL_LAUNCH(reduce2_kernel<T>, grid_for(n, 16 / sizeof(T)), kEwThreads, 0, stream, 
                          static_cast<T*>(dst), static_cast<const T*>(src), n, op)));
  return ::mccl::launch_status();
}

cudaError_t launch_scale(ElemType t, void* buf, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  MCCL_EW_DISPATCH(t, (MCCL_LAUNCH(scale_kernel<T>, grid_for(n, 16 / sizeof(T)), kEwThreads, 0, stream, static_cast<T*>(buf), n, scale)));
  return ::mccl::launch_status();
}

cudaError_t launch_reduce2_scale(ElemType t, void* dst, const void* src, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  MCCL_EW_DISPATCH(t, (MCCL_LAUNCH(reduce2_scale_kernel<T>, grid_for(n, 16 / sizeof(T)), kEwThreads, 0, stream, 
                          static_cast<T*>(dst), static_cast<const T*>(src), n, scale)));
  return ::mccl::launch_status();
}

}  // namespace dev
}  // namespace mccl
