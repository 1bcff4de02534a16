// Memory-bound model operators: normalisation (forward / backward), fused
// AdamW, softmax cross entropy (forward + backward in one pass), transpose,
// casts and the GELU derivative.  Every kernel moves 16 bytes per access and
// reads each operand once from HBM (re-reads of a row hit L1/L2).
#include "../core/launch.hpp"
#include <atomic>

#include "ops.hpp"

namespace mccl {
namespace ops {

namespace {
std::atomic<uint64_t> g_launches{0};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}
}  // namespace

uint64_t launch_count() { return g_launches.load(); }
void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n)); }

// ------------------------------------------------------------------- norm --
// One warp per row; dim must be a multiple of 8.
template <bool kLayerNorm>
__global__ void __launch_bounds__(256) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                                       int dim, float eps) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(warp) * dim);
  const int vecs = dim >> 3;
  float sum = 0.f;
  for (int v = lane; v < vecs; v += 32) {
    float f[8];
    unpack8(xr[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) sum += f[i];
  }
  const float mean = kLayerNorm ? warp_sum(sum) / dim : 0.f;
  float sq = 0.f;
  for (int v = lane; v < vecs; v += 32) {
    float f[8];
    unpack8(xr[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) sq += (f[i] - mean) * (f[i] - mean);
  }
  const float rstd = rsqrtf(warp_sum(sq) / dim + eps);
  if (lane == 0) {
    mean_out[warp] = mean;
    rstd_out[warp] = rstd;
  }
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(warp) * dim);
  for (int v = lane; v < vecs; v += 32) {
    float f[8], o[8];
    unpack8(xr[v], f);
    const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float bb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (kLayerNorm) {
      const float4 b0 = reinterpret_cast<const float4*>(b)[2 * v], b1 = reinterpret_cast<const float4*>(b)[2 * v + 1];
      bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (f[i] - mean) * rstd * ww[i] + bb[i];
    yr[v] = pack8(o);
  }
}

template <bool kLayerNorm>
__global__ void __launch_bounds__(256) norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ w, const float* __restrict__ mean,
                                                          const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                                          const __nv_bfloat16* __restrict__ dx_add, int rows, int dim) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(warp) * dim);
  // optional: a second gradient of the same tensor (the residual path), added before the one rounding to bf16
  const uint4* ar = dx_add ? reinterpret_cast<const uint4*>(dx_add + static_cast<size_t>(warp) * dim) : nullptr;
  const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(warp) * dim);
  const int vecs = dim >> 3;
  const float mu = mean[warp], rs = rstd[warp];
  float c1 = 0.f, c2 = 0.f;  // sum(dy*w*xhat), sum(dy*w)
  for (int v = lane; v < vecs; v += 32) {
    float f[8], g[8];
    unpack8(xr[v], f);
    unpack8(gr[v], g);
    const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gw = g[i] * ww[i];
      c1 += gw * (f[i] - mu) * rs;
      c2 += gw;
    }
  }
  c1 = warp_sum(c1) / dim;
  c2 = kLayerNorm ? warp_sum(c2) / dim : 0.f;
  uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(warp) * dim);
  for (int v = lane; v < vecs; v += 32) {
    float f[8], g[8], o[8];
    unpack8(xr[v], f);
    unpack8(gr[v], g);
    const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = rs * (g[i] * ww[i] - c2 - (f[i] - mu) * rs * c1);
    if (ar != nullptr) {
      float a[8];
      unpack8(ar[v], a);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += a[i];
    }
    dr[v] = pack8(o);
  }
}

// Column reductions over the rows: dw[c] = sum_r dy[r,c] * xhat[r,c] and
// db[c] = sum_r dy[r,c] (kNorm), or just the column sum (bias gradients).
// Stage 1: a block of 32 x 8 threads covers 256 columns (8 per thread, one
// 16-byte load per row) and a slab of kSlabRows rows, and writes one partial
// row.  Stage 2 adds the partial rows in a fixed order, so the result does not
// depend on scheduling.
constexpr int kSlabRows = 64;

template <bool kNorm>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                             const float* __restrict__ mean, const float* __restrict__ rstd,
                                                             float* __restrict__ part_w, float* __restrict__ part_b, int rows,
                                                             int dim, int atomic) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  __shared__ float sw[8][32][9], sb[8][32][9];
  const int cg = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + cg * 8;
  const int r0 = blockIdx.y * kSlabRows;
  const int r1 = min(r0 + kSlabRows, rows);
  float aw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ab[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < dim) {
    for (int r = r0 + ry; r < r1; r += 8) {
      float g[8];
      unpack8(*reinterpret_cast<const uint4*>(dy + static_cast<size_t>(r) * dim + col), g);
      if (kNorm) {
        float xv[8];
        unpack8(*reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * dim + col), xv);
        const float mu = mean[r], rs = rstd[r];
#pragma unroll
        for (int i = 0; i < 8; ++i) aw[i] += g[i] * (xv[i] - mu) * rs;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ab[i] += g[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sw[ry][cg][i] = aw[i];
    sb[ry][cg][i] = ab[i];
  }
  __syncthreads();
  // 256 threads, 256 columns: thread t finishes column t of this block
  const int c = threadIdx.x, ccg = c >> 3, ci = c & 7;
  if (blockIdx.x * 256 + c < dim) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      tw += sw[k][ccg][ci];
      tb += sb[k][ccg][ci];
    }
    if (atomic) {
      // single pass: add this slab's sums straight into the (pre-zeroed or accumulating) outputs
      if (kNorm) atomicAdd(part_w + blockIdx.x * 256 + c, tw);
      if (part_b) atomicAdd(part_b + blockIdx.x * 256 + c, tb);
    } else {
      const size_t o = static_cast<size_t>(blockIdx.y) * dim + blockIdx.x * 256 + c;
      if (kNorm) part_w[o] = tw;
      if (part_b) part_b[o] = tb;
    }
  }
}

// 32 columns x 8 slab lanes per block: thread (c, l) adds slabs l, l+8, ... of column c,
// then the 8 lanes are combined in a fixed order.
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ part_w, const float* __restrict__ part_b,
                                                           float* __restrict__ dw, float* __restrict__ db, int slabs, int dim) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  __shared__ float sw[8][33], sb[8][33];
  const int cx = threadIdx.x & 31, ly = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float tw = 0.f, tb = 0.f;
  if (c < dim) {
    for (int s = ly; s < slabs; s += 8) {
      if (part_w) tw += part_w[static_cast<size_t>(s) * dim + c];
      if (part_b) tb += part_b[static_cast<size_t>(s) * dim + c];
    }
  }
  sw[ly][cx] = tw;
  sb[ly][cx] = tb;
  __syncthreads();
  if (ly == 0 && c < dim) {
    float aw = 0.f, ab = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      aw += sw[k][cx];
      ab += sb[k][cx];
    }
    if (dw) dw[c] = aw;
    if (db) db[c] = ab;
  }
}

int colsum_slabs(int rows) { return (rows + kSlabRows - 1) / kSlabRows; }

cudaError_t norm_fwd(const __nv_bfloat16* x, const float* w, const float* b, __nv_bfloat16* y, float* mean, float* rstd,
                     int rows, int dim, float eps, cudaStream_t stream) {
  if (dim % 8 != 0) return cudaErrorNotSupported;
  const int blocks = (rows + 7) / 8;
  if (b) MCCL_LAUNCH_PDL(norm_fwd_kernel<true>, blocks, 256, 0, stream, x, w, b, y, mean, rstd, rows, dim, eps);
  else MCCL_LAUNCH_PDL(norm_fwd_kernel<false>, blocks, 256, 0, stream, x, w, b, y, mean, rstd, rows, dim, eps);
  count_launch();
  return ::mccl::launch_status();
}

cudaError_t norm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const float* w, const float* mean, const float* rstd,
                     __nv_bfloat16* dx, float* dw, float* db, float* scratch, int rows, int dim, bool layernorm,
                     cudaStream_t stream, const __nv_bfloat16* dx_add, int parts) {
  if (dim % 8 != 0) return cudaErrorNotSupported;
  const int blocks = (rows + 7) / 8;
  if (parts & 1) {
    if (layernorm) MCCL_LAUNCH_PDL(norm_bwd_dx_kernel<true>, blocks, 256, 0, stream, dy, x, w, mean, rstd, dx, dx_add, rows, dim);
    else MCCL_LAUNCH_PDL(norm_bwd_dx_kernel<false>, blocks, 256, 0, stream, dy, x, w, mean, rstd, dx, dx_add, rows, dim);
    count_launch();
  }
  if (!(parts & 2)) return ::mccl::launch_status();
  const int slabs = colsum_slabs(rows);
  dim3 grid((dim + 255) / 256, slabs);
  if (!scratch) {
    // no scratch: dw / db accumulate the slab sums atomically (they must hold the value to add to)
    MCCL_LAUNCH_PDL(colsum_partial_kernel<true>, grid, 256, 0, stream, dy, x, mean, rstd, dw, layernorm ? db : nullptr, rows, dim, 1);
    count_launch();
    return ::mccl::launch_status();
  }
  float* part_w = scratch;
  float* part_b = layernorm ? scratch + static_cast<size_t>(slabs) * dim : nullptr;
  MCCL_LAUNCH_PDL(colsum_partial_kernel<true>, grid, 256, 0, stream, dy, x, mean, rstd, part_w, part_b, rows, dim, 0);
  MCCL_LAUNCH_PDL(colsum_final_kernel, (dim + 31) / 32, 256, 0, stream, part_w, part_b, dw, layernorm ? db : nullptr, slabs, dim);
  count_launch(2);
  return ::mccl::launch_status();
}

cudaError_t colsum_bf16(const __nv_bfloat16* in, float* out, float* scratch, int rows, int dim, cudaStream_t stream) {
  if (dim % 8 != 0 || (reinterpret_cast<uintptr_t>(in) & 15u)) return cudaErrorNotSupported;
  const int slabs = colsum_slabs(rows);
  dim3 grid((dim + 255) / 256, slabs);
  if (!scratch) {
    MCCL_LAUNCH_PDL(colsum_partial_kernel<false>, grid, 256, 0, stream, in, nullptr, nullptr, nullptr, nullptr, out, rows, dim, 1);
    count_launch();
    return ::mccl::launch_status();
  }
  MCCL_LAUNCH_PDL(colsum_partial_kernel<false>, grid, 256, 0, stream, in, nullptr, nullptr, nullptr, nullptr, scratch, rows, dim, 0);
  MCCL_LAUNCH_PDL(colsum_final_kernel, (dim + 31) / 32, 256, 0, stream, nullptr, scratch, nullptr, out, slabs, dim);
  count_launch(2);
  return ::mccl::launch_status();
}

// ------------------------------------------------------------------ AdamW --
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                                    float* __restrict__ v, __nv_bfloat16* __restrict__ p16, long long n4, long long n,
                                                    float lr, float b1, float b2, float eps, float wd,
                                                    const float* __restrict__ step_ptr, float gscale, int zero_grad) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  const float step = *step_ptr;
  const float bc1 = 1.f - powf(b1, step), bc2 = 1.f - powf(b2, step);
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2), decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i], gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    float* P = &pp.x; float* G = &gg.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = G[k] * gscale;
      M[k] = b1 * M[k] + (1.f - b1) * gk;
      V[k] = b2 * V[k] + (1.f - b2) * gk * gk;
      const float denom = sqrtf(V[k]) * inv_sqrt_bc2 + eps;
      P[k] = P[k] * decay - lr * (M[k] * inv_bc1) / denom;
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(p16)[i] = packed;
    }
  }
  // scalar tail (n not a multiple of 4)
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      const float gk = g[i] * gscale;
      const float mk = b1 * m[i] + (1.f - b1) * gk, vk = b2 * v[i] + (1.f - b2) * gk * gk;
      m[i] = mk;
      v[i] = vk;
      const float pk = p[i] * decay - lr * (mk * inv_bc1) / (sqrtf(vk) * inv_sqrt_bc2 + eps);
      p[i] = pk;
      if (zero_grad) g[i] = 0.f;
      if (p16) p16[i] = __float2bfloat16_rn(pk);
    }
  }
}

cudaError_t adamw_flat(float* p, float* g, float* m, float* v, __nv_bfloat16* p16, long long n, float lr, float beta1,
                       float beta2, float eps, float wd, const float* step, float grad_scale, cudaStream_t stream, bool zero_grad,
                       int ctas_per_sm) {
  if (n <= 0) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15u)
    return cudaErrorNotSupported;
  const long long n4 = n / 4;
  // The CTAs stride over the buffer and live as long as the kernel: eight of 256 threads fill an SM, so a kernel
  // launched beside this one (a collective of the buckets still in flight) would wait for the whole update.
  // ctas_per_sm < 8 leaves it room.
  if (ctas_per_sm < 1 || ctas_per_sm > 8) ctas_per_sm = 8;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * ctas_per_sm) blocks = 148 * ctas_per_sm;
  if (blocks < 1) blocks = 1;
  MCCL_LAUNCH_PDL(adamw_kernel, static_cast<int>(blocks), 256, 0, stream, p, g, m, v, p16, n4, n, lr, beta1, beta2, eps, wd, step, grad_scale,
              zero_grad ? 1 : 0);
  count_launch();
  return ::mccl::launch_status();
}

// ---------------------------------------------------------- cross entropy --
// One CTA per row.  Pass 1: running max and sum of exp (online softmax).
// Pass 2: overwrite the row with (softmax - onehot) * scale.
__global__ void __launch_bounds__(512) ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                 float* __restrict__ loss_rows, int vocab, float scale) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  __shared__ float s_max[16], s_sum[16];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  __nv_bfloat16* lr = logits + static_cast<size_t>(row) * vocab;
  uint4* lv = reinterpret_cast<uint4*>(lr);
  const int vecs = vocab >> 3;
  float mx = -INFINITY, sm = 0.f;
  for (int v = tid; v < vecs; v += blockDim.x) {
    float f[8];
    unpack8(lv[v], f);
    float local = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) local = fmaxf(local, f[i]);
    if (local > mx) {
      sm *= __expf(mx - local);
      mx = local;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm += __expf(f[i] - mx);
  }
  for (int c = vecs * 8 + tid; c < vocab; c += blockDim.x) {
    const float f = __bfloat162float(lr[c]);
    if (f > mx) {
      sm *= __expf(mx - f);
      mx = f;
    }
    sm += __expf(f - mx);
  }
  // combine (max, sum) pairs: warp, then block
  const float wmx = warp_max(mx);
  sm = warp_sum(mx == -INFINITY ? 0.f : sm * __expf(mx - wmx));  // threads without elements hold (-inf, 0)
  if (lane == 0) {
    s_max[wid] = wmx;
    s_sum[wid] = sm;
  }
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float bmx = -INFINITY;
  for (int i = 0; i < nw; ++i) bmx = fmaxf(bmx, s_max[i]);
  float bsum = 0.f;
  for (int i = 0; i < nw; ++i) bsum += s_max[i] == -INFINITY ? 0.f : s_sum[i] * __expf(s_max[i] - bmx);
  const long long tgt = targets[row];
  const bool ignore = tgt < 0 || tgt >= vocab;
  if (tid == 0) loss_rows[row] = ignore ? 0.f : (logf(bsum) + bmx - __bfloat162float(lr[tgt]));
  __syncthreads();  // the target logit is read before anyone overwrites it
  const float inv = ignore ? 0.f : scale / bsum;
  for (int v = tid; v < vecs; v += blockDim.x) {
    float f[8], o[8];
    unpack8(lv[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o[i] = __expf(f[i] - bmx) * inv;
      if (!ignore && v * 8 + i == tgt) o[i] -= scale;
    }
    lv[v] = pack8(o);
  }
  for (int c = vecs * 8 + tid; c < vocab; c += blockDim.x) {
    float o = __expf(__bfloat162float(lr[c]) - bmx) * inv;
    if (!ignore && c == tgt) o -= scale;
    lr[c] = __float2bfloat16_rn(o);
  }
}

cudaError_t cross_entropy_fwd_bwd(__nv_bfloat16* logits, const long long* targets, float* loss_rows, int rows, int vocab,
                                  float grad_scale, cudaStream_t stream) {
  if (vocab % 8 != 0 || (reinterpret_cast<uintptr_t>(logits) & 15u)) return cudaErrorNotSupported;
  // (A variant that kept the row in registers - one read, one exponential per value - was measured at 222 us against
  // this kernel's 125 us on 4096 x 32000: its 512-thread CTAs run one per SM and nothing hides their load latency.)
  MCCL_LAUNCH_PDL(ce_kernel, rows, 512, 0, stream, logits, targets, loss_rows, vocab, grad_scale);
  count_launch();
  return ::mccl::launch_status();
}

// -------------------------------------------------------------- transpose --
__global__ void __launch_bounds__(256) transpose_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                        int rows, int cols) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  __shared__ __nv_bfloat16 tile[64][66];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int rr = ty; rr < 64; rr += 8) {
    const int r = r0 + rr;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = c0 + tx * 2 + h;
      tile[rr][tx * 2 + h] = (r < rows && c < cols) ? in[static_cast<size_t>(r) * cols + c] : __float2bfloat16(0.f);
    }
  }
  __syncthreads();
  for (int cc = ty; cc < 64; cc += 8) {
    const int c = c0 + cc;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = r0 + tx * 2 + h;
      if (c < cols && r < rows) out[static_cast<size_t>(c) * rows + r] = tile[tx * 2 + h][cc];
    }
  }
}

cudaError_t transpose_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, int rows, int cols, cudaStream_t stream) {
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  MCCL_LAUNCH_PDL(transpose_kernel, grid, 256, 0, stream, in, out, rows, cols);
  count_launch();
  return ::mccl::launch_status();
}

// ------------------------------------------------------------------ casts --
__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 f = reinterpret_cast<const float4*>(in)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(out)[i] = packed;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) out[i] = __float2bfloat16_rn(in[i]);
}

cudaError_t cast_f32_bf16(const float* in, __nv_bfloat16* out, long long n, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(out) & 7u)) return cudaErrorNotSupported;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  MCCL_LAUNCH_PDL(cast_kernel, static_cast<int>(blocks), 256, 0, stream, in, out, n);
  count_launch();
  return ::mccl::launch_status();
}

// ------------------------------------------------------------- GELU bwd ---
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                                                       __nv_bfloat16* __restrict__ dz, long long n8) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[8], zz[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(dy)[i], g);
    unpack8(reinterpret_cast<const uint4*>(z)[i], zz);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x = zz[k];
      const float cdf = 0.5f * (1.f + erff(x * 0.70710678f));
      const float pdf = 0.39894228f * __expf(-0.5f * x * x);
      o[k] = g[k] * (cdf + x * pdf);
    }
    reinterpret_cast<uint4*>(dz)[i] = pack8(o);
  }
}

cudaError_t gelu_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* z, __nv_bfloat16* dz, long long n, cudaStream_t stream) {
  if (n % 8 != 0) return cudaErrorNotSupported;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  MCCL_LAUNCH_PDL(gelu_bwd_kernel, static_cast<int>(blocks), 256, 0, stream, dy, z, dz, n / 8);
  count_launch();
  return ::mccl::launch_status();
}

// ------------------------------------------------------------ embedding ---
// One thread per 8 output elements; ids outside [0, vocab) read row 0 and add nothing.
__global__ void __launch_bounds__(256) embed_fwd_kernel(const long long* __restrict__ ids, const float* __restrict__ tok,
                                                        const float* __restrict__ pos, __nv_bfloat16* __restrict__ y, long long n8,
                                                        int seq, int dim8, int vocab) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / dim8;
    const int c = static_cast<int>(i % dim8);
    long long id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    const float4* row = reinterpret_cast<const float4*>(tok + id * dim8 * 8) + 2 * c;
    float4 a = row[0], b = row[1];
    if (pos != nullptr) {
      const float4* prow = reinterpret_cast<const float4*>(pos + (t % seq) * dim8 * 8) + 2 * c;
      const float4 pa = prow[0], pb = prow[1];
      a.x += pa.x, a.y += pa.y, a.z += pa.z, a.w += pa.w;
      b.x += pb.x, b.y += pb.y, b.z += pb.z, b.w += pb.w;
    }
    const float o[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    reinterpret_cast<uint4*>(y)[i] = pack8(o);
  }
}

__global__ void __launch_bounds__(256) embed_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                                        float* __restrict__ dtok, float* __restrict__ dpos, long long n8, int seq,
                                                        int dim8, int vocab, float scale) {
  // dependent launch: the CTA may be resident before the previous kernel of the stream has finished
  ::mccl::pdl_trigger();
  ::mccl::pdl_wait();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / dim8;
    const int c = static_cast<int>(i % dim8);
    float g[8];
    unpack8(reinterpret_cast<const uint4*>(dy)[i], g);
    const float4 lo = make_float4(g[0] * scale, g[1] * scale, g[2] * scale, g[3] * scale);
    const float4 hi = make_float4(g[4] * scale, g[5] * scale, g[6] * scale, g[7] * scale);
    const long long id = ids[t];
    if (dtok != nullptr && id >= 0 && id < vocab) {
      float4* row = reinterpret_cast<float4*>(dtok + id * dim8 * 8) + 2 * c;
      atomicAdd(row, lo);
      atomicAdd(row + 1, hi);
    }
    if (dpos != nullptr) {
      float4* prow = reinterpret_cast<float4*>(dpos + (t % seq) * dim8 * 8) + 2 * c;
      atomicAdd(prow, lo);
      atomicAdd(prow + 1, hi);
    }
  }
}

static int embed_blocks(long long n8) {
  long long blocks = (n8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return blocks < 1 ? 1 : static_cast<int>(blocks);
}

cudaError_t embed_fwd(const long long* ids, const float* tok, const float* pos, __nv_bfloat16* y, int tokens, int seq, int dim,
                      int vocab, cudaStream_t stream) {
  if (dim % 8 != 0 || tokens <= 0 || seq <= 0) return cudaErrorNotSupported;
  const long long n8 = static_cast<long long>(tokens) * (dim / 8);
  MCCL_LAUNCH_PDL(embed_fwd_kernel, embed_blocks(n8), 256, 0, stream, ids, tok, pos, y, n8, seq, dim / 8, vocab);
  count_launch();
  return ::mccl::launch_status();
}

cudaError_t embed_bwd(const long long* ids, const __nv_bfloat16* dy, float* dtok, float* dpos, int tokens, int seq, int dim,
                      int vocab, cudaStream_t stream, float scale) {
  if (dim % 8 != 0 || tokens <= 0 || seq <= 0) return cudaErrorNotSupported;
  const long long n8 = static_cast<long long>(tokens) * (dim / 8);
  MCCL_LAUNCH_PDL(embed_bwd_kernel, embed_blocks(n8), 256, 0, stream, ids, dy, dtok, dpos, n8, seq, dim / 8, vocab, scale);
  count_launch();
  return ::mccl::launch_status();
}

}  // namespace ops
}  // namespace mccl

// ---------------------------------------------------------------------------
// Allocation-free column sum (see noalloc.h for who needs it and the rules).
// The partial sums live in an array that is part of this library's device
// image.  Host code may not use the array's name as a pointer: the address the
// kernels need is looked up once per device with cudaGetSymbolAddress.
// ---------------------------------------------------------------------------
#include <cstdio>

#include "noalloc.h"

namespace {

static __device__ __align__(256) float g_noalloc_scratch[MCCL_NOALLOC_SCRATCH_FLOATS];

constexpr int kNoallocMaxDevices = 64;
// Filled once per device; an atomic pointer because two threads may make their first call at the same time
// (both would store the same address, but an unsynchronised store is still a data race).
std::atomic<float*> g_noalloc_scratch_ptr[kNoallocMaxDevices];
thread_local char t_noalloc_error[256] = "";

// Device address of the scratch array on the current device (looked up on first use).
float* noalloc_scratch_for_current_device() {
  int device = -1;
  cudaError_t rc = cudaGetDevice(&device);
  if (rc != cudaSuccess || device < 0 || device >= kNoallocMaxDevices) {
    std::snprintf(t_noalloc_error, sizeof(t_noalloc_error), "cannot identify the current device: %s",
                  rc == cudaSuccess ? "index out of range" : cudaGetErrorString(rc));
    return nullptr;
  }
  float* ptr = g_noalloc_scratch_ptr[device].load(std::memory_order_acquire);
  if (!ptr) {
    rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (rc != cudaSuccess || !ptr) {
      std::snprintf(t_noalloc_error, sizeof(t_noalloc_error), "cudaGetSymbolAddress failed on device %d: %s", device,
                    cudaGetErrorString(rc));
      return nullptr;
    }
    g_noalloc_scratch_ptr[device].store(ptr, std::memory_order_release);
  }
  return ptr;
}

// True when `p` is device memory of `device` (or memory CUDA cannot classify, which is let through).
bool noalloc_on_device(const void* p, int device) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return true;
  }
  if (attr.type == cudaMemoryTypeDevice) return attr.device == device;
  return attr.type != cudaMemoryTypeHost;   // pinned host memory is not what the kernels expect
}

}  // namespace

extern "C" const char* mccl_noalloc_last_error(void) { return t_noalloc_error; }

extern "C" int mccl_colsum_bf16_noalloc(const void* in_bf16, float* out, int rows, int dim, void* stream) {
  t_noalloc_error[0] = 0;
  if (!in_bf16 || !out || rows <= 0 || dim <= 0 || dim % 8 != 0 || (reinterpret_cast<uintptr_t>(in_bf16) & 15u)) {
    std::snprintf(t_noalloc_error, sizeof(t_noalloc_error),
                  "bad argument: need non-null pointers, rows > 0, dim a positive multiple of 8 and a 16-byte aligned input");
    return MCCL_NOALLOC_BAD_ARGUMENT;
  }
  const long long slabs = mccl::ops::colsum_slabs(rows);
  const long long need = slabs * dim;
  if (need > MCCL_NOALLOC_SCRATCH_FLOATS) {
    std::snprintf(t_noalloc_error, sizeof(t_noalloc_error),
                  "problem too large for the fixed scratch array: ceil(rows/64)*dim = %lld floats, limit %d", need,
                  MCCL_NOALLOC_SCRATCH_FLOATS);
    return MCCL_NOALLOC_TOO_LARGE;
  }
  if (slabs > MCCL_NOALLOC_MAX_SLABS) {
    // many rows of a narrow matrix: the partial sums would fit, but one grid dimension of the first stage is the
    // number of slabs, and that dimension is limited to 65535
    std::snprintf(t_noalloc_error, sizeof(t_noalloc_error),
                  "problem too large: ceil(rows/64) = %lld row slabs, limit %d (rows <= %d)", slabs, MCCL_NOALLOC_MAX_SLABS,
                  MCCL_NOALLOC_MAX_SLABS * 64);
    return MCCL_NOALLOC_TOO_LARGE;
  }
  float* scratch = noalloc_scratch_for_current_device();
  if (!scratch) return MCCL_NOALLOC_CUDA_ERROR;
  int device = -1;
  cudaGetDevice(&device);
  if (!noalloc_on_device(in_bf16, device) || !noalloc_on_device(out, device)) {
    std::snprintf(t_noalloc_error, sizeof(t_noalloc_error),
                  "bad argument: in and out must be device memory of the current device (%d); the scratch array used is that device's", device);
    return MCCL_NOALLOC_BAD_ARGUMENT;
  }
  cudaError_t rc = mccl::ops::colsum_bf16(static_cast<const __nv_bfloat16*>(in_bf16), out, scratch, rows, dim,
                                          static_cast<cudaStream_t>(stream));
  if (rc != cudaSuccess) {
    std::snprintf(t_noalloc_error, sizeof(t_noalloc_error), "kernel launch failed: %s", cudaGetErrorString(rc));
    return MCCL_NOALLOC_CUDA_ERROR;
  }
  return MCCL_NOALLOC_OK;
}
