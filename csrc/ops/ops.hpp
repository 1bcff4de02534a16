// Host entry points of the model-operator kernels (sm_100a).  All launchers
// enqueue on the given stream and return the launch status.  The reference has
// no counterpart for these: its models run on stock PyTorch/MPS operators
// (examples/ddp_utils.py:41-147); they exist here because the headline
// benchmark is a training step, and on a B200 that step is bound by these
// operators, not by the collectives.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

namespace mccl {
namespace ops {

// Number of operator kernels launched so far (all launchers below count).
uint64_t launch_count();
void count_launch(int n = 1);

// ---- normalisation: y = (x - mean) * rstd * w + b  (LayerNorm, bias != null)
//                     y = x * rstd * w                (RMSNorm, bias == null)
// x, y: [rows, dim] bf16; w, b: fp32; mean / rstd: fp32 [rows] saved for backward.
cudaError_t norm_fwd(const __nv_bfloat16* x, const float* w, const float* b, __nv_bfloat16* y, float* mean, float* rstd,
                     int rows, int dim, float eps, cudaStream_t stream);
// dx: [rows, dim] bf16; dw, db: fp32 [dim].  With scratch (fp32, 2 * colsum_slabs(rows) * dim
// elements) dw / db are overwritten by a two-stage, order-fixed reduction; with scratch == nullptr
// the slab sums are added to dw / db atomically in one pass.  dx_add (optional, [rows, dim] bf16) is a
// second gradient of x (a residual path) that is added to dx before the one rounding to bf16.
cudaError_t norm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const float* w, const float* mean, const float* rstd,
                     __nv_bfloat16* dx, float* dw, float* db, float* scratch, int rows, int dim, bool layernorm,
                     cudaStream_t stream, const __nv_bfloat16* dx_add = nullptr, int parts = 3);
// out[c] = sum over rows of in[r, c] (bias gradients).  scratch: colsum_slabs(rows) * dim floats,
// or nullptr to add into out atomically in one pass.
cudaError_t colsum_bf16(const __nv_bfloat16* in, float* out, float* scratch, int rows, int dim, cudaStream_t stream);
int colsum_slabs(int rows);

// ---- fused AdamW over flat fp32 buffers; step is a device scalar (float) so the
// launch can be replayed from a CUDA graph.  p16 (optional) receives bf16(p).  With zero_grad the gradient
// is cleared in the same pass (it has just been read), which replaces the memset at the start of the next step.
cudaError_t adamw_flat(float* p, float* g, float* m, float* v, __nv_bfloat16* p16, long long n, float lr, float beta1,
                       float beta2, float eps, float wd, const float* step, float grad_scale, cudaStream_t stream,
                       bool zero_grad = false, int ctas_per_sm = 8);

// ---- softmax cross entropy, forward and backward in one pass over the logits:
// loss_rows[t] = logsumexp(logits[t]) - logits[t, target[t]];
// logits[t] is overwritten by (softmax - onehot) * grad_scale.
cudaError_t cross_entropy_fwd_bwd(__nv_bfloat16* logits, const long long* targets, float* loss_rows, int rows, int vocab,
                                  float grad_scale, cudaStream_t stream);

// ---- out[c, r] = in[r, c] for a bf16 matrix [rows, cols].
cudaError_t transpose_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, int rows, int cols, cudaStream_t stream);
// fp32 → bf16 cast of n elements.
cudaError_t cast_f32_bf16(const float* in, __nv_bfloat16* out, long long n, cudaStream_t stream);
// GELU backward on a pre-activation: dz = dy * gelu'(z).
cudaError_t gelu_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* z, __nv_bfloat16* dz, long long n, cudaStream_t stream);

// ---- token (+ learned position) embedding.  y[t, :] = bf16(tok[ids[t], :] + pos[t % seq, :]);
// tok / pos are fp32 [vocab, dim] / [>= seq, dim] (pos may be null); dim % 8 == 0.
cudaError_t embed_fwd(const long long* ids, const float* tok, const float* pos, __nv_bfloat16* y, int tokens, int seq, int dim,
                      int vocab, cudaStream_t stream);
// Adds dy[t, :] into dtok[ids[t], :] and dpos[t % seq, :] (fp32, atomically; dpos may be null).
cudaError_t embed_bwd(const long long* ids, const __nv_bfloat16* dy, float* dtok, float* dpos, int tokens, int seq, int dim,
                      int vocab, cudaStream_t stream, float scale = 1.f);

// ---- causal self-attention, head dimension 64, straight from the fused QKV projection.
// qkv: [B, S, 3, H, 64] bf16; o: [B, S, H, 64] bf16; lse: [B, H, S] fp32 (log2 domain, saved for backward).
// Forward needs S % 128 == 0; backward S == 128 or 256 (cudaErrorNotSupported otherwise: the caller falls back).
cudaError_t attention_fwd(const __nv_bfloat16* qkv, __nv_bfloat16* o, float* lse, int B, int S, int H, float softmax_scale,
                          cudaStream_t stream);
// dqkv: [B, S, 3, H, 64] bf16, every element written.
cudaError_t attention_bwd(const __nv_bfloat16* qkv, const __nv_bfloat16* o, const __nv_bfloat16* d_o, const float* lse,
                          __nv_bfloat16* dqkv, int B, int S, int H, float softmax_scale, cudaStream_t stream);

// ---- tcgen05 GEMM: D[M,N] = A[M,K] · B[N,K]^T (+ bias[N]) (GELU) ; A, B bf16 with K contiguous.
enum GemmEpilogue : int {
  EPI_NONE = 0,       // D = acc
  EPI_BIAS = 1,       // D = acc + bias[n]
  EPI_BIAS_GELU = 2,  // Z = acc + bias[n] (written to aux), D = gelu(Z)
  EPI_GELU = 3,       // Z = acc (written to aux), D = gelu(Z)
  EPI_BIAS_GELU_D = 4,  // Z = acc + bias[n], D = gelu(Z), aux = gelu'(Z): backward then only multiplies (see GemmArgs::mul)
  EPI_GELU_D = 5,       // the same without bias
};
struct GemmArgs {
  const __nv_bfloat16* a = nullptr;  // [M, K], row stride lda (elements); a_mn_major: stored [K, M]
  const __nv_bfloat16* b = nullptr;  // [N, K], row stride ldb;            b_mn_major: stored [K, N]
  bool a_mn_major = false;
  bool b_mn_major = false;
  void* d = nullptr;                 // [M, N] bf16 or fp32, row stride ldd
  __nv_bfloat16* aux = nullptr;      // [M, N] pre-activation (GELU epilogues)
  const float* bias = nullptr;       // [N]
  const __nv_bfloat16* residual = nullptr;  // [M, N] added after bias / activation, row stride ldd
  const __nv_bfloat16* mul = nullptr;       // [M, N]: D = acc * mul (e.g. the saved gelu'(z): the input gradient through a GELU), row stride ldd
  int m = 0, n = 0, k = 0;
  int lda = 0, ldb = 0, ldd = 0;
  bool d_fp32 = false;
  bool accumulate = false;           // D += result (fp32 output only)
  int epilogue = EPI_NONE;
};
// Returns cudaErrorNotSupported for shapes the kernel does not cover
// (K % 64 != 0, N % 8 != 0, unaligned pointers); the caller falls back.
cudaError_t gemm_bf16_tn(const GemmArgs& args, cudaStream_t stream);
// Caps the number of CTAs (= SMs) plain GEMM launches occupy from now on; 0 restores one CTA per SM.  A
// data-parallel trainer lowers it during backward so that a few SMs stay free for the gradient collectives
// that run beside the GEMMs.  The value is read at launch time, so it is baked into a captured CUDA graph.
void set_gemm_cta_limit(int ctas);
// Which kernel plain products use: "pair" (CTA pairs, the default), "persistent" (one CTA per SM), "tile"; "" = default.
void set_gemm_kernel(const std::string& name);
int gemm_cta_limit();
int gemm_sm_count();
// Why the last gemm_bf16_tn call on this thread returned cudaErrorNotSupported ("" otherwise).
const char* gemm_last_reason();
// Non-zero when a pipeline wait inside a GEMM kernel ran out (kernel returned early).
int gemm_error_flag();

}  // namespace ops
}  // namespace mccl
