// Host entry points of the collective kernels.  Every launcher enqueues one
// kernel on cfg.stream and returns the launch status; nothing synchronises.
// With cfg.nlocal > 1 the launch is cooperative and carries nlocal virtual
// ranks in blockIdx.y (single-GPU emulation used by the tests).
#pragma once

#include <cuda_runtime.h>

#include "coll_args.hpp"

namespace mccl {
namespace dev {

struct DevComm;  // comm_device.cuh
struct P2PComm;  // comm_device.cuh

enum class ElemType : int { F32 = 0, F16, BF16, F64, I32, I64 };

struct LaunchCfg {
  int ctas = 1;
  int threads = 0;   // threads per CTA; 0 = default (MCCL_COMM_THREADS or 256)
  int nlocal = 1;
  cudaStream_t stream = nullptr;
};

cudaError_t launch_allreduce_twoshot(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
// two-shot whose all-gather half is pushed as well (no loads from peers); needs twoshot_push_bytes of arena
cudaError_t launch_allreduce_twoshot_push(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
cudaError_t launch_allreduce_oneshot(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
cudaError_t launch_allreduce_ring(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
cudaError_t launch_allreduce_tree(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
// staged: copy in → arena, reduce in the switch, copy arena → out.
// not staged: local_sym / mc_sym are the unicast and multicast mappings of a
// symmetric buffer that already holds the wire-typed data; reduced in place.
cudaError_t launch_allreduce_nvls(ElemType t, bool bf16_wire, bool staged, const DevComm& c, const CollArgs& a,
                                  char* local_sym, char* mc_sym, const LaunchCfg& cfg);
// In place on a symmetric-heap buffer: a.in[r] = rank r's copy as mapped here,
// a.per = chunk elements (multiple of 16), buffer padded to world * per.
cudaError_t launch_allreduce_symm(ElemType t, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
cudaError_t launch_reduce_scatter(ElemType t, bool bf16_wire, const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);
cudaError_t launch_allgather(const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);   // a.numel = bytes per rank
cudaError_t launch_broadcast(const DevComm& c, const CollArgs& a, const LaunchCfg& cfg);   // a.numel = bytes, a.out = data
cudaError_t launch_alltoall(const DevComm& c, const A2AArgs& a, const LaunchCfg& cfg);
cudaError_t launch_barrier(const DevComm& c, const LaunchCfg& cfg);
// One message between pairs of ranks (send / recv); cfg.ctas must agree on both sides of a pair.
cudaError_t launch_p2p(const P2PComm& c, const P2PArgs& a, const LaunchCfg& cfg);

// Element-wise kernels (standalone forms of what the collectives fuse).
// op is dev::Op; n elements; pointers may have any alignment.
cudaError_t launch_reduce2(ElemType t, int op, void* dst, const void* src, long long n, cudaStream_t stream);
cudaError_t launch_scale(ElemType t, void* buf, long long n, float scale, cudaStream_t stream);
cudaError_t launch_reduce2_scale(ElemType t, void* dst, const void* src, long long n, float scale, cudaStream_t stream);

}  // namespace dev
}  // namespace mccl
