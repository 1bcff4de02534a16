// Host implementations of the collectives over the TCP mesh, and the host
// restatement of the element-wise reduce kernels.
//
// Parity: allreduce ring / tree / butterfly follow the reference's schedules
// (csrc/backend/AllreduceAlgos.cpp:52-206): ring = N-1 reduce-scatter steps +
// N-1 allgather steps on ceil(numel/N)-sized chunks whose tail chunks may be
// short or empty; tree = binomial reduce to rank 0 + binomial broadcast;
// butterfly = direct all-to-all reduce-scatter + local reduce + all-to-all
// allgather.  AVG is SUM followed by a 1/world scale.  Unlike the reference,
// which reduces in bf16 when MCCL_WIRE_DTYPE=bf16
// (ProcessGroupMCCL.cpp:116-133), the bf16 wire here only narrows what
// crosses the wire: accumulation stays fp32, and the owner of each chunk
// rounds its result to bf16 too so that every rank ends with the same bits.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include "../core/config.hpp"
#include "../net/tcp_mesh.hpp"
#include "dtypes.hpp"

namespace mccl {

// Chunking used by ring, butterfly, reduce-scatter and the device kernels:
// per = ceil(numel / world); chunk i = [min(i*per, numel), min((i+1)*per, numel)).
struct Chunks {
  size_t numel = 0, per = 0;
  int world = 1;
  Chunks(size_t n, int w) : numel(n), per(w > 0 ? (n + w - 1) / w : n), world(w) {}
  size_t offset(int i) const {
    size_t o = static_cast<size_t>(i) * per;
    return o < numel ? o : numel;
  }
  size_t len(int i) const { return offset(i + 1 > world ? world : i + 1) - offset(i); }
};

// ---- element-wise primitives (host restatement of the device kernels) ----
// dst[i] = dst[i] ∘ src[i]
void reduce_into(DType t, RedOp op, void* dst, const void* src, size_t n);
// buf[i] *= s  (integers: divided by round(1/s) when s < 1, exact for AVG)
void scale_inplace(DType t, void* buf, size_t n, double s);
// dst[i] = (dst[i] + src[i]) * s
void reduce_scale(DType t, void* dst, const void* src, size_t n, double s);
void f32_to_bf16(const float* src, uint16_t* dst, size_t n);
void bf16_to_f32(const uint16_t* src, float* dst, size_t n);
// dst[i] = dst[i] ∘ float(src[i])
void reduce_bf16_into_f32(RedOp op, float* dst, const uint16_t* src, size_t n);
// Rounds fp32 values to bf16 precision in place.
void round_f32_to_bf16_inplace(float* buf, size_t n);

struct AllreduceArgs {
  void* data = nullptr;  // in place
  size_t numel = 0;
  DType dtype = DType::F32;
  RedOp op = RedOp::SUM;
  WireDtype wire = WireDtype::NATIVE;  // BF16 only honoured for F32 data
};

// Picks the schedule the way the reference does (ProcessGroupMCCL.cpp:135-145):
// AUTO → TREE when bytes ≤ tree_below else RING; RING with numel < world → TREE;
// BUTTERFLY with world < 2 or numel < world → TREE.  ONESHOT maps to TREE and
// NVLS to BUTTERFLY on the host (they are device-only schedules).
Algo resolve_cpu_algo(Algo requested, size_t numel, size_t bytes, int world, int64_t tree_below);

void allreduce_ring(TcpMesh& mesh, const AllreduceArgs& a);
void allreduce_tree(TcpMesh& mesh, const AllreduceArgs& a);
void allreduce_butterfly(TcpMesh& mesh, const AllreduceArgs& a);
void allreduce(TcpMesh& mesh, const AllreduceArgs& a, Algo algo);

// Binomial broadcast of nbytes from root.
void broadcast(TcpMesh& mesh, void* data, size_t nbytes, int root);
// Binomial reduce to root (result valid on root only; other ranks' data is scratch).
void reduce(TcpMesh& mesh, void* data, size_t numel, DType t, RedOp op, int root);
// out has world * nbytes bytes; slot r holds rank r's input.
void allgather(TcpMesh& mesh, const void* in, void* out, size_t nbytes);
// in has world * numel elements; out gets the reduced slice [rank*numel, (rank+1)*numel).
void reduce_scatter(TcpMesh& mesh, const void* in, void* out, size_t numel, DType t, RedOp op);
// Variable all-to-all in bytes: send in[in_off[p] .. +in_len[p]) to p, receive into out[out_off[p] ..).
void alltoallv(TcpMesh& mesh, const void* in, const std::vector<size_t>& in_off, const std::vector<size_t>& in_len,
               void* out, const std::vector<size_t>& out_off, const std::vector<size_t>& out_len);
void gather(TcpMesh& mesh, const void* in, void* out /* root only */, size_t nbytes, int root);
void scatter(TcpMesh& mesh, const void* in /* root only */, void* out, size_t nbytes, int root);

// Tagged point-to-point framing: header {int32 tag, int64 nbytes} then payload.
// recv_tagged checks size and tag (tag < 0 on the receiver matches any tag).
void send_tagged(TcpMesh& mesh, int dst, const void* data, size_t nbytes, int tag);
void recv_tagged(TcpMesh& mesh, int src, void* data, size_t nbytes, int tag);

}  // namespace mccl
