// Device communicator: one per (process group, GPU).
//
// Owns the peer-mapped symmetric arena and signal pads of the group
// (SymmMesh), the per-rank device state words the kernels keep between
// launches, and the pinned status word the kernels write when a bounded wait
// runs out.  Every method enqueues kernels on the given CUDA stream and
// returns at once; nothing here blocks the host on the GPU.
//
// This is the NVLink replacement for what the reference does with one TCP
// socket per peer and Metal reduce kernels (csrc/backend/PeerMesh.cpp,
// csrc/backend/AllreduceAlgos.cpp, csrc/metal/MetalKernels.mm): the schedule
// names are the same (ring / tree / butterfly), but the data moves by loads
// and stores to peer GPUs' memory issued from inside the kernels.
//
// One collective at a time: all launches of a communicator share its arena
// halves, flags and epochs, so they are ordered on the device.  Launches on
// the same stream are ordered by the stream; a launch on a different stream
// than the previous one first waits for an event recorded after that one.
// Inside a CUDA graph capture the caller's capture dependencies must provide
// the order (fork the comm stream from, and join it back into, the capturing
// stream), and a captured graph must not run concurrently with eager
// collectives of the same communicator.
//
// A communicator built with the single-process constructor carries `world`
// virtual ranks on one GPU; its methods then take one pointer per virtual
// rank and run all ranks as one cooperative launch.  The kernel tests use
// that form to check indexing and the flag protocol on a single device.
//
// The header is free of CUDA and torch types so that the process group and
// the bindings can include it cheaply; streams travel as void*.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../core/config.hpp"
#include "../net/kv_store.hpp"
#include "dtypes.hpp"

namespace mccl {

class SymmMesh;
struct SymmAlloc;

class DeviceComm {
 public:
  // One process per GPU; collective over the group.
  DeviceComm(KVStore* store, int rank, int world, int device, const std::string& prefix, const EnvConfig& cfg,
             int64_t timeout_ms);
  // Single process, `world` virtual ranks on `device`.
  DeviceComm(int world, int device, const EnvConfig& cfg);
  ~DeviceComm();
  DeviceComm(const DeviceComm&) = delete;
  DeviceComm& operator=(const DeviceComm&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }
  int device() const { return device_; }
  int nlocal() const { return nlocal_; }  // pointers expected per call (1 unless emulating)
  bool nvls_available() const;
  size_t arena_bytes() const;
  const char* symm_mode() const;

  // Schedule an allreduce of `numel` elements would run with.  Explicit
  // requests are honoured (NVLS falls back to two-shot when the multicast
  // object is missing, the op is not SUM/AVG or the type is not a float type;
  // RING needs numel >= world, else TREE, as in the reference).  AUTO picks
  // one-shot up to tree_below wire bytes, else NVLS when available, else
  // two-shot.
  Algo decide_allreduce(Algo requested, size_t numel, DType t, RedOp op, WireDtype wire, int64_t tree_below) const;

  // ins / outs hold nlocal() pointers.  outs[i] may equal ins[i].
  Algo allreduce(const void* const* ins, void* const* outs, size_t numel, DType t, RedOp op, Algo requested,
                 WireDtype wire, int64_t tree_below, void* stream);
  void broadcast(void* const* datas, size_t nbytes, int root, void* stream);
  void allgather(const void* const* ins, void* const* outs, size_t nbytes_per_rank, void* stream);
  // ins: world*numel elements each, outs: numel elements each.
  void reduce_scatter(const void* const* ins, void* const* outs, size_t numel, DType t, RedOp op, WireDtype wire,
                      void* stream);
  // Offsets / lengths in bytes: [virtual rank][peer].
  void alltoallv(const void* const* ins, void* const* outs, const std::vector<std::vector<size_t>>& in_off,
                 const std::vector<std::vector<size_t>>& in_len, const std::vector<std::vector<size_t>>& out_off,
                 const std::vector<std::vector<size_t>>& out_len, void* stream);
  void barrier(void* stream);

  // Point-to-point: the n-th send to a peer pairs with the n-th recv from it on the other side (tags are
  // not matched, as with NCCL).  The data travels through a two-buffer slot per (receiver, source) in
  // peer-mapped memory, so a message of up to two slots (MCCL_P2P_SLOT_MB each, 4 MiB by default) is
  // sent without the receiver having arrived; longer ones are streamed as the receiver drains them.
  // These launches use flags and memory of their own and are not ordered against the collectives, so a
  // process group may run sends, receives and collectives on three different streams.
  void send(const void* data, size_t nbytes, int peer, void* stream);
  void recv(void* data, size_t nbytes, int peer, void* stream);
  // Single-GPU emulation: ops[v] = {buffer, peer or -1, is_send} for virtual rank v, one cooperative launch.
  struct P2POp {
    void* buf = nullptr;
    int peer = -1;
    bool is_send = false;
  };
  void p2p_emulated(const std::vector<P2POp>& ops, size_t nbytes, void* stream);
  size_t p2p_slot_bytes() const;

  // Single-pointer conveniences for the one-process-per-GPU case.
  Algo allreduce(const void* in, void* out, size_t numel, DType t, RedOp op, Algo requested, WireDtype wire,
                 int64_t tree_below, void* stream) {
    return allreduce(&in, &out, numel, t, op, requested, wire, tree_below, stream);
  }
  void broadcast(void* data, size_t nbytes, int root, void* stream) { broadcast(&data, nbytes, root, stream); }
  void allgather(const void* in, void* out, size_t nbytes_per_rank, void* stream) {
    allgather(&in, &out, nbytes_per_rank, stream);
  }
  void reduce_scatter(const void* in, void* out, size_t numel, DType t, RedOp op, WireDtype wire, void* stream) {
    reduce_scatter(&in, &out, numel, t, op, wire, stream);
  }
  void alltoallv(const void* in, const std::vector<size_t>& in_off, const std::vector<size_t>& in_len, void* out,
                 const std::vector<size_t>& out_off, const std::vector<size_t>& out_len, void* stream) {
    alltoallv(&in, &out, {in_off}, {in_len}, {out_off}, {out_len}, stream);
  }

  // Symmetric heap: collective allocation of `bytes` on every rank, mapped
  // into every rank's address space (and bound to a multicast object when
  // NVLS is available).
  std::shared_ptr<SymmAlloc> symm_alloc(size_t bytes);
  // In-place allreduce (SUM / AVG) of a region of a symmetric allocation: no
  // staging copy; in-switch reduction when the allocation has a multicast
  // mapping, otherwise peers' copies are read directly.
  Algo allreduce_symm(const SymmAlloc& buf, size_t byte_offset, size_t numel, DType t, RedOp op, void* stream);

  // 0 while healthy; otherwise the code a kernel wrote when a wait ran out.
  int status() const;
  // Throws TimeoutError with peer / phase decoded from the status word.
  void check_status() const;
  // MCCL_DEBUG_BOUNDS=1 only: synchronises the device and verifies the pattern behind the staging arena.
  void check_canaries() const;
  bool debug_bounds() const { return cfg_.debug_bounds; }
  // MCCL_DEBUG_BOUNDS=1 only, for tests: the kernels are told the arena ends after `bytes` (0 = its real end),
  // which makes their extent check refuse launches the host-side checks let through.
  void set_debug_arena_limit(size_t bytes);
  void clear_status();
  // Host-made fault for tests: this rank withholds its signals during the
  // next `count` collectives, so the peers' bounded waits run out.
  void inject_skip_signals(int count);
  // Overrides the bound of every device-side wait (milliseconds).
  void set_device_timeout_ms(int64_t ms);
  int64_t device_timeout_ms() const;
  // Geometry of the collective kernels launched from now on: at most `max_ctas` CTAs of `threads` threads
  // (0 keeps the current value, threads < 0 restores the default).  512-thread CTAs need a whole register file and so only run on SMs that
  // hold no persistent GEMM CTA; a trainer that leaves k SMs free of GEMM work asks for (k, 512).
  void set_launch_shape(int max_ctas, int threads);   // max_ctas < 0: back to the defaults (and automatic shaping)
  int max_ctas() const;
  bool launch_shape_auto() const;   // no shape was asked for: large messages take every CTA, 512 threads each
  int launch_threads() const;   // 0 = kernel default

  SymmMesh& mesh() { return *mesh_; }
  uint64_t launches() const { return launches_; }

 private:
  struct Impl;
  void init_common();
  int rank_ = 0, world_ = 1, device_ = 0, nlocal_ = 1;
  EnvConfig cfg_;
  std::unique_ptr<SymmMesh> mesh_;
  std::unique_ptr<Impl> impl_;
  uint64_t launches_ = 0;
  int64_t group_timeout_ms_ = 0;
};

}  // namespace mccl
