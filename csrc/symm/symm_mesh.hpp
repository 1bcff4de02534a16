// Symmetric memory across the GPUs of one process group.
//
// Every rank allocates a block of the same size and maps every other rank's
// block into its own address space, so kernels reach peer memory over NVLink
// with ordinary loads and stores; where the fabric offers it, the blocks are
// also bound to one multicast object whose mapping feeds multimem.ld_reduce /
// multimem.st (in-switch reduction).
//
// This is the NVLink stand-in for the reference's RDMA plumbing: its
// SharedBuffer (page-aligned buffer registered with every protection domain,
// csrc/transport/rdma/SharedBuffer.cpp:22-99), the per-peer RdmaConnection
// with its exchanged RdmaDestination (csrc/transport/rdma/RdmaConnection.hpp:15-116)
// and the memory-region registration of the DistributedMemoryManager
// (csrc/dmem/DistributedMemoryManager.cpp:104-148).  Instead of queue pairs
// and rkeys there are allocation handles, exported as POSIX file descriptors
// and passed between the ranks over a Unix socket.
//
// Three modes:
//   VMM   cuMemCreate + fd export/import + cuMemMap (multicast capable)
//   IPC   cudaMalloc + cudaIpcGetMemHandle (fallback when fd export is refused)
//   LOCAL all "ranks" are blocks on one GPU in one process (kernel tests)
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

#include "../core/config.hpp"
#include "../net/kv_store.hpp"

namespace mccl {

constexpr int kSymmMaxRanks = 8;

struct SymmAlloc {
  size_t bytes = 0;                      // usable bytes (as requested, rounded to the mapping granularity)
  int world = 1;
  int rank = 0;                          // owner's rank (LOCAL mode: 0)
  void* ptrs[kSymmMaxRanks] = {};        // ptrs[r] = rank r's block as mapped in this process
  void* mc_ptr = nullptr;                // multicast mapping, or nullptr
  uint32_t id = 0;                       // allocation number, equal on all ranks
  void* local() const { return ptrs[rank]; }
  struct Priv;
  std::shared_ptr<Priv> priv;            // handles and reservations; released with the last reference
};

class SymmMesh {
 public:
  enum class Mode { VMM, IPC, LOCAL };

  // One process per GPU.  Collective: every rank of the group constructs it.
  SymmMesh(KVStore* store, int rank, int world, int device, const std::string& prefix, const EnvConfig& cfg,
           int64_t timeout_ms);
  // Single process, `world` virtual ranks on `device`.
  SymmMesh(int world, int device);
  ~SymmMesh();
  SymmMesh(const SymmMesh&) = delete;
  SymmMesh& operator=(const SymmMesh&) = delete;

  // Collective.  The block is zero-filled on return and stays mapped until the
  // returned object (and every copy of it) is gone.
  std::shared_ptr<SymmAlloc> alloc(size_t bytes, bool want_multicast);

  Mode mode() const { return mode_; }
  const char* mode_name() const { return mode_ == Mode::VMM ? "vmm" : mode_ == Mode::IPC ? "ipc" : "local"; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  int device() const { return device_; }
  // True when every rank reported multicast support and the user did not turn NVLS off.
  bool multicast_usable() const { return multicast_; }
  // Store barrier with a caller-chosen unique tag (setup-time only).
  void store_barrier(const std::string& tag);

 private:
  struct FdServer;
  std::shared_ptr<SymmAlloc> alloc_vmm(size_t bytes, bool want_multicast);
  std::shared_ptr<SymmAlloc> alloc_ipc(size_t bytes);
  std::shared_ptr<SymmAlloc> alloc_local(size_t bytes);
  bool all_ranks_agree(const std::string& what, bool mine);

  KVStore* store_ = nullptr;
  int rank_ = 0, world_ = 1, device_ = 0;
  std::string prefix_;
  int64_t timeout_ms_ = 0;
  Mode mode_ = Mode::LOCAL;
  bool multicast_ = false;
  uint32_t next_id_ = 0;
  std::unique_ptr<FdServer> server_;
  std::vector<std::string> peer_names_;   // fd servers of the peers (VMM mode), looked up at the first allocation
};

}  // namespace mccl
