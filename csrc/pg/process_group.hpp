// The c10d backend registered as "mccl" for CPU and CUDA tensors.
//
// Parity: the reference's ProcessGroupMCCL overrides broadcast, allreduce,
// allgather, _allgather_base, reduce_scatter, _reduce_scatter_base,
// alltoall_base, alltoall, barrier, send and recv
// (csrc/backend/ProcessGroupMCCL.hpp:28-102) for MPS tensors over one TCP
// socket per peer.  This class keeps the name, the environment semantics
// (MCCL_ALLREDUCE_ALGO, MCCL_TREE_BELOW and MCCL_WIRE_DTYPE re-read on every
// call) and the world==1 fast paths, and widens the surface with reduce,
// gather, scatter and the coalesced variants that DDP and FSDP use on CUDA.
//
// Two data planes:
//   * CPU tensors: TcpMesh + host algorithms, run in submission order on the
//     Progress thread;
//   * CUDA tensors: DeviceComm (peer-mapped symmetric arena + signal pads over
//     NVLink) driving the collective kernels on the group's comm stream;
//     send/recv go to an NCCL point-to-point group supplied by Python.
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <atomic>
#include <functional>
#include <memory>
#include <mutex>

#include "../core/config.hpp"
#include "../engine/progress.hpp"
#include "../net/kv_store.hpp"
#include "../net/tcp_mesh.hpp"
#include "dtypes.hpp"
#include "work.hpp"

namespace mccl {

class DeviceComm;     // csrc/pg/device_comm.hpp
class StreamWatcher;  // completion thread for CUDA collectives (process_group.cpp)

// c10d::Store seen through the transport-level KVStore interface.
class StoreAdapter : public KVStore {
 public:
  explicit StoreAdapter(c10::intrusive_ptr<c10d::Store> s) : store_(std::move(s)) {}
  void set(const std::string& key, const std::vector<uint8_t>& value) override { store_->set(key, value); }
  std::vector<uint8_t> get(const std::string& key, int64_t timeout_ms) override;
  int64_t add(const std::string& key, int64_t delta) override { return store_->add(key, delta); }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
};

class ProcessGroupMCCL : public c10d::Backend {
 public:
  struct Options : c10d::Backend::Options {
    explicit Options(std::chrono::milliseconds t = std::chrono::minutes(30)) : c10d::Backend::Options("mccl", t) {}
  };

  ProcessGroupMCCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                   std::chrono::milliseconds timeout);
  ~ProcessGroupMCCL() override;

  static c10::intrusive_ptr<c10d::Backend> create(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                  std::chrono::milliseconds timeout);

  const std::string getBackendName() const override { return "mccl"; }
  bool supportsCoalescing() const override { return false; }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                           const c10d::BroadcastOptions& opts = c10d::BroadcastOptions()) override;
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts = c10d::AllreduceOptions()) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(
      std::vector<at::Tensor>& tensors,
      const c10d::AllreduceCoalescedOptions& opts = c10d::AllreduceCoalescedOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors,
                                        const c10d::ReduceOptions& opts = c10d::ReduceOptions()) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputTensors,
                                           std::vector<at::Tensor>& inputTensors,
                                           const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& outputBuffer, at::Tensor& inputBuffer,
                                                 const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& outputTensorLists,
                                                     std::vector<at::Tensor>& inputTensors,
                                                     const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputTensors,
                                        std::vector<at::Tensor>& inputTensors,
                                        const c10d::GatherOptions& opts = c10d::GatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputTensors,
                                         std::vector<std::vector<at::Tensor>>& inputTensors,
                                         const c10d::ScatterOptions& opts = c10d::ScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(
      std::vector<at::Tensor>& outputTensors, std::vector<std::vector<at::Tensor>>& inputTensors,
      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(
      at::Tensor& outputBuffer, at::Tensor& inputBuffer,
      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& outputBuffer, at::Tensor& inputBuffer,
                                               std::vector<int64_t>& outputSplitSizes,
                                               std::vector<int64_t>& inputSplitSizes,
                                               const c10d::AllToAllOptions& opts = c10d::AllToAllOptions()) override;
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outputTensors,
                                          std::vector<at::Tensor>& inputTensors,
                                          const c10d::AllToAllOptions& opts = c10d::AllToAllOptions()) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dstRank, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int srcRank, int tag) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts = c10d::BarrierOptions()) override;

  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return op_seq_.load(); }
  void abort() override;
  void shutdown() override;
  void eagerConnectSingleDevice(at::Device device) override;

  // ---- extras reachable from Python ----
  // allreduce with the algorithm and the wire dtype given as arguments instead of being read from
  // MCCL_ALLREDUCE_ALGO / MCCL_WIRE_DTYPE (what a DDP communication hook needs: it runs on autograd's
  // thread and must not edit the process environment around each bucket).
  c10::intrusive_ptr<c10d::Work> allreduceWith(std::vector<at::Tensor>& tensors, RedOp op, Algo algo, WireDtype wire);
  // Supplies the lazily built NCCL group used for CUDA send/recv when MCCL_P2P=nccl.
  void setP2PFactory(std::function<c10::intrusive_ptr<c10d::Backend>()> f) { p2p_factory_ = std::move(f); }
  // Device communicator of this group for `device` (built collectively on first use).
  std::shared_ptr<DeviceComm> deviceComm(at::Device device);
  // Name of the algorithm the last allreduce used (for tests and logs).
  std::string lastAlgo() const;
  // Throws if a device-side wait of this group timed out.
  void checkDeviceStatus();
  // Size of the symmetric staging arena this group's device communicator will allocate (before its first
  // CUDA collective).  Sub-groups get a smaller arena than the world group: messages beyond it go in pieces.
  void setArenaBytes(int64_t bytes) { cfg_.arena_bytes = bytes; }
  // The group's key-value store and timeout (used by the distributed-memory fabric).
  KVStore* kv() { return kv_.get(); }
  int64_t timeoutMs() const { return timeout_.count(); }

 private:
  using Body = std::function<void()>;
  c10::intrusive_ptr<c10d::Work> submitHost(c10d::OpType op, const char* title, uint64_t bytes,
                                            std::vector<at::Tensor> outputs, Body body);
  c10::intrusive_ptr<c10d::Work> submitStream(c10d::OpType op, const char* title, uint64_t bytes,
                                              const std::string& algo, std::vector<at::Tensor> inputs,
                                              std::vector<at::Tensor> outputs, at::Device device,
                                              const std::function<void(DeviceComm&, void* /*cudaStream_t*/)>& launch,
                                              int lane = 0);
  c10::intrusive_ptr<c10d::Backend> p2p();
  TcpMesh& mesh();
  StreamWatcher& watcher();

  c10::intrusive_ptr<c10d::Store> store_;
  std::unique_ptr<StoreAdapter> kv_;
  EnvConfig cfg_;
  std::chrono::milliseconds timeout_;
  std::unique_ptr<TcpMesh> mesh_;
  std::unique_ptr<Progress> engine_;
  std::mutex dev_mu_;
  std::shared_ptr<DeviceComm> dev_;
  std::function<c10::intrusive_ptr<c10d::Backend>()> p2p_factory_;
  c10::intrusive_ptr<c10d::Backend> p2p_;
  std::atomic<uint64_t> op_seq_{0};
  std::atomic<uint64_t> barrier_seq_{0};
  mutable std::mutex algo_mu_;
  std::string last_algo_;
  std::atomic<bool> aborted_{false};
  std::mutex watcher_mu_;
  std::shared_ptr<StreamWatcher> watcher_;
  bool use_nccl_p2p_ = false;    // MCCL_P2P=nccl: CUDA send/recv through the NCCL comparison arm
  bool device_metrics_ = true;   // MCCL_DEVICE_METRICS: time CUDA collectives with an event pair
};

}  // namespace mccl
