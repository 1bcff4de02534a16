// c10d::Work for the mccl backend.
//
// Parity: the reference's WorkMCCL offers isCompleted / isSuccess / exception /
// wait(timeout) / result / getFuture, returns false from wait on a timeout,
// rethrows a stored exception, and types its Future as List[Tensor] on the
// tensors' devices (csrc/backend/WorkMCCL.cpp:10-104).  Two kinds of work
// exist here:
//   * host work: finished by the progress engine thread (CPU tensors);
//   * stream work: a CUDA collective already enqueued on the group's comm
//     stream.  wait() makes the caller's current stream wait for the
//     completion event (no host block, like NCCL) unless MCCL_BLOCKING_WAIT=1,
//     and the Future is completed at enqueue time with the comm stream
//     current so that DDP's reducer chains its callbacks on the right stream.
#pragma once

#include <torch/csrc/distributed/c10d/Work.hpp>

#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <vector>

namespace mccl {

// Opaque CUDA event holder implemented in the CUDA translation unit so that
// this header does not need cuda_runtime.h.
struct StreamCompletion {
  virtual ~StreamCompletion() = default;
  virtual bool query() = 0;                  // true when the device finished
  virtual void block_current_stream() = 0;   // stream-ordered wait
  virtual bool synchronize(int64_t timeout_ms) = 0;  // host wait; false on timeout
  virtual void check_status() = 0;           // throws if a device wait timed out
};

class WorkMCCL : public c10d::Work {
 public:
  WorkMCCL(int rank, c10d::OpType op, const char* title, std::vector<at::Tensor> outputs);
  ~WorkMCCL() override = default;

  static c10::intrusive_ptr<WorkMCCL> completed(int rank, c10d::OpType op, const char* title,
                                                std::vector<at::Tensor> outputs);

  bool isCompleted() override;
  bool isSuccess() const override;
  std::exception_ptr exception() const override;
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
  void synchronize() override;
  std::vector<at::Tensor> result() override;
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;

  // Host work: called by the engine thread.
  void markDone();
  void markFailed(std::exception_ptr e);
  // Stream work: attaches the completion event and completes the Future.
  // Must be called with the comm stream set as the current stream.
  void attachStream(std::shared_ptr<StreamCompletion> sc, bool blocking_wait);
  // Stream work: the completion thread found that the collective failed on the device (a bounded
  // wait ran out).  wait(), isSuccess() and exception() report it from then on.
  void markStreamFailed(std::exception_ptr e);

 private:
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
  std::shared_ptr<StreamCompletion> stream_done_;
  bool blocking_wait_ = false;
  mutable std::mutex wmu_;
  std::condition_variable wcv_;
  bool done_ = false;
  std::exception_ptr error_;
};

}  // namespace mccl
