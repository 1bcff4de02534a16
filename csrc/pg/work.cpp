#include "work.hpp"

#include <ATen/core/ivalue.h>
#include <c10/core/DeviceGuard.h>

namespace mccl {

namespace {
std::vector<c10::Device> cuda_devices_of(const std::vector<at::Tensor>& ts) {
  std::vector<c10::Device> devs;
  for (auto& t : ts) {
    if (!t.defined() || !t.device().is_cuda()) continue;
    bool seen = false;
    for (auto& d : devs) seen = seen || d == t.device();
    if (!seen) devs.push_back(t.device());
  }
  return devs;
}
}  // namespace

WorkMCCL::WorkMCCL(int rank, c10d::OpType op, const char* title, std::vector<at::Tensor> outputs)
    : c10d::Work(rank, op, title), outputs_(std::move(outputs)) {
  future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                     cuda_devices_of(outputs_));
}

c10::intrusive_ptr<WorkMCCL> WorkMCCL::completed(int rank, c10d::OpType op, const char* title,
                                                 std::vector<at::Tensor> outputs) {
  auto w = c10::make_intrusive<WorkMCCL>(rank, op, title, std::move(outputs));
  w->markDone();
  return w;
}

bool WorkMCCL::isCompleted() {
  std::lock_guard<std::mutex> g(wmu_);
  if (error_) return true;
  if (stream_done_) return stream_done_->query();
  return done_;
}

bool WorkMCCL::isSuccess() const {
  std::lock_guard<std::mutex> g(wmu_);
  if (error_) return false;
  if (stream_done_) return stream_done_->query();
  return done_;
}

std::exception_ptr WorkMCCL::exception() const {
  std::lock_guard<std::mutex> g(wmu_);
  return error_;
}

bool WorkMCCL::wait(std::chrono::milliseconds timeout) {
  if (stream_done_) {
    {
      std::lock_guard<std::mutex> g(wmu_);
      if (error_) std::rethrow_exception(error_);
    }
    if (blocking_wait_) {
      bool ok = stream_done_->synchronize(timeout == kNoTimeout ? -1 : timeout.count());
      if (!ok) return false;
      stream_done_->check_status();
    } else {
      stream_done_->block_current_stream();
      // Stream-ordered wait: the host does not block.  If the device has already finished this
      // collective, a wait that ran out inside it is known now and is reported on this Work.
      if (stream_done_->query()) stream_done_->check_status();
    }
    return true;
  }
  std::unique_lock<std::mutex> g(wmu_);
  if (timeout == kNoTimeout) {
    wcv_.wait(g, [&] { return done_; });
  } else if (!wcv_.wait_for(g, timeout, [&] { return done_; })) {
    return false;
  }
  if (error_) std::rethrow_exception(error_);
  return true;
}

void WorkMCCL::synchronize() {
  if (stream_done_) stream_done_->block_current_stream();
}

std::vector<at::Tensor> WorkMCCL::result() { return outputs_; }

c10::intrusive_ptr<c10::ivalue::Future> WorkMCCL::getFuture() { return future_; }

void WorkMCCL::markDone() {
  {
    std::lock_guard<std::mutex> g(wmu_);
    if (done_) return;
    done_ = true;
  }
  wcv_.notify_all();
  if (!future_->completed()) future_->markCompleted(c10::IValue(outputs_));
}

void WorkMCCL::markFailed(std::exception_ptr e) {
  {
    std::lock_guard<std::mutex> g(wmu_);
    if (done_) return;
    done_ = true;
    error_ = e;
  }
  wcv_.notify_all();
  if (!future_->completed()) future_->setError(e);
}

void WorkMCCL::markStreamFailed(std::exception_ptr e) {
  std::lock_guard<std::mutex> g(wmu_);
  if (!error_) error_ = e;
}

void WorkMCCL::attachStream(std::shared_ptr<StreamCompletion> sc, bool blocking_wait) {
  {
    std::lock_guard<std::mutex> g(wmu_);
    stream_done_ = std::move(sc);
    blocking_wait_ = blocking_wait;
    done_ = true;
  }
  // The Future records an event on the current (comm) stream of each device.
  if (!future_->completed()) future_->markCompleted(c10::IValue(outputs_));
}

}  // namespace mccl
