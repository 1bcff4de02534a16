#include "process_group.hpp"

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>

#include <condition_variable>
#include <deque>
#include <map>
#include <thread>

#include "../core/errors.hpp"
#include "../core/log.hpp"
#include "../engine/metrics.hpp"
#include "cpu_algos.hpp"
#include "device_comm.hpp"

namespace mccl {

// ------------------------------------------------------------ small helpers --
std::vector<uint8_t> StoreAdapter::get(const std::string& key, int64_t timeout_ms) {
  try {
    store_->wait({key}, std::chrono::milliseconds(timeout_ms));
  } catch (const std::exception& e) {
    MCCL_CHECK_T(false, TimeoutError, "store: key '" << key << "' not set within " << timeout_ms << " ms");
  }
  return store_->get(key);
}

namespace {

DType to_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return DType::F32;
    case at::kDouble: return DType::F64;
    case at::kHalf: return DType::F16;
    case at::kBFloat16: return DType::BF16;
    case at::kChar: return DType::I8;
    case at::kShort: return DType::I16;
    case at::kInt: return DType::I32;
    case at::kLong: return DType::I64;
    case at::kByte: return DType::U8;
    case at::kBool: return DType::BOOL;
    default: MCCL_CHECK_T(false, TensorError, "unsupported dtype " << c10::toString(t));
  }
  return DType::F32;
}

RedOp to_redop(const c10d::ReduceOp& op) {
  switch (op.op_) {
    case c10d::ReduceOp::SUM: return RedOp::SUM;
    case c10d::ReduceOp::AVG: return RedOp::AVG;
    case c10d::ReduceOp::PRODUCT: return RedOp::PRODUCT;
    case c10d::ReduceOp::MIN: return RedOp::MIN;
    case c10d::ReduceOp::MAX: return RedOp::MAX;
    case c10d::ReduceOp::BAND: return RedOp::BAND;
    case c10d::ReduceOp::BOR: return RedOp::BOR;
    case c10d::ReduceOp::BXOR: return RedOp::BXOR;
    default: MCCL_CHECK(false, "unsupported reduce op " << static_cast<int>(op.op_));
  }
  return RedOp::SUM;
}

// Same acceptance rules as the reference's TensorChecks.hpp:10-58, with CUDA
// in place of MPS: dense, contiguous, non-empty, known dtype.
void check_tensor(const at::Tensor& t, const char* what) {
  MCCL_CHECK_TENSOR(t.defined(), what << ": undefined tensor");
  MCCL_CHECK_TENSOR(t.device().is_cpu() || t.device().is_cuda(),
                    what << ": tensor must live on CPU or CUDA, got " << t.device());
  MCCL_CHECK_TENSOR(t.layout() == at::kStrided, what << ": tensor must be dense");
  MCCL_CHECK_TENSOR(t.is_contiguous(), what << ": tensor must be contiguous");
  (void)to_dtype(t.scalar_type());
}
void check_single(const std::vector<at::Tensor>& ts, const char* what) {
  MCCL_CHECK_TENSOR(ts.size() == 1, what << ": expected exactly one tensor, got " << ts.size());
  check_tensor(ts[0], what);
}
void check_same(const at::Tensor& a, const at::Tensor& b, const char* what) {
  MCCL_CHECK_TENSOR(a.scalar_type() == b.scalar_type(), what << ": dtype mismatch");
  MCCL_CHECK_TENSOR(a.device() == b.device(), what << ": device mismatch");
}
size_t nbytes(const at::Tensor& t) { return static_cast<size_t>(t.numel()) * t.element_size(); }

// Element types the device reduce kernels cover directly.
bool device_reducible(at::ScalarType t) {
  return t == at::kFloat || t == at::kHalf || t == at::kBFloat16 || t == at::kDouble || t == at::kInt ||
         t == at::kLong;
}

class EventCompletion : public StreamCompletion {
 public:
  EventCompletion(std::shared_ptr<DeviceComm> dev, c10::DeviceIndex idx, bool host_sync_on_wait, bool timed)
      : ev_(timed ? cudaEventDefault : cudaEventDisableTiming), start_(timed ? cudaEventDefault : cudaEventDisableTiming),
        dev_(std::move(dev)), idx_(idx), host_sync_(host_sync_on_wait), timed_(timed) {}
  void record_start(const c10::cuda::CUDAStream& s) {
    if (timed_) start_.record(s);
  }
  void record(const c10::cuda::CUDAStream& s) { ev_.record(s); }
  // Device time between the two events in milliseconds (only after query() returned true); < 0 when untimed.
  double device_ms() {
    if (!timed_) return -1.0;
    return static_cast<double>(start_.elapsed_time(ev_));
  }
  int device_status() { return dev_ ? dev_->status() : 0; }
  bool query() override { return ev_.query(); }
  void block_current_stream() override {
    ev_.block(c10::cuda::getCurrentCUDAStream(idx_));
    if (host_sync_ && cudaStreamIsCapturingNow() == false) {
      ev_.synchronize();
      if (dev_) dev_->check_status();
    }
  }
  bool synchronize(int64_t timeout_ms) override {
    if (timeout_ms < 0) {
      ev_.synchronize();
      return true;
    }
    auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    while (!ev_.query()) {
      if (std::chrono::steady_clock::now() > deadline) return false;
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    return true;
  }
  void check_status() override {
    if (dev_) dev_->check_status();
  }

 private:
  bool cudaStreamIsCapturingNow() {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(c10::cuda::getCurrentCUDAStream(idx_).stream(), &st);
    return st != cudaStreamCaptureStatusNone;
  }
  at::cuda::CUDAEvent ev_;
  at::cuda::CUDAEvent start_;
  std::shared_ptr<DeviceComm> dev_;
  c10::DeviceIndex idx_;
  bool host_sync_;
  bool timed_;
};

bool stream_capturing(const c10::cuda::CUDAStream& s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s.stream(), &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return st != cudaStreamCaptureStatusNone;
}

std::mutex g_stream_mu;
std::map<std::pair<const void*, int>, c10::cuda::CUDAStream> g_comm_streams;

// lane 0: collectives; lane 1: sends; lane 2: receives (a rank's send and receive of one exchange must be
// able to run at the same time, and neither may queue behind a collective that waits for other ranks).
c10::cuda::CUDAStream comm_stream_for(const void* pg, c10::DeviceIndex idx, int lane = 0) {
  std::lock_guard<std::mutex> g(g_stream_mu);
  auto key = std::make_pair(pg, static_cast<int>(idx) * 4 + lane);
  auto it = g_comm_streams.find(key);
  if (it == g_comm_streams.end())
    it = g_comm_streams.emplace(key, c10::cuda::getStreamFromPool(/*isHighPriority=*/true, idx)).first;
  return it->second;
}

}  // namespace

// ------------------------------------------------------- completion thread --
// Follows every CUDA collective that was enqueued outside a graph capture: when its end event
// has fired it stores the device time (CUDA event pair) in the metrics record, and when the
// pinned status word says that a bounded device wait ran out it fails THAT Work with a
// TimeoutError, the counterpart of the reference's finishWithException on its progress thread
// (csrc/backend/ProcessGroupMCCL.cpp:60-68).
class StreamWatcher {
 public:
  struct Item {
    c10::intrusive_ptr<WorkMCCL> work;
    std::shared_ptr<EventCompletion> done;
    uint64_t metric_seq = 0;
  };
  StreamWatcher() : thread_([this] { run(); }) {}
  ~StreamWatcher() { stop(); }
  void watch(Item item) {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stopping_) {
        Metrics::global().op_end(item.metric_seq, false);
        return;
      }
      q_.push_back(std::move(item));
    }
    cv_.notify_one();
  }
  // Returns once every watched op has been seen to finish (or `ms` passed).
  void drain(int64_t ms) {
    auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(ms);
    std::unique_lock<std::mutex> g(mu_);
    idle_cv_.wait_until(g, deadline, [&] { return q_.empty() && !busy_; });
  }
  void stop() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stopping_) return;
      stopping_ = true;
    }
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
  }
  bool failed() const { return failed_.load(); }

 private:
  void run() {
    for (;;) {
      Item item;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [&] { return stopping_ || !q_.empty(); });
        if (q_.empty()) return;   // stopping and nothing left
        item = std::move(q_.front());
        q_.pop_front();
        busy_ = true;
      }
      finish(item);
      {
        std::lock_guard<std::mutex> g(mu_);
        busy_ = false;
      }
      idle_cv_.notify_all();
    }
  }
  void finish(Item& item) {
    // After stop() the remaining ops get two seconds; a process that is going away must not hang here.
    auto give_up = std::chrono::steady_clock::time_point::max();
    bool done = false;
    int spins = 0;
    try {
      for (;;) {
        if (item.done->query()) {
          done = true;
          break;
        }
        bool stopping;
        {
          std::lock_guard<std::mutex> g(mu_);
          stopping = stopping_;
        }
        if (stopping) {
          if (give_up == std::chrono::steady_clock::time_point::max())
            give_up = std::chrono::steady_clock::now() + std::chrono::seconds(2);
          if (std::chrono::steady_clock::now() > give_up) break;
        }
        if (++spins < 200) std::this_thread::yield();
        else std::this_thread::sleep_for(std::chrono::microseconds(50));
      }
      if (done) {
        const double ms = item.done->device_ms();
        if (ms >= 0) Metrics::global().record_phase(item.metric_seq, "device", ms);
      }
      bool bad = false;
      if (done && item.done->device_status() != 0) {
        try {
          item.done->check_status();
        } catch (...) {
          bad = true;
          failed_.store(true);
          item.work->markStreamFailed(std::current_exception());
        }
      }
      Metrics::global().op_end(item.metric_seq, bad);
    } catch (...) {
      // a CUDA error while querying (context torn down, sticky fault): the op cannot be vouched for
      failed_.store(true);
      item.work->markStreamFailed(std::current_exception());
      Metrics::global().op_end(item.metric_seq, true);
    }
  }

  std::mutex mu_;
  std::condition_variable cv_, idle_cv_;
  std::deque<Item> q_;
  bool stopping_ = false, busy_ = false;
  std::atomic<bool> failed_{false};
  std::thread thread_;
};

// ------------------------------------------------------------- construction --
ProcessGroupMCCL::ProcessGroupMCCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                   std::chrono::milliseconds timeout)
    : c10d::Backend(rank, size), store_(store), kv_(new StoreAdapter(store)), cfg_(EnvConfig::from_env()),
      timeout_(timeout) {
  set_log_rank(rank);
  device_metrics_ = env::flag("MCCL_DEVICE_METRICS", true);
  use_nccl_p2p_ = env::str("MCCL_P2P") == "nccl";
  if (size > 1) {
    mesh_.reset(new TcpMesh(kv_.get(), rank, size, timeout.count(), "mccl", cfg_));
    engine_.reset(new Progress(static_cast<size_t>(cfg_.max_queue_depth)));
  }
  MCCL_INFO("process group up: rank " << rank << " of " << size);
}

ProcessGroupMCCL::~ProcessGroupMCCL() {
  try {
    shutdown();
  } catch (...) {
  }
  std::lock_guard<std::mutex> g(g_stream_mu);
  for (auto it = g_comm_streams.begin(); it != g_comm_streams.end();)
    it = (it->first.first == this) ? g_comm_streams.erase(it) : std::next(it);
}

c10::intrusive_ptr<c10d::Backend> ProcessGroupMCCL::create(const c10::intrusive_ptr<c10d::Store>& store, int rank,
                                                           int size, std::chrono::milliseconds timeout) {
  return c10::make_intrusive<ProcessGroupMCCL>(store, rank, size, timeout);
}

StreamWatcher& ProcessGroupMCCL::watcher() {
  std::lock_guard<std::mutex> g(watcher_mu_);
  if (!watcher_) watcher_.reset(new StreamWatcher());
  return *watcher_;
}

void ProcessGroupMCCL::shutdown() {
  {
    std::lock_guard<std::mutex> g(watcher_mu_);
    if (watcher_) watcher_->stop();
  }
  if (engine_) engine_->shutdown();
  if (mesh_) Metrics::global().record_transport_bytes(mesh_->bytes_sent(), mesh_->bytes_received());
}

void ProcessGroupMCCL::abort() {
  aborted_ = true;
  if (mesh_) mesh_->close_all();  // wakes any host transfer with a TransportError
  if (engine_) engine_->shutdown();
}

TcpMesh& ProcessGroupMCCL::mesh() {
  MCCL_CHECK(mesh_ != nullptr, "no TCP mesh in a single-rank group");
  return *mesh_;
}

std::string ProcessGroupMCCL::lastAlgo() const {
  std::lock_guard<std::mutex> g(algo_mu_);
  return last_algo_;
}

std::shared_ptr<DeviceComm> ProcessGroupMCCL::deviceComm(at::Device device) {
  MCCL_CHECK_TENSOR(device.is_cuda(), "device communicator needs a CUDA device");
  std::lock_guard<std::mutex> g(dev_mu_);
  if (!dev_) {
    MCCL_CHECK(!aborted_, "process group was aborted");
    dev_ = std::make_shared<DeviceComm>(kv_.get(), getRank(), getSize(), static_cast<int>(device.index()), "mccl/dev",
                                        cfg_, timeout_.count());
  }
  MCCL_CHECK_TENSOR(dev_->device() == device.index(),
                    "this group is bound to cuda:" << dev_->device() << " but got a tensor on " << device);
  return dev_;
}

void ProcessGroupMCCL::eagerConnectSingleDevice(at::Device device) {
  if (device.is_cuda() && getSize() > 1) deviceComm(device);
}

void ProcessGroupMCCL::checkDeviceStatus() {
  std::lock_guard<std::mutex> g(dev_mu_);
  if (dev_) dev_->check_status();
}

c10::intrusive_ptr<c10d::Backend> ProcessGroupMCCL::p2p() {
  if (!p2p_) {
    MCCL_CHECK(static_cast<bool>(p2p_factory_), "send/recv on CUDA tensors needs the NCCL p2p group (none configured)");
    p2p_ = p2p_factory_();
    MCCL_CHECK(p2p_ != nullptr, "NCCL p2p group factory returned nothing");
  }
  return p2p_;
}

// --------------------------------------------------------------- submission --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::submitHost(c10d::OpType op, const char* title, uint64_t bytes,
                                                            std::vector<at::Tensor> outputs, Body body) {
  MCCL_CHECK(!aborted_, "process group was aborted");
  ++op_seq_;
  auto work = c10::make_intrusive<WorkMCCL>(getRank(), op, title, std::move(outputs));
  ProgressTask t;
  t.name = title;
  t.bytes = bytes;
  t.metric_seq = Metrics::global().op_start(title, bytes);
  t.execute = std::move(body);
  t.on_complete = [work] { work->markDone(); };
  t.on_error = [work](std::exception_ptr e) { work->markFailed(e); };
  engine_->submit(std::move(t));
  return work;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::submitStream(
    c10d::OpType op, const char* title, uint64_t bytes, const std::string& algo, std::vector<at::Tensor> inputs,
    std::vector<at::Tensor> outputs, at::Device device,
    const std::function<void(DeviceComm&, void*)>& launch, int lane) {
  MCCL_CHECK(!aborted_, "process group was aborted");
  ++op_seq_;
  auto dev = deviceComm(device);
  if (dev->status() != 0) dev->check_status();
  c10::cuda::CUDAGuard guard(device);
  auto cur = c10::cuda::getCurrentCUDAStream(device.index());
  auto comm = comm_stream_for(this, device.index(), lane);
  uint64_t mseq = Metrics::global().op_start(title, bytes, algo);

  at::cuda::CUDAEvent ready;
  ready.record(cur);
  ready.block(comm);

  // Outside a graph capture the op is timed with an event pair and handed to the completion thread.
  const bool watched = !stream_capturing(cur);
  const bool timed = watched && device_metrics_;
  auto work = c10::make_intrusive<WorkMCCL>(getRank(), op, title, outputs);
  std::shared_ptr<EventCompletion> done;
  {
    c10::cuda::CUDAStreamGuard sg(comm);
    done = std::make_shared<EventCompletion>(dev, device.index(), op == c10d::OpType::BARRIER, timed);
    done->record_start(comm);
    launch(*dev, static_cast<void*>(comm.stream()));
    done->record(comm);
    work->attachStream(done, cfg_.blocking_wait);
  }
  for (auto& t : inputs)
    if (t.defined() && t.device().is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), comm);
  for (auto& t : outputs)
    if (t.defined() && t.device().is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), comm);
  if (watched) {
    Metrics::global().op_execute_start(mseq);
    watcher().watch({work, done, mseq});
  } else {
    Metrics::global().op_end(mseq, false);
  }
  return work;
}

// ---------------------------------------------------------------- allreduce --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce(std::vector<at::Tensor>& tensors,
                                                           const c10d::AllreduceOptions& opts) {
  // Per-call knobs, read on the caller thread like the reference does.
  return allreduceWith(tensors, to_redop(opts.reduceOp), requested_algo(), requested_wire());
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduceWith(std::vector<at::Tensor>& tensors, RedOp op, Algo req,
                                                               WireDtype wire) {
  MCCL_CHECK_TENSOR(!tensors.empty(), "allreduce: empty tensor list");
  for (auto& t : tensors) check_tensor(t, "allreduce");
  if (getSize() == 1) return WorkMCCL::completed(getRank(), c10d::OpType::ALLREDUCE, "mccl:allreduce", tensors);

  int64_t below = tensors[0].device().is_cuda() ? device_oneshot_below_bytes() : tree_below_bytes();
  uint64_t bytes = 0;
  for (auto& t : tensors) bytes += nbytes(t);

  if (tensors[0].device().is_cuda()) {
    std::vector<at::Tensor> ts = tensors;
    auto self = this;
    return submitStream(
        c10d::OpType::ALLREDUCE, "mccl:allreduce", bytes, algo_name(req), ts, ts, tensors[0].device(),
        [ts, op, req, wire, below, self](DeviceComm& dev, void* stream) {
          for (auto& t : ts) {
            if (t.numel() == 0) continue;
            Algo ran;
            if (device_reducible(t.scalar_type())) {
              ran = dev.allreduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()),
                                  to_dtype(t.scalar_type()), op, req, wire, below, stream);
            } else {
              // Narrow integer and bool types ride as int32.
              at::Tensor wide = t.to(at::kInt);
              ran = dev.allreduce(wide.data_ptr(), wide.data_ptr(), static_cast<size_t>(wide.numel()), DType::I32,
                                  op, req, WireDtype::NATIVE, below, stream);
              t.copy_(wide);
            }
            std::lock_guard<std::mutex> g(self->algo_mu_);
            self->last_algo_ = algo_name(ran);
          }
        });
  }

  std::vector<at::Tensor> ts = tensors;
  return submitHost(c10d::OpType::ALLREDUCE, "mccl:allreduce", bytes, ts, [this, ts, op, req, wire, below] {
    for (auto& t : ts) {
      if (t.numel() == 0) continue;
      AllreduceArgs a;
      a.data = t.data_ptr();
      a.numel = static_cast<size_t>(t.numel());
      a.dtype = to_dtype(t.scalar_type());
      a.op = op;
      a.wire = wire;
      Algo algo = resolve_cpu_algo(req, a.numel, nbytes(t), getSize(), below);
      {
        std::lock_guard<std::mutex> g(algo_mu_);
        last_algo_ = algo_name(algo);
      }
      mccl::allreduce(mesh(), a, algo);
    }
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                                     const c10d::AllreduceCoalescedOptions& opts) {
  c10d::AllreduceOptions o;
  o.reduceOp = opts.reduceOp;
  o.timeout = opts.timeout;
  return allreduce(tensors, o);
}

// ---------------------------------------------------------------- broadcast --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::broadcast(std::vector<at::Tensor>& tensors,
                                                           const c10d::BroadcastOptions& opts) {
  check_single(tensors, "broadcast");
  int root = static_cast<int>(opts.rootRank);
  MCCL_CHECK(root >= 0 && root < getSize(), "broadcast: bad root " << root);
  if (getSize() == 1) return WorkMCCL::completed(getRank(), c10d::OpType::BROADCAST, "mccl:broadcast", tensors);
  at::Tensor t = tensors[0];
  if (t.numel() == 0) return WorkMCCL::completed(getRank(), c10d::OpType::BROADCAST, "mccl:broadcast", tensors);
  if (t.device().is_cuda()) {
    return submitStream(c10d::OpType::BROADCAST, "mccl:broadcast", nbytes(t), "", {t}, {t}, t.device(),
                        [t, root](DeviceComm& dev, void* stream) { dev.broadcast(t.data_ptr(), nbytes(t), root, stream); });
  }
  return submitHost(c10d::OpType::BROADCAST, "mccl:broadcast", nbytes(t), {t},
                    [this, t, root] { mccl::broadcast(mesh(), t.data_ptr(), nbytes(t), root); });
}

// ------------------------------------------------------------------- reduce --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::reduce(std::vector<at::Tensor>& tensors,
                                                        const c10d::ReduceOptions& opts) {
  check_single(tensors, "reduce");
  int root = static_cast<int>(opts.rootRank);
  RedOp op = to_redop(opts.reduceOp);
  if (getSize() == 1) return WorkMCCL::completed(getRank(), c10d::OpType::REDUCE, "mccl:reduce", tensors);
  at::Tensor t = tensors[0];
  if (t.device().is_cuda()) {
    // Every rank joins a full allreduce; non-root ranks reduce into a scratch
    // copy so their tensor keeps its value.
    bool is_root = getRank() == root;
    Algo req = requested_algo();
    int64_t below = device_oneshot_below_bytes();
    return submitStream(c10d::OpType::REDUCE, "mccl:reduce", nbytes(t), "", {t}, {t}, t.device(),
                        [t, op, is_root, req, below](DeviceComm& dev, void* stream) {
                          at::Tensor src = device_reducible(t.scalar_type()) ? t : t.to(at::kInt);
                          at::Tensor dst = (is_root && src.is_same(t)) ? t : at::empty_like(src);
                          dev.allreduce(src.data_ptr(), dst.data_ptr(), static_cast<size_t>(src.numel()),
                                        to_dtype(src.scalar_type()), op, req, WireDtype::NATIVE, below, stream);
                          if (is_root && !dst.is_same(t)) t.copy_(dst);
                        });
  }
  return submitHost(c10d::OpType::REDUCE, "mccl:reduce", nbytes(t), {t}, [this, t, op, root] {
    if (getRank() == root) {
      mccl::reduce(mesh(), t.data_ptr(), static_cast<size_t>(t.numel()), to_dtype(t.scalar_type()), op, root);
    } else {
      at::Tensor scratch = t.clone();
      mccl::reduce(mesh(), scratch.data_ptr(), static_cast<size_t>(t.numel()), to_dtype(t.scalar_type()), op, root);
    }
  });
}

// ---------------------------------------------------------------- allgather --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::_allgather_base(at::Tensor& out, at::Tensor& in,
                                                                 const c10d::AllgatherOptions&) {
  check_tensor(in, "allgather_base(input)");
  check_tensor(out, "allgather_base(output)");
  check_same(in, out, "allgather_base");
  MCCL_CHECK_TENSOR(out.numel() == in.numel() * getSize(),
                    "allgather_base: output numel " << out.numel() << " != input numel " << in.numel() << " * world "
                                                    << getSize());
  if (getSize() == 1) {
    if (out.data_ptr() != in.data_ptr()) out.copy_(in.view_as(out));
    return WorkMCCL::completed(getRank(), c10d::OpType::_ALLGATHER_BASE, "mccl:allgather_base", {out});
  }
  at::Tensor o = out, i = in;
  if (i.numel() == 0) return WorkMCCL::completed(getRank(), c10d::OpType::_ALLGATHER_BASE, "mccl:allgather_base", {o});
  if (i.device().is_cuda()) {
    return submitStream(c10d::OpType::_ALLGATHER_BASE, "mccl:allgather_base", nbytes(o), "", {i}, {o}, i.device(),
                        [o, i](DeviceComm& dev, void* stream) { dev.allgather(i.data_ptr(), o.data_ptr(), nbytes(i), stream); });
  }
  return submitHost(c10d::OpType::_ALLGATHER_BASE, "mccl:allgather_base", nbytes(o), {o},
                    [this, o, i] { mccl::allgather(mesh(), i.data_ptr(), o.data_ptr(), nbytes(i)); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allgather(std::vector<std::vector<at::Tensor>>& outs,
                                                           std::vector<at::Tensor>& ins,
                                                           const c10d::AllgatherOptions&) {
  MCCL_CHECK_TENSOR(ins.size() == outs.size(), "allgather: " << ins.size() << " inputs but " << outs.size()
                                                             << " output lists");
  const int N = getSize();
  for (size_t k = 0; k < ins.size(); ++k) {
    check_tensor(ins[k], "allgather(input)");
    MCCL_CHECK_TENSOR(static_cast<int>(outs[k].size()) == N, "allgather: output list must have world entries");
    for (auto& o : outs[k]) {
      check_tensor(o, "allgather(output)");
      check_same(o, ins[k], "allgather");
      MCCL_CHECK_TENSOR(o.numel() == ins[k].numel(), "allgather: output numel differs from input numel");
    }
  }
  std::vector<at::Tensor> flat_out;
  for (auto& l : outs)
    for (auto& o : l) flat_out.push_back(o);
  if (N == 1) {
    for (size_t k = 0; k < ins.size(); ++k) outs[k][0].copy_(ins[k]);
    return WorkMCCL::completed(getRank(), c10d::OpType::ALLGATHER, "mccl:allgather", flat_out);
  }
  auto outs_c = outs;
  auto ins_c = ins;
  uint64_t bytes = 0;
  for (auto& t : flat_out) bytes += nbytes(t);
  if (ins[0].device().is_cuda()) {
    return submitStream(c10d::OpType::ALLGATHER, "mccl:allgather", bytes, "", ins_c, flat_out, ins[0].device(),
                        [outs_c, ins_c, N](DeviceComm& dev, void* stream) {
                          for (size_t k = 0; k < ins_c.size(); ++k) {
                            if (ins_c[k].numel() == 0) continue;
                            at::Tensor flat = at::empty({N * ins_c[k].numel()}, ins_c[k].options());
                            dev.allgather(ins_c[k].data_ptr(), flat.data_ptr(), nbytes(ins_c[k]), stream);
                            auto parts = flat.chunk(N);
                            for (int r = 0; r < N; ++r) outs_c[k][r].copy_(parts[r].view_as(outs_c[k][r]), true);
                          }
                        });
  }
  return submitHost(c10d::OpType::ALLGATHER, "mccl:allgather", bytes, flat_out, [this, outs_c, ins_c, N] {
    for (size_t k = 0; k < ins_c.size(); ++k) {
      size_t nb = nbytes(ins_c[k]);
      if (nb == 0) continue;
      std::vector<IoSpan> sends, recvs;
      for (int p = 0; p < N; ++p) {
        if (p == getRank()) continue;
        sends.push_back({p, ins_c[k].data_ptr(), nb});
        recvs.push_back({p, outs_c[k][p].data_ptr(), nb});
      }
      mesh().exchange(sends, recvs);
      if (outs_c[k][getRank()].data_ptr() != ins_c[k].data_ptr()) outs_c[k][getRank()].copy_(ins_c[k]);
    }
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allgather_coalesced(std::vector<std::vector<at::Tensor>>& outLists,
                                                                     std::vector<at::Tensor>& ins,
                                                                     const c10d::AllgatherOptions& opts) {
  // outLists[r][k] receives rank r's k-th input: transpose into per-input lists.
  const int N = getSize();
  MCCL_CHECK_TENSOR(static_cast<int>(outLists.size()) == N, "allgather_coalesced: need one output list per rank");
  std::vector<std::vector<at::Tensor>> per_input(ins.size());
  for (size_t k = 0; k < ins.size(); ++k)
    for (int r = 0; r < N; ++r) {
      MCCL_CHECK_TENSOR(outLists[r].size() == ins.size(), "allgather_coalesced: ragged output lists");
      per_input[k].push_back(outLists[r][k]);
    }
  return allgather(per_input, ins, opts);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                                                 std::vector<at::Tensor>& inputs,
                                                                                 const c10d::AllgatherOptions& opts) {
  MCCL_CHECK_TENSOR(outputs.size() == inputs.size() && !inputs.empty(), "allgather_into_tensor_coalesced: list sizes differ");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t k = 0; k < inputs.size(); ++k) last = _allgather_base(outputs[k], inputs[k], opts);
  return last;  // stream / FIFO order makes the last work cover the earlier ones
}

// ----------------------------------------------------------- reduce_scatter --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::_reduce_scatter_base(at::Tensor& out, at::Tensor& in,
                                                                      const c10d::ReduceScatterOptions& opts) {
  check_tensor(in, "reduce_scatter_base(input)");
  check_tensor(out, "reduce_scatter_base(output)");
  check_same(in, out, "reduce_scatter_base");
  MCCL_CHECK_TENSOR(in.numel() == out.numel() * getSize(),
                    "reduce_scatter_base: input numel " << in.numel() << " != output numel " << out.numel()
                                                        << " * world " << getSize());
  RedOp op = to_redop(opts.reduceOp);
  if (getSize() == 1) {
    if (out.data_ptr() != in.data_ptr()) out.copy_(in.view_as(out));
    return WorkMCCL::completed(getRank(), c10d::OpType::_REDUCE_SCATTER_BASE, "mccl:reduce_scatter_base", {out});
  }
  at::Tensor o = out, i = in;
  if (o.numel() == 0)
    return WorkMCCL::completed(getRank(), c10d::OpType::_REDUCE_SCATTER_BASE, "mccl:reduce_scatter_base", {o});
  WireDtype wire = requested_wire();
  if (i.device().is_cuda()) {
    return submitStream(c10d::OpType::_REDUCE_SCATTER_BASE, "mccl:reduce_scatter_base", nbytes(i), "", {i}, {o},
                        i.device(), [o, i, op, wire](DeviceComm& dev, void* stream) {
                          if (device_reducible(i.scalar_type())) {
                            dev.reduce_scatter(i.data_ptr(), o.data_ptr(), static_cast<size_t>(o.numel()),
                                               to_dtype(i.scalar_type()), op, wire, stream);
                          } else {
                            at::Tensor wi = i.to(at::kInt), wo = at::empty(o.sizes(), wi.options());
                            dev.reduce_scatter(wi.data_ptr(), wo.data_ptr(), static_cast<size_t>(o.numel()), DType::I32,
                                               op, WireDtype::NATIVE, stream);
                            o.copy_(wo);
                          }
                        });
  }
  return submitHost(c10d::OpType::_REDUCE_SCATTER_BASE, "mccl:reduce_scatter_base", nbytes(i), {o}, [this, o, i, op] {
    mccl::reduce_scatter(mesh(), i.data_ptr(), o.data_ptr(), static_cast<size_t>(o.numel()),
                         to_dtype(i.scalar_type()), op);
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::reduce_scatter(std::vector<at::Tensor>& outs,
                                                                std::vector<std::vector<at::Tensor>>& ins,
                                                                const c10d::ReduceScatterOptions& opts) {
  check_single(outs, "reduce_scatter(output)");
  MCCL_CHECK_TENSOR(ins.size() == 1 && static_cast<int>(ins[0].size()) == getSize(),
                    "reduce_scatter: need one input list with world entries");
  for (auto& t : ins[0]) {
    check_tensor(t, "reduce_scatter(input)");
    check_same(t, outs[0], "reduce_scatter");
    MCCL_CHECK_TENSOR(t.numel() == outs[0].numel(), "reduce_scatter: input numel differs from output numel");
  }
  if (getSize() == 1) {
    outs[0].copy_(ins[0][0]);
    return WorkMCCL::completed(getRank(), c10d::OpType::REDUCE_SCATTER, "mccl:reduce_scatter", outs);
  }
  // Pack the per-rank inputs into one buffer and reuse the flat path.
  at::Tensor packed = at::empty({getSize() * outs[0].numel()}, outs[0].options());
  auto parts = packed.chunk(getSize());
  for (int r = 0; r < getSize(); ++r) parts[r].copy_(ins[0][r].reshape({-1}));
  at::Tensor o = outs[0];
  at::Tensor oflat = o.view({-1});
  return _reduce_scatter_base(oflat, packed, opts);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::reduce_scatter_tensor_coalesced(
    std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::ReduceScatterOptions& opts) {
  MCCL_CHECK_TENSOR(outputs.size() == inputs.size() && !inputs.empty(), "reduce_scatter_tensor_coalesced: list sizes differ");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t k = 0; k < inputs.size(); ++k) last = _reduce_scatter_base(outputs[k], inputs[k], opts);
  return last;
}

// ----------------------------------------------------------------- alltoall --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::alltoall_base(at::Tensor& out, at::Tensor& in,
                                                               std::vector<int64_t>& outSplits,
                                                               std::vector<int64_t>& inSplits,
                                                               const c10d::AllToAllOptions&) {
  check_tensor(in, "alltoall_base(input)");
  check_tensor(out, "alltoall_base(output)");
  check_same(in, out, "alltoall_base");
  const int N = getSize();
  // Split sizes count rows of dim 0; a row is numel/size(0) elements.  (The
  // reference multiplies by the element size only, ProcessGroupMCCL.cpp:508-520,
  // which is right for 1-D tensors only.)
  auto layout = [N](const at::Tensor& t, const std::vector<int64_t>& splits, std::vector<size_t>& off,
                    std::vector<size_t>& len, const char* what) {
    off.assign(N, 0);
    len.assign(N, 0);
    size_t row = t.dim() > 0 && t.size(0) > 0 ? static_cast<size_t>(t.numel() / t.size(0)) * t.element_size()
                                              : t.element_size();
    if (splits.empty()) {
      MCCL_CHECK_TENSOR(t.dim() > 0 && t.size(0) % N == 0, what << ": dim 0 (" << (t.dim() ? t.size(0) : 0)
                                                                 << ") is not divisible by world " << N);
      size_t each = static_cast<size_t>(t.size(0) / N) * row;
      for (int p = 0; p < N; ++p) {
        off[p] = p * each;
        len[p] = each;
      }
    } else {
      MCCL_CHECK_TENSOR(static_cast<int>(splits.size()) == N, what << ": need world split sizes");
      size_t acc = 0;
      int64_t rows = 0;
      for (int p = 0; p < N; ++p) {
        MCCL_CHECK_TENSOR(splits[p] >= 0, what << ": negative split");
        off[p] = acc;
        len[p] = static_cast<size_t>(splits[p]) * row;
        acc += len[p];
        rows += splits[p];
      }
      MCCL_CHECK_TENSOR(rows == (t.dim() ? t.size(0) : 1), what << ": splits sum to " << rows << " but dim 0 is "
                                                                 << (t.dim() ? t.size(0) : 1));
    }
  };
  std::vector<size_t> ioff, ilen, ooff, olen;
  layout(in, inSplits, ioff, ilen, "alltoall_base(input)");
  layout(out, outSplits, ooff, olen, "alltoall_base(output)");
  if (N == 1) {
    out.copy_(in.view_as(out));
    return WorkMCCL::completed(getRank(), c10d::OpType::ALLTOALL_BASE, "mccl:alltoall_base", {out});
  }
  at::Tensor o = out, i = in;
  if (i.device().is_cuda()) {
    return submitStream(c10d::OpType::ALLTOALL_BASE, "mccl:alltoall_base", nbytes(i), "", {i}, {o}, i.device(),
                        [o, i, ioff, ilen, ooff, olen](DeviceComm& dev, void* stream) {
                          dev.alltoallv(i.data_ptr(), ioff, ilen, o.data_ptr(), ooff, olen, stream);
                        });
  }
  return submitHost(c10d::OpType::ALLTOALL_BASE, "mccl:alltoall_base", nbytes(i), {o},
                    [this, o, i, ioff, ilen, ooff, olen] {
                      mccl::alltoallv(mesh(), i.data_ptr(), ioff, ilen, o.data_ptr(), ooff, olen);
                    });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins,
                                                          const c10d::AllToAllOptions&) {
  const int N = getSize();
  MCCL_CHECK_TENSOR(static_cast<int>(ins.size()) == N && static_cast<int>(outs.size()) == N,
                    "alltoall: need world input and output tensors");
  for (int p = 0; p < N; ++p) {
    check_tensor(ins[p], "alltoall(input)");
    check_tensor(outs[p], "alltoall(output)");
    check_same(ins[p], outs[p], "alltoall");
  }
  if (N == 1) {
    outs[0].copy_(ins[0]);
    return WorkMCCL::completed(getRank(), c10d::OpType::ALLTOALL, "mccl:alltoall", outs);
  }
  auto outs_c = outs, ins_c = ins;
  uint64_t bytes = 0;
  for (auto& t : ins) bytes += nbytes(t);
  if (ins[0].device().is_cuda()) {
    return submitStream(c10d::OpType::ALLTOALL, "mccl:alltoall", bytes, "", ins_c, outs_c, ins[0].device(),
                        [outs_c, ins_c, N](DeviceComm& dev, void* stream) {
                          // Pack, exchange with per-peer byte counts, unpack.
                          std::vector<size_t> ioff(N), ilen(N), ooff(N), olen(N);
                          size_t ib = 0, ob = 0;
                          for (int p = 0; p < N; ++p) {
                            ioff[p] = ib; ilen[p] = nbytes(ins_c[p]); ib += (ilen[p] + 15) / 16 * 16;
                            ooff[p] = ob; olen[p] = nbytes(outs_c[p]); ob += (olen[p] + 15) / 16 * 16;
                          }
                          auto bopt = ins_c[0].options().dtype(at::kByte);
                          at::Tensor pin = at::empty({static_cast<int64_t>(std::max<size_t>(ib, 16))}, bopt);
                          at::Tensor pout = at::empty({static_cast<int64_t>(std::max<size_t>(ob, 16))}, bopt);
                          for (int p = 0; p < N; ++p)
                            if (ilen[p])
                              cudaMemcpyAsync(static_cast<char*>(pin.data_ptr()) + ioff[p], ins_c[p].data_ptr(), ilen[p],
                                              cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
                          dev.alltoallv(pin.data_ptr(), ioff, ilen, pout.data_ptr(), ooff, olen, stream);
                          for (int p = 0; p < N; ++p)
                            if (olen[p])
                              cudaMemcpyAsync(outs_c[p].data_ptr(), static_cast<char*>(pout.data_ptr()) + ooff[p], olen[p],
                                              cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
                        });
  }
  return submitHost(c10d::OpType::ALLTOALL, "mccl:alltoall", bytes, outs_c, [this, outs_c, ins_c, N] {
    std::vector<IoSpan> sends, recvs;
    for (int p = 0; p < N; ++p) {
      if (p == getRank()) {
        outs_c[p].copy_(ins_c[p].view_as(outs_c[p]));
        continue;
      }
      if (nbytes(ins_c[p])) sends.push_back({p, ins_c[p].data_ptr(), nbytes(ins_c[p])});
      if (nbytes(outs_c[p])) recvs.push_back({p, outs_c[p].data_ptr(), nbytes(outs_c[p])});
    }
    mesh().exchange(sends, recvs);
  });
}

// ---------------------------------------------------------- gather / scatter --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::gather(std::vector<std::vector<at::Tensor>>& outs,
                                                        std::vector<at::Tensor>& ins, const c10d::GatherOptions& opts) {
  check_single(ins, "gather(input)");
  const int N = getSize(), root = static_cast<int>(opts.rootRank);
  const bool is_root = getRank() == root;
  if (is_root) {
    MCCL_CHECK_TENSOR(outs.size() == 1 && static_cast<int>(outs[0].size()) == N,
                      "gather: root needs one output list with world entries");
    for (auto& o : outs[0]) {
      check_tensor(o, "gather(output)");
      MCCL_CHECK_TENSOR(o.numel() == ins[0].numel(), "gather: output numel differs from input numel");
    }
  }
  at::Tensor in = ins[0];
  std::vector<at::Tensor> o = is_root ? outs[0] : std::vector<at::Tensor>{};
  if (N == 1) {
    o[0].copy_(in);
    return WorkMCCL::completed(getRank(), c10d::OpType::GATHER, "mccl:gather", o);
  }
  if (in.device().is_cuda()) {
    return submitStream(c10d::OpType::GATHER, "mccl:gather", nbytes(in) * N, "", {in}, o, in.device(),
                        [in, o, N, is_root](DeviceComm& dev, void* stream) {
                          at::Tensor flat = at::empty({N * in.numel()}, in.options());
                          dev.allgather(in.data_ptr(), flat.data_ptr(), nbytes(in), stream);
                          if (is_root) {
                            auto parts = flat.chunk(N);
                            for (int r = 0; r < N; ++r) o[r].copy_(parts[r].view_as(o[r]), true);
                          }
                        });
  }
  return submitHost(c10d::OpType::GATHER, "mccl:gather", nbytes(in) * N, o, [this, in, o, N, root, is_root] {
    if (is_root) {
      at::Tensor flat = at::empty({N * in.numel()}, in.options());
      mccl::gather(mesh(), in.data_ptr(), flat.data_ptr(), nbytes(in), root);
      auto parts = flat.chunk(N);
      for (int r = 0; r < N; ++r) o[r].copy_(parts[r].view_as(o[r]));
    } else {
      mccl::gather(mesh(), in.data_ptr(), nullptr, nbytes(in), root);
    }
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::scatter(std::vector<at::Tensor>& outs,
                                                         std::vector<std::vector<at::Tensor>>& ins,
                                                         const c10d::ScatterOptions& opts) {
  check_single(outs, "scatter(output)");
  const int N = getSize(), root = static_cast<int>(opts.rootRank);
  const bool is_root = getRank() == root;
  if (is_root) {
    MCCL_CHECK_TENSOR(ins.size() == 1 && static_cast<int>(ins[0].size()) == N,
                      "scatter: root needs one input list with world entries");
    for (auto& t : ins[0]) {
      check_tensor(t, "scatter(input)");
      MCCL_CHECK_TENSOR(t.numel() == outs[0].numel(), "scatter: input numel differs from output numel");
    }
  }
  at::Tensor out = outs[0];
  std::vector<at::Tensor> i = is_root ? ins[0] : std::vector<at::Tensor>{};
  if (N == 1) {
    out.copy_(i[0]);
    return WorkMCCL::completed(getRank(), c10d::OpType::SCATTER, "mccl:scatter", {out});
  }
  if (out.device().is_cuda()) {
    int rank = getRank();
    return submitStream(c10d::OpType::SCATTER, "mccl:scatter", nbytes(out) * N, "", i, {out}, out.device(),
                        [out, i, N, is_root, rank, root](DeviceComm& dev, void* stream) {
                          // Root sends slice p to rank p; everyone else sends nothing.
                          size_t nb = nbytes(out);
                          std::vector<size_t> ioff(N, 0), ilen(N, 0), ooff(N, 0), olen(N, 0);
                          at::Tensor packed = at::empty({is_root ? N * out.numel() : 1}, out.options());
                          if (is_root) {
                            auto parts = packed.chunk(N);
                            for (int p = 0; p < N; ++p) {
                              parts[p].copy_(i[p].reshape({-1}), true);
                              ioff[p] = p * nb;
                              ilen[p] = nb;
                            }
                          }
                          olen[root] = nb;
                          (void)rank;
                          dev.alltoallv(packed.data_ptr(), ioff, ilen, out.data_ptr(), ooff, olen, stream);
                        });
  }
  return submitHost(c10d::OpType::SCATTER, "mccl:scatter", nbytes(out) * N, {out}, [this, out, i, N, root, is_root] {
    if (is_root) {
      at::Tensor packed = at::empty({N * out.numel()}, out.options());
      auto parts = packed.chunk(N);
      for (int p = 0; p < N; ++p) parts[p].copy_(i[p].reshape({-1}));
      mccl::scatter(mesh(), packed.data_ptr(), out.data_ptr(), nbytes(out), root);
    } else {
      mccl::scatter(mesh(), nullptr, out.data_ptr(), nbytes(out), root);
    }
  });
}

// ---------------------------------------------------------------- send/recv --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::send(std::vector<at::Tensor>& tensors, int dst, int tag) {
  check_single(tensors, "send");
  MCCL_CHECK(dst >= 0 && dst < getSize() && dst != getRank(), "send: bad destination rank " << dst);
  at::Tensor t = tensors[0];
  if (t.device().is_cuda()) {
    if (use_nccl_p2p_) return p2p()->send(tensors, dst, tag);
    if (t.numel() == 0) return WorkMCCL::completed(getRank(), c10d::OpType::SEND, "mccl:send", {});
    return submitStream(c10d::OpType::SEND, "mccl:send", nbytes(t), "", {t}, {}, t.device(),
                        [t, dst](DeviceComm& dev, void* stream) { dev.send(t.data_ptr(), nbytes(t), dst, stream); }, 1);
  }
  return submitHost(c10d::OpType::SEND, "mccl:send", nbytes(t), {},
                    [this, t, dst, tag] { send_tagged(mesh(), dst, t.data_ptr(), nbytes(t), tag); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::recv(std::vector<at::Tensor>& tensors, int src, int tag) {
  check_single(tensors, "recv");
  MCCL_CHECK(src >= 0 && src < getSize() && src != getRank(), "recv: bad source rank " << src);
  at::Tensor t = tensors[0];
  if (t.device().is_cuda()) {
    if (use_nccl_p2p_) return p2p()->recv(tensors, src, tag);
    if (t.numel() == 0) return WorkMCCL::completed(getRank(), c10d::OpType::RECV, "mccl:recv", {t});
    return submitStream(c10d::OpType::RECV, "mccl:recv", nbytes(t), "", {}, {t}, t.device(),
                        [t, src](DeviceComm& dev, void* stream) { dev.recv(t.data_ptr(), nbytes(t), src, stream); }, 2);
  }
  return submitHost(c10d::OpType::RECV, "mccl:recv", nbytes(t), {t},
                    [this, t, src, tag] { recv_tagged(mesh(), src, t.data_ptr(), nbytes(t), tag); });
}

// ------------------------------------------------------------------ barrier --
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::barrier(const c10d::BarrierOptions& opts) {
  if (getSize() == 1) return WorkMCCL::completed(getRank(), c10d::OpType::BARRIER, "mccl:barrier", {});
  // The ranks always meet over the TCP mesh first and tell one another, in the token they exchange,
  // whether they hold a device communicator (or were told which GPU to use).  Only when every rank
  // does, the barrier kernel follows on the comm stream, so the path is chosen from group-wide state
  // and two ranks can never wait for each other on different planes.
  std::shared_ptr<DeviceComm> dev;
  {
    std::lock_guard<std::mutex> g(dev_mu_);
    dev = dev_;
  }
  c10::optional<at::Device> device;
  if (dev) device = at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(dev->device()));
  else if (opts.device.has_value() && opts.device->is_cuda()) device = opts.device;
  else if (!opts.device_ids.empty()) device = at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(opts.device_ids[0]));
  barrier_seq_++;
  const uint8_t mine = device.has_value() ? 2 : 1;
  auto tokens = std::make_shared<std::vector<uint8_t>>(static_cast<size_t>(getSize()), 0);
  auto host = submitHost(c10d::OpType::BARRIER, "mccl:barrier", 0, {}, [this, tokens, mine] {
    uint8_t token = mine;
    mccl::allgather(mesh(), &token, tokens->data(), 1);
  });
  if (!device.has_value()) return host;   // at least this rank has no GPU side: the host meeting is the barrier
  host->wait();
  bool all_device = true;
  for (uint8_t t : *tokens) all_device = all_device && t == 2;
  if (!all_device) {
    // Some rank has no device side: keep the promise that this rank's GPU work is finished.
    c10::cuda::CUDAGuard guard(*device);
    cudaStreamSynchronize(c10::cuda::getCurrentCUDAStream(device->index()).stream());
    return host;
  }
  return submitStream(c10d::OpType::BARRIER, "mccl:barrier", 0, "", {}, {}, *device,
                      [](DeviceComm& d, void* stream) { d.barrier(stream); });
}

}  // namespace mccl
