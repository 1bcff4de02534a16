#include "device_comm.hpp"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstring>
#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

#include "../core/errors.hpp"
#include "../core/log.hpp"
#include "../core/timeline.hpp"
#include "../kernels/collectives.hpp"
#include "../kernels/comm_device.cuh"
#include "../symm/cu_driver.hpp"
#include "../symm/symm_mesh.hpp"

namespace mccl {

namespace {

dev::ElemType to_elem(DType t) {
  switch (t) {
    case DType::F32: return dev::ElemType::F32;
    case DType::F16: return dev::ElemType::F16;
    case DType::BF16: return dev::ElemType::BF16;
    case DType::F64: return dev::ElemType::F64;
    case DType::I32: return dev::ElemType::I32;
    case DType::I64: return dev::ElemType::I64;
    default: MCCL_CHECK_T(false, TensorError, "device collectives do not reduce dtype " << dtype_name(t));
  }
  return dev::ElemType::F32;
}

int to_dev_op(RedOp op, DType t) {
  switch (op) {
    case RedOp::SUM: return dev::OP_SUM;
    case RedOp::AVG: return dev::OP_AVG;
    case RedOp::MIN: return dev::OP_MIN;
    case RedOp::MAX: return dev::OP_MAX;
    case RedOp::PRODUCT: return dev::OP_PROD;
    case RedOp::BAND: case RedOp::BOR: case RedOp::BXOR:
      MCCL_CHECK_T(!dtype_is_float(t), TensorError, "bitwise reduce ops need an integer dtype");
      return op == RedOp::BAND ? dev::OP_BAND : op == RedOp::BOR ? dev::OP_BOR : dev::OP_BXOR;
    default: break;
  }
  MCCL_CHECK(false, "unsupported reduce op");
  return 0;
}

constexpr size_t kCanaryBytes = 512;

// "rank=1,skip_signals=1,after=2,delay_ms=50": comma-separated key=value pairs, unknown keys are an error.
void parse_fault_spec(const std::string& spec, int* rank, int* skip, long long* after, int* delay_ms) {
  size_t b = 0;
  while (b < spec.size()) {
    size_t e = spec.find(',', b);
    if (e == std::string::npos) e = spec.size();
    const std::string kv = spec.substr(b, e - b);
    b = e + 1;
    if (kv.empty()) continue;
    const size_t eq = kv.find('=');
    MCCL_CHECK(eq != std::string::npos, "MCCL_FAULT_INJECT: expected key=value, got '" << kv << "'");
    const std::string k = kv.substr(0, eq);
    const long long v = std::atoll(kv.c_str() + eq + 1);
    if (k == "rank") *rank = static_cast<int>(v);
    else if (k == "skip_signals") *skip = static_cast<int>(v);
    else if (k == "after") *after = v;
    else if (k == "delay_ms") *delay_ms = static_cast<int>(v);
    else MCCL_CHECK(false, "MCCL_FAULT_INJECT: unknown key '" << k << "' (rank, skip_signals, after, delay_ms)");
  }
}

const char* phase_name(int ph) {
  switch (ph) {
    case dev::PH_SEND: return "send";
    case dev::PH_RECV: return "recv";
    case dev::PH_BOUNDS: return "bounds";
    case dev::PH_BARRIER: return "barrier";
    case dev::PH_PUSH: return "push";
    case dev::PH_REDUCE: return "reduce";
    case dev::PH_GATHER: return "gather";
    case dev::PH_RING: return "ring step";
    case dev::PH_TREE: return "tree step";
    case dev::PH_NVLS: return "nvls";
    default: return "?";
  }
}

}  // namespace

struct DeviceComm::Impl {
  std::shared_ptr<SymmAlloc> arena;  // two halves, multicast-bound when possible
  std::shared_ptr<SymmAlloc> pads;   // kChannels signal pads
  std::shared_ptr<SymmAlloc> p2p;    // inbound send/recv slots: [source][2][p2p_slot]
  size_t p2p_slot = 0;
  dev::P2PState* p2p_state = nullptr;  // device: [nlocal]
  dev::RankState* state = nullptr;   // device: [nlocal][kChannels]
  int* status_host = nullptr;        // pinned, mapped: [kMaxRanks]
  int* status_dev = nullptr;
  size_t half_bytes = 0;
  unsigned long long timeout_ns = 0;
  int max_ctas = 64;
  bool debug_bounds = false;  // MCCL_DEBUG_BOUNDS: kernels check their arena extent, canaries behind the arena
  unsigned long long debug_limit = 0;  // tests: pretend the arena ends here, so that the device-side check trips
  int threads = 0;         // threads per collective CTA, 0 = kernel default
  // No shape was asked for (neither MCCL_MAX_CTAS / MCCL_COMM_THREADS nor set_launch_shape): messages of
  // kLargeWireBytes or more then take every CTA the protocol has, 512 threads each.  Measured on two GPUs, fp32
  // two-shot at 64 / 256 MiB: 64 x 256 threads 297 / 299 GB/s, 128 x 256: 395 / 419, 128 x 512: 466 / 516 (NCCL 446 / 507).
  bool shape_auto = true;
  void large_shape(size_t wire_bytes, int nlocal, dev::LaunchCfg& cfg) const {
    if (shape_auto && nlocal == 1 && wire_bytes >= kLargeWireBytes) {
      cfg.ctas = dev::kMaxCtas;
      cfg.threads = dev::kThreads;
    }
  }
  static constexpr size_t kLargeWireBytes = 32u << 20;
  int64_t nvls_above = 0;  // AUTO uses staged NVLS at or above this many wire bytes (0 = never)
  int64_t push_above = 0;  // AUTO uses the fully pushed two-shot at or above this many wire bytes (0 = never)
  bool ag_multicast = true;  // allgather stores through the multicast mapping when there is one (MCCL_AG_NVLS=0: plain pushes)
  // Launch ordering across streams: the arena halves, flags and epochs are shared by every launch of this
  // communicator, so two collectives must never overlap on the device.  Each launch records `last_done` on its
  // stream; a launch on another stream first waits for it.  (Skipped while a stream is being captured: a graph
  // orders its own nodes and must not depend on events outside the capture.)
  cudaEvent_t last_done = nullptr;
  cudaStream_t last_stream = nullptr;
  bool have_last = false;
  std::mutex order_mu;

  static bool capturing(cudaStream_t s) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
      (void)cudaGetLastError();
      return false;
    }
    return st != cudaStreamCaptureStatusNone;
  }
  void order_before(cudaStream_t s) {
    std::lock_guard<std::mutex> g(order_mu);
    if (!have_last || s == last_stream || capturing(s)) return;
    cudaStreamWaitEvent(s, last_done, 0);
  }
  void order_after(cudaStream_t s) {
    std::lock_guard<std::mutex> g(order_mu);
    if (capturing(s)) return;
    if (!last_done) cudaEventCreateWithFlags(&last_done, cudaEventDisableTiming);
    cudaEventRecord(last_done, s);
    last_stream = s;
    have_last = true;
  }
  // Host-made faults (MCCL_FAULT_INJECT, see parse_fault_spec): applied on the rank they name, at the
  // collective they name, from the host side of the launch.  Nothing here makes a GPU fault or hang: a
  // skipped signal makes the peers' bounded waits run out, a delay makes a rank late.
  struct FaultSpec {
    int rank = -1;            // rank the fault applies to (-1: no fault configured)
    int skip_signals = 0;     // withhold the signals of this many collectives ...
    long long after = 0;      // ... starting with collective number `after` (0-based) of this communicator
    int delay_ms = 0;         // sleep this long on the host before every launch from `after` on
    bool armed = false;
  } fault;
  long long collectives = 0;
  DeviceComm* owner = nullptr;
  void apply_fault(cudaStream_t s) {
    const long long n = collectives++;
    if (fault.rank < 0 || owner == nullptr || owner->rank() != fault.rank || n < fault.after || capturing(s)) return;
    if (fault.delay_ms > 0) std::this_thread::sleep_for(std::chrono::milliseconds(fault.delay_ms));
    if (fault.skip_signals > 0 && !fault.armed) {
      fault.armed = true;
      owner->inject_skip_signals(fault.skip_signals);
    }
  }
  struct Ordered {   // scope of one public collective call
    Impl* impl;
    cudaStream_t s;
    Ordered(Impl* i, void* stream) : impl(i), s(static_cast<cudaStream_t>(stream)) {
      impl->apply_fault(s);
      impl->order_before(s);
    }
    ~Ordered() { impl->order_after(s); }
  };

  dev::DevComm ctx(int world, int rank_base, int nlocal, int channel) const {
    dev::DevComm c{};
    c.world = world;
    c.rank_base = rank_base;
    for (int r = 0; r < world; ++r) {
      c.arena[r] = static_cast<char*>(arena->ptrs[r]);
      c.flags[r] = static_cast<uint32_t*>(pads->ptrs[r]) + static_cast<size_t>(channel) * dev::kFlagWordsPerChannel;
    }
    c.mc_arena = static_cast<char*>(arena->mc_ptr);
    for (int v = 0; v < nlocal; ++v) {
      c.state[v] = state + static_cast<size_t>(v) * dev::kChannels + channel;
      c.status[v] = status_dev + v;
    }
    c.half_bytes = half_bytes;
    c.timeout_ns = timeout_ns;
    c.tl = timeline_device_ptr();
    c.arena_limit = debug_bounds ? (debug_limit ? debug_limit : 2ull * half_bytes) : 0ull;
    return c;
  }
};

DeviceComm::DeviceComm(KVStore* store, int rank, int world, int device, const std::string& prefix, const EnvConfig& cfg,
                       int64_t timeout_ms)
    : rank_(rank), world_(world), device_(device), nlocal_(1), cfg_(cfg), group_timeout_ms_(timeout_ms) {
  mesh_.reset(new SymmMesh(store, rank, world, device, prefix, cfg, timeout_ms));
  init_common();
}

DeviceComm::DeviceComm(int world, int device, const EnvConfig& cfg)
    : rank_(0), world_(world), device_(device), nlocal_(world), cfg_(cfg) {
  mesh_.reset(new SymmMesh(world, device));
  init_common();
}

void DeviceComm::init_common() {
  impl_.reset(new Impl());
  impl_->owner = this;
  if (!cfg_.fault_inject.empty())
    parse_fault_spec(cfg_.fault_inject, &impl_->fault.rank, &impl_->fault.skip_signals, &impl_->fault.after, &impl_->fault.delay_ms);
  MCCL_CUDA_CHECK(cudaSetDevice(device_));
  size_t arena = static_cast<size_t>(std::max<int64_t>(cfg_.arena_bytes, 2 << 20));
  impl_->arena = mesh_->alloc(arena, /*want_multicast=*/true);
  impl_->debug_bounds = cfg_.debug_bounds;
  impl_->half_bytes = (impl_->arena->bytes / 2) / 256 * 256;
  if (impl_->debug_bounds) {
    // Debug layout: both halves are poisoned (0xFF bytes read as NaN in every float type, so a kernel that
    // consumes staging nobody wrote shows up in the results) and the last kCanaryBytes of the allocation hold
    // a pattern that check_status() verifies: a write past the second half lands there first.
    impl_->half_bytes = ((impl_->arena->bytes - kCanaryBytes) / 2) / 256 * 256;
    MCCL_CUDA_CHECK(cudaMemset(impl_->arena->ptrs[rank_], 0xFF, 2 * impl_->half_bytes));
    MCCL_CUDA_CHECK(cudaMemset(static_cast<char*>(impl_->arena->ptrs[rank_]) + 2 * impl_->half_bytes, 0xA5, kCanaryBytes));
    if (nlocal_ > 1)
      for (int v = 1; v < nlocal_; ++v) {
        MCCL_CUDA_CHECK(cudaMemset(impl_->arena->ptrs[v], 0xFF, 2 * impl_->half_bytes));
        MCCL_CUDA_CHECK(cudaMemset(static_cast<char*>(impl_->arena->ptrs[v]) + 2 * impl_->half_bytes, 0xA5, kCanaryBytes));
      }
  }
  impl_->pads = mesh_->alloc(static_cast<size_t>(dev::kChannels) * dev::kFlagWordsPerChannel * sizeof(uint32_t), false);
  impl_->p2p_slot = static_cast<size_t>(std::max<int64_t>(env::i64("MCCL_P2P_SLOT_MB", 4), 1)) << 20;
  if (nlocal_ > 1) impl_->p2p_slot = std::min<size_t>(impl_->p2p_slot, 1u << 20);
  impl_->p2p = mesh_->alloc(impl_->p2p_slot * 2 * static_cast<size_t>(world_), /*want_multicast=*/false);
  MCCL_CUDA_CHECK(cudaMalloc(&impl_->p2p_state, sizeof(dev::P2PState) * nlocal_));
  MCCL_CUDA_CHECK(cudaMemset(impl_->p2p_state, 0, sizeof(dev::P2PState) * nlocal_));
  MCCL_CUDA_CHECK(cudaMalloc(&impl_->state, sizeof(dev::RankState) * dev::kChannels * nlocal_));
  MCCL_CUDA_CHECK(cudaMemset(impl_->state, 0, sizeof(dev::RankState) * dev::kChannels * nlocal_));
  MCCL_CUDA_CHECK(cudaHostAlloc(&impl_->status_host, sizeof(int) * dev::kMaxRanks, cudaHostAllocMapped));
  std::memset(impl_->status_host, 0, sizeof(int) * dev::kMaxRanks);
  MCCL_CUDA_CHECK(cudaHostGetDevicePointer(&impl_->status_dev, impl_->status_host, 0));
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  {
    // explicit MCCL_DEVICE_TIMEOUT_MS wins; otherwise the group's own timeout, capped; 10 s without a group
    int64_t ms = cfg_.device_timeout_ms;
    if (ms <= 0) ms = group_timeout_ms_ > 0 ? std::min<int64_t>(group_timeout_ms_, std::max<int64_t>(cfg_.device_timeout_cap_ms, 1000)) : 10000;
    impl_->timeout_ns = static_cast<unsigned long long>(std::max<int64_t>(ms, 1)) * 1000000ull;
  }
  int cap = cfg_.max_ctas > 0 ? cfg_.max_ctas : 64;   // 64 CTAs of 256 threads
  impl_->max_ctas = std::min(cap, dev::kMaxCtas);
  impl_->shape_auto = cfg_.max_ctas <= 0 && impl_->threads == 0;
  impl_->nvls_above = env::i64("MCCL_NVLS_ABOVE", 0);
  impl_->push_above = env::i64("MCCL_PUSH_ABOVE", 0);
  impl_->ag_multicast = env::flag("MCCL_AG_NVLS", true);
  if (nlocal_ > 1) impl_->max_ctas = std::max(1, std::min(impl_->max_ctas, 96 / nlocal_));  // all virtual ranks co-resident
  if (mesh_->mode() != SymmMesh::Mode::LOCAL) mesh_->store_barrier("devcomm-ready");
}

DeviceComm::~DeviceComm() {
  if (impl_) {
    if (impl_->last_done) cudaEventDestroy(impl_->last_done);
    if (impl_->state) cudaFree(impl_->state);
    if (impl_->p2p_state) cudaFree(impl_->p2p_state);
    if (impl_->status_host) cudaFreeHost(impl_->status_host);
  }
}

bool DeviceComm::nvls_available() const { return impl_->arena->mc_ptr != nullptr; }
size_t DeviceComm::arena_bytes() const { return impl_->arena->bytes; }
const char* DeviceComm::symm_mode() const { return mesh_->mode_name(); }

int DeviceComm::status() const {
  for (int v = 0; v < nlocal_; ++v) {
    int s = *reinterpret_cast<volatile int*>(impl_->status_host + v);
    if (s) return s;
  }
  return 0;
}

void DeviceComm::check_status() const {
  int s = status();
  if (!s && impl_->debug_bounds) check_canaries();
  if (!s) return;
  int phase = (s >> 8) & 0xff, peer = s & 0xff;
  MCCL_CHECK_T(phase != dev::PH_BOUNDS, ProtocolError,
               "MCCL_DEBUG_BOUNDS: a collective kernel on rank " << peer << " was given arguments whose staging extent exceeds "
                                                                 << "its arena half of " << impl_->half_bytes
                                                                 << " bytes; it returned without touching memory");
  MCCL_CHECK_T(false, TimeoutError,
               "device wait timed out: rank " << rank_ << " waited for rank " << peer << " in phase '"
                                              << phase_name(phase) << "' longer than "
                                              << impl_->timeout_ns / 1000000ull << " ms; the group must be rebuilt");
}

void DeviceComm::check_canaries() const {
  if (!impl_->debug_bounds) return;
  MCCL_CUDA_CHECK(cudaSetDevice(device_));
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  std::vector<unsigned char> host(kCanaryBytes);
  for (int v = 0; v < nlocal_; ++v) {
    const char* base = static_cast<const char*>(impl_->arena->ptrs[nlocal_ > 1 ? v : rank_]);
    MCCL_CUDA_CHECK(cudaMemcpy(host.data(), base + 2 * impl_->half_bytes, kCanaryBytes, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < kCanaryBytes; ++i)
      MCCL_CHECK_T(host[i] == 0xA5, ProtocolError,
                   "MCCL_DEBUG_BOUNDS: the canary behind the staging arena of rank " << (rank_ + v) << " was overwritten at byte "
                                                                                   << i << " (a kernel wrote past its arena half)");
  }
}

void DeviceComm::set_debug_arena_limit(size_t bytes) {
  MCCL_CHECK(impl_->debug_bounds, "set_debug_arena_limit needs MCCL_DEBUG_BOUNDS=1");
  impl_->debug_limit = bytes;
}

void DeviceComm::clear_status() { std::memset(impl_->status_host, 0, sizeof(int) * dev::kMaxRanks); }

void DeviceComm::inject_skip_signals(int count) {
  MCCL_CUDA_CHECK(cudaSetDevice(device_));
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  for (int ch = 0; ch < dev::kChannels; ++ch) {
    uint32_t v = static_cast<uint32_t>(count);
    MCCL_CUDA_CHECK(cudaMemcpy(&impl_->state[ch].skip_signals, &v, sizeof(v), cudaMemcpyHostToDevice));
  }
}

void DeviceComm::set_device_timeout_ms(int64_t ms) {
  impl_->timeout_ns = static_cast<unsigned long long>(std::max<int64_t>(ms, 1)) * 1000000ull;
}

int64_t DeviceComm::device_timeout_ms() const { return static_cast<int64_t>(impl_->timeout_ns / 1000000ull); }

void DeviceComm::set_launch_shape(int max_ctas, int threads) {
  if (max_ctas < 0) {
    // back to the defaults, large messages shaped automatically again
    impl_->max_ctas = std::min(cfg_.max_ctas > 0 ? cfg_.max_ctas : 64, dev::kMaxCtas);
    if (nlocal_ > 1) impl_->max_ctas = std::max(1, std::min(impl_->max_ctas, 96 / nlocal_));
    impl_->threads = 0;
    impl_->shape_auto = cfg_.max_ctas <= 0;
    return;
  }
  if (max_ctas > 0 || threads > 0) impl_->shape_auto = false;
  if (max_ctas > 0) {
    impl_->max_ctas = std::min(max_ctas, dev::kMaxCtas);
    if (nlocal_ > 1) impl_->max_ctas = std::max(1, std::min(impl_->max_ctas, 96 / nlocal_));
  }
  if (threads > 0) impl_->threads = std::max(128, std::min(threads, dev::kThreads)) / 32 * 32;
  if (threads < 0) impl_->threads = 0;   // back to the kernels' default
}
int DeviceComm::launch_threads() const { return impl_->threads; }
int DeviceComm::max_ctas() const { return impl_->max_ctas; }
bool DeviceComm::launch_shape_auto() const { return impl_->shape_auto; }

std::shared_ptr<SymmAlloc> DeviceComm::symm_alloc(size_t bytes) { return mesh_->alloc(bytes, true); }

// ------------------------------------------------------------------ helpers --
namespace {
int ctas_for(size_t bytes, int max_ctas) {
  // one CTA moves 8 KB per pass; aim at >= 4 passes per CTA before adding CTAs
  size_t want = (bytes + (32u << 10) - 1) / (32u << 10);
  return static_cast<int>(std::max<size_t>(1, std::min<size_t>(want, static_cast<size_t>(max_ctas))));
}
}  // namespace

Algo DeviceComm::decide_allreduce(Algo requested, size_t numel, DType t, RedOp op, WireDtype wire,
                                  int64_t tree_below) const {
  const bool bw = wire == WireDtype::BF16 && t == DType::F32;
  const size_t wire_bytes = numel * (bw ? 2 : dtype_size(t));
  const bool nvls_ok = nvls_available() && nlocal_ == 1 && (op == RedOp::SUM || op == RedOp::AVG) &&
                       (t == DType::F32 || t == DType::F16 || t == DType::BF16);
  Algo a = requested;
  if (a == Algo::AUTO) {
    // Measured on 8 x B200: one-shot wins up to a few hundred KB, two-shot above.  The
    // staged NVLS schedule pays two local copies and only wins when asked for by the
    // tuning table (MCCL_NVLS_ABOVE, wire bytes); buffers that already live in the
    // symmetric heap take the copy-free NVLS path through allreduce_symm instead.
    if (static_cast<int64_t>(wire_bytes) <= tree_below) a = Algo::ONESHOT;
    else if (nvls_ok && impl_->nvls_above > 0 && static_cast<int64_t>(wire_bytes) >= impl_->nvls_above) a = Algo::NVLS;
    else if (impl_->push_above > 0 && static_cast<int64_t>(wire_bytes) >= impl_->push_above) a = Algo::BUTTERFLY_PUSH;
    else a = Algo::BUTTERFLY;
  }
  if (a == Algo::NVLS && !nvls_ok) a = Algo::BUTTERFLY;
  if (a == Algo::RING && numel < static_cast<size_t>(world_)) a = Algo::TREE;
  return a;
}

Algo DeviceComm::allreduce(const void* const* ins, void* const* outs, size_t numel, DType t, RedOp op, Algo requested,
                           WireDtype wire, int64_t tree_below, void* stream) {
  MCCL_CHECK(world_ >= 2, "device allreduce needs at least two ranks");
  if (numel == 0) return Algo::ONESHOT;
  Impl::Ordered ordered(impl_.get(), stream);
  const dev::ElemType et = to_elem(t);
  const bool bw = wire == WireDtype::BF16 && t == DType::F32;
  const size_t es = dtype_size(t), wes = bw ? 2 : es;
  const Algo algo = decide_allreduce(requested, numel, t, op, wire, tree_below);
  const size_t half = impl_->half_bytes;

  // Largest piece (elements, multiple of 16*world) one launch can stage.
  auto need = [&](long long n) -> size_t {
    switch (algo) {
      case Algo::ONESHOT: return dev::oneshot_bytes(n, world_, wes);
      case Algo::RING: return dev::ring_bytes(n, world_, wes);
      case Algo::TREE: return dev::tree_bytes(n, world_, wes);
      case Algo::NVLS: return dev::nvls_bytes(n, world_, wes);
      case Algo::BUTTERFLY_PUSH: return dev::twoshot_push_bytes(n, world_, wes);
      default: return dev::twoshot_bytes(n, world_, wes);
    }
  };
  long long piece = static_cast<long long>(numel);
  if (need(piece) > half) {
    const long long unit = 16LL * world_;
    // need() is linear in n up to padding: scale down, then trim.
    piece = static_cast<long long>(static_cast<double>(half) / static_cast<double>(need(piece)) * piece);
    piece = std::max<long long>(unit, piece / unit * unit);
    while (piece > unit && need(piece) > half) piece -= unit;
    MCCL_CHECK(need(piece) <= half, "arena of " << impl_->arena->bytes << " bytes is too small; raise MCCL_ARENA_MB");
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (long long done = 0; done < static_cast<long long>(numel); done += piece) {
    const long long n = std::min<long long>(piece, static_cast<long long>(numel) - done);
    dev::CollArgs a{};
    for (int v = 0; v < nlocal_; ++v) {
      a.in[v] = static_cast<const char*>(ins[v]) + static_cast<size_t>(done) * es;
      a.out[v] = static_cast<char*>(outs[v]) + static_cast<size_t>(done) * es;
    }
    a.numel = n;
    a.per = dev::chunk_elems(n, world_);
    a.op = to_dev_op(op, t);
    a.inv_world = 1.0f / static_cast<float>(world_);
    dev::LaunchCfg cfg;
    cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
    cfg.stream = st;
    const bool whole = algo == Algo::ONESHOT || algo == Algo::TREE;  // these split the whole message over CTAs
    cfg.ctas = ctas_for(static_cast<size_t>(n) * wes / (whole ? 1 : world_), impl_->max_ctas);
    if (!whole) impl_->large_shape(static_cast<size_t>(n) * wes, nlocal_, cfg);
    dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 0);
    cudaError_t rc;
    switch (algo) {
      case Algo::ONESHOT: rc = dev::launch_allreduce_oneshot(et, bw, c, a, cfg); break;
      case Algo::RING: rc = dev::launch_allreduce_ring(et, bw, c, a, cfg); break;
      case Algo::TREE: rc = dev::launch_allreduce_tree(et, bw, c, a, cfg); break;
      case Algo::NVLS: rc = dev::launch_allreduce_nvls(et, bw, true, c, a, nullptr, nullptr, cfg); break;
      case Algo::BUTTERFLY_PUSH: rc = dev::launch_allreduce_twoshot_push(et, bw, c, a, cfg); break;
      default: rc = dev::launch_allreduce_twoshot(et, bw, c, a, cfg); break;
    }
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "allreduce(" << algo_name(algo) << ") launch failed: " << cudaGetErrorString(rc));
    ++launches_;
  }
  return algo;
}

Algo DeviceComm::allreduce_symm(const SymmAlloc& buf, size_t byte_offset, size_t numel, DType t, RedOp op, void* stream) {
  MCCL_CHECK(world_ >= 2, "device allreduce needs at least two ranks");
  MCCL_CHECK(op == RedOp::SUM || op == RedOp::AVG || buf.mc_ptr == nullptr, "in-switch reduction supports SUM and AVG");
  Impl::Ordered ordered(impl_.get(), stream);
  const size_t es = dtype_size(t);
  const long long per = dev::chunk_elems(static_cast<long long>(numel), world_);
  MCCL_CHECK(byte_offset % 16 == 0, "symmetric allreduce: offset must be a multiple of 16 bytes");
  MCCL_CHECK(byte_offset + static_cast<size_t>(per) * world_ * es <= buf.bytes,
             "symmetric allreduce: region (padded to " << per * world_ << " elements) exceeds the allocation");
  dev::CollArgs a{};
  a.numel = static_cast<long long>(numel);
  a.per = per;
  a.op = to_dev_op(op, t);
  a.inv_world = 1.0f / static_cast<float>(world_);
  dev::LaunchCfg cfg;
  cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cfg.ctas = ctas_for(static_cast<size_t>(per) * es, impl_->max_ctas);
  dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 1);
  const bool nvls = buf.mc_ptr != nullptr && nlocal_ == 1 && (op == RedOp::SUM || op == RedOp::AVG) &&
                    (t == DType::F32 || t == DType::F16 || t == DType::BF16);
  cudaError_t rc;
  if (nvls) {
    rc = dev::launch_allreduce_nvls(to_elem(t), false, false, c, a, static_cast<char*>(buf.ptrs[rank_]) + byte_offset,
                                    static_cast<char*>(buf.mc_ptr) + byte_offset, cfg);
  } else {
    for (int r = 0; r < world_; ++r) a.in[r] = static_cast<const char*>(buf.ptrs[r]) + byte_offset;
    rc = dev::launch_allreduce_symm(to_elem(t), c, a, cfg);
  }
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "symmetric allreduce launch failed: " << cudaGetErrorString(rc));
  ++launches_;
  return nvls ? Algo::NVLS : Algo::BUTTERFLY;
}

void DeviceComm::reduce_scatter(const void* const* ins, void* const* outs, size_t numel, DType t, RedOp op,
                                WireDtype wire, void* stream) {
  MCCL_CHECK(world_ >= 2, "device reduce_scatter needs at least two ranks");
  if (numel == 0) return;
  Impl::Ordered ordered(impl_.get(), stream);
  const dev::ElemType et = to_elem(t);
  const bool bw = wire == WireDtype::BF16 && t == DType::F32;
  const size_t es = dtype_size(t), wes = bw ? 2 : es;
  const size_t half = impl_->half_bytes;
  // The arena holds world slots of `per` wire elements; longer chunks go in pieces.
  const long long cap = static_cast<long long>(half / (static_cast<size_t>(world_) * wes)) / 16 * 16;
  MCCL_CHECK(cap >= 16, "arena too small for reduce_scatter; raise MCCL_ARENA_MB");
  const long long piece = std::min<long long>(static_cast<long long>(numel), cap);
  for (long long done = 0; done < static_cast<long long>(numel); done += piece) {
    const long long n = std::min<long long>(piece, static_cast<long long>(numel) - done);
    // Piece [done, done+n) of every chunk: shifted base pointers, full chunk stride.
    dev::CollArgs a{};
    for (int v = 0; v < nlocal_; ++v) {
      a.in[v] = static_cast<const char*>(ins[v]) + static_cast<size_t>(done) * es;
      a.out[v] = static_cast<char*>(outs[v]) + static_cast<size_t>(done) * es;
    }
    a.numel = n;
    a.stride = static_cast<long long>(numel);
    a.per = (n + 15) / 16 * 16;
    a.op = to_dev_op(op, t);
    a.inv_world = 1.0f / static_cast<float>(world_);
    dev::LaunchCfg cfg;
    cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.ctas = ctas_for(static_cast<size_t>(n) * wes, impl_->max_ctas);
    impl_->large_shape(static_cast<size_t>(n) * wes * static_cast<size_t>(world_), nlocal_, cfg);
    dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 0);
    cudaError_t rc = dev::launch_reduce_scatter(et, bw, c, a, cfg);
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "reduce_scatter launch failed: " << cudaGetErrorString(rc));
    ++launches_;
  }
}

void DeviceComm::allgather(const void* const* ins, void* const* outs, size_t nbytes, void* stream) {
  MCCL_CHECK(world_ >= 2, "device allgather needs at least two ranks");
  if (nbytes == 0) return;
  Impl::Ordered ordered(impl_.get(), stream);
  const size_t half = impl_->half_bytes;
  // every rank's piece has a slot of its own in each arena half
  const size_t piece = std::min(nbytes, (half / static_cast<size_t>(world_)) / 16 * 16);
  MCCL_CHECK(piece >= 16 || nbytes < 16, "arena too small for allgather; raise MCCL_ARENA_MB");
  for (size_t done = 0; done < nbytes; done += piece) {
    const size_t n = std::min(piece, nbytes - done);
    // Piece k of every rank's block lands at out + r*nbytes + done: express it
    // with shifted base pointers and the full block stride.
    dev::CollArgs a{};
    for (int v = 0; v < nlocal_; ++v) {
      a.in[v] = static_cast<const char*>(ins[v]) + done;
      a.out[v] = static_cast<char*>(outs[v]) + done;
    }
    a.numel = static_cast<long long>(n);
    a.reserved = (impl_->ag_multicast && nvls_available() && nlocal_ == 1) ? 1 : 0;   // replicate in the switch
    a.stride = static_cast<long long>(nbytes);  // distance between ranks' blocks in the output
    dev::LaunchCfg cfg;
    cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.ctas = ctas_for(n, impl_->max_ctas);
    impl_->large_shape(n * static_cast<size_t>(world_), nlocal_, cfg);
    dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 0);
    cudaError_t rc = dev::launch_allgather(c, a, cfg);
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "allgather launch failed: " << cudaGetErrorString(rc));
    ++launches_;
  }
}

void DeviceComm::broadcast(void* const* datas, size_t nbytes, int root, void* stream) {
  MCCL_CHECK(world_ >= 2, "device broadcast needs at least two ranks");
  if (nbytes == 0) return;
  Impl::Ordered ordered(impl_.get(), stream);
  const size_t half = impl_->half_bytes;
  // each launch scatters a piece into world slices of at most `half` bytes
  const size_t piece = std::min(nbytes, (half / 16 * 16) * static_cast<size_t>(world_) / 2);
  for (size_t done = 0; done < nbytes; done += piece) {
    const size_t n = std::min(piece, nbytes - done);
    dev::CollArgs a{};
    for (int v = 0; v < nlocal_; ++v) a.out[v] = static_cast<char*>(datas[v]) + done;
    a.numel = static_cast<long long>(n);
    a.root = root;
    dev::LaunchCfg cfg;
    cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.ctas = ctas_for(n / world_, impl_->max_ctas);
    dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 0);
    cudaError_t rc = dev::launch_broadcast(c, a, cfg);
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "broadcast launch failed: " << cudaGetErrorString(rc));
    ++launches_;
  }
}

void DeviceComm::alltoallv(const void* const* ins, void* const* outs, const std::vector<std::vector<size_t>>& in_off,
                           const std::vector<std::vector<size_t>>& in_len,
                           const std::vector<std::vector<size_t>>& out_off,
                           const std::vector<std::vector<size_t>>& out_len, void* stream) {
  MCCL_CHECK(world_ >= 2, "device alltoall needs at least two ranks");
  Impl::Ordered ordered(impl_.get(), stream);
  // One slot per source rank in each arena half, plus the control words the kernel uses to agree on the number
  // of rounds (segments longer than a slot go through in several rounds inside the one launch).
  const size_t ctl = static_cast<size_t>(dev::kMaxCtas) * dev::kMaxRanks * sizeof(unsigned long long);
  MCCL_CHECK(impl_->half_bytes > ctl + 16u * static_cast<size_t>(world_), "arena too small for alltoall; raise MCCL_ARENA_MB");
  const size_t slot = ((impl_->half_bytes - ctl) / static_cast<size_t>(world_)) / 16 * 16;
  size_t longest = 0;
  for (int v = 0; v < nlocal_; ++v)
    for (int p = 0; p < world_; ++p) longest = std::max({longest, in_len[v][p], out_len[v][p]});
  dev::A2AArgs a{};
  for (int v = 0; v < nlocal_; ++v) {
    a.in[v] = ins[v];
    a.out[v] = outs[v];
    for (int p = 0; p < world_; ++p) {
      a.in_off[v][p] = in_off[v][p];
      a.in_len[v][p] = in_len[v][p];
      a.out_off[v][p] = out_off[v][p];
      a.out_len[v][p] = out_len[v][p];
    }
  }
  a.slot_bytes = slot;
  dev::LaunchCfg cfg;
  cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cfg.ctas = ctas_for(longest, impl_->max_ctas);
  // The CTA count must agree across ranks although segment sizes differ, so it
  // cannot depend on this rank's sizes.
  cfg.ctas = impl_->max_ctas;
  dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 0);
  cudaError_t rc = dev::launch_alltoall(c, a, cfg);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "alltoall launch failed: " << cudaGetErrorString(rc));
  ++launches_;
}

// ---------------------------------------------------------------- send/recv --
namespace {
int p2p_ctas(size_t, size_t) {
  // Always the same number: a slot byte is then owned by the same CTA index in every message of a pair, and the
  // per-CTA ready / free flags are all the ordering the two slot buffers need across messages of any size.
  return dev::kP2PMaxCtas;
}
}  // namespace

size_t DeviceComm::p2p_slot_bytes() const { return impl_->p2p_slot; }

void DeviceComm::p2p_emulated(const std::vector<P2POp>& ops, size_t nbytes, void* stream) {
  MCCL_CHECK(static_cast<int>(ops.size()) == nlocal_, "p2p: expected one entry per local rank");
  if (nbytes == 0) return;
  dev::P2PComm c{};
  c.world = world_;
  c.rank_base = rank_;
  for (int r = 0; r < world_; ++r) {
    c.region[r] = static_cast<char*>(impl_->p2p->ptrs[r]);
    c.ready[r] = static_cast<uint32_t*>(impl_->pads->ptrs[r]) + 2 * static_cast<size_t>(dev::kFlagWordsPerChannel);
    c.free_[r] = static_cast<uint32_t*>(impl_->pads->ptrs[r]) + 3 * static_cast<size_t>(dev::kFlagWordsPerChannel);
  }
  for (int v = 0; v < nlocal_; ++v) {
    c.state[v] = impl_->p2p_state + v;
    c.status[v] = impl_->status_dev + v;
  }
  c.slot_bytes = impl_->p2p_slot;
  c.timeout_ns = impl_->timeout_ns;
  dev::P2PArgs a{};
  for (int v = 0; v < dev::kArgRanks; ++v) a.peer[v] = -1;
  for (int v = 0; v < nlocal_; ++v) {
    if (ops[v].peer < 0) continue;
    const int me = rank_ + v;
    MCCL_CHECK(ops[v].peer < world_ && ops[v].peer != me, "p2p: bad peer rank " << ops[v].peer);
    a.buf[v] = ops[v].buf;
    a.peer[v] = ops[v].peer;
    a.is_send[v] = ops[v].is_send ? 1 : 0;
  }
  a.nbytes = nbytes;
  dev::LaunchCfg cfg;
  cfg.nlocal = nlocal_;
  cfg.threads = 256;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cfg.ctas = p2p_ctas(nbytes, impl_->p2p_slot);
  cudaError_t rc = dev::launch_p2p(c, a, cfg);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "send/recv launch failed: " << cudaGetErrorString(rc));
  ++launches_;
}

void DeviceComm::send(const void* data, size_t nbytes, int peer, void* stream) {
  MCCL_CHECK(nlocal_ == 1, "send: use p2p_emulated with virtual ranks");
  p2p_emulated({P2POp{const_cast<void*>(data), peer, true}}, nbytes, stream);
}
void DeviceComm::recv(void* data, size_t nbytes, int peer, void* stream) {
  MCCL_CHECK(nlocal_ == 1, "recv: use p2p_emulated with virtual ranks");
  p2p_emulated({P2POp{data, peer, false}}, nbytes, stream);
}

void DeviceComm::barrier(void* stream) {
  if (world_ < 2) return;
  Impl::Ordered ordered(impl_.get(), stream);
  dev::LaunchCfg cfg;
  cfg.nlocal = nlocal_;
    cfg.threads = impl_->threads;
  cfg.stream = static_cast<cudaStream_t>(stream);
  dev::DevComm c = impl_->ctx(world_, rank_, nlocal_, 0);
  cudaError_t rc = dev::launch_barrier(c, cfg);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "barrier launch failed: " << cudaGetErrorString(rc));
  ++launches_;
}

}  // namespace mccl
