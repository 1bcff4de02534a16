#include "symm_mesh.hpp"

#include <cuda_runtime_api.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

#include "../core/errors.hpp"
#include "../core/log.hpp"
#include "cu_driver.hpp"

namespace mccl {

// ------------------------------------------------------------- fd passing --
// Each rank serves its exported handles on an abstract Unix socket.  A peer
// connects, names (allocation id, kind) and gets the descriptor back in an
// SCM_RIGHTS message.  A request for an allocation this rank has not exported
// yet waits until it has (the ranks reach the same alloc() call at different
// times).
struct SymmMesh::FdServer {
  struct Req {
    uint32_t id;
    uint32_t kind;  // 0 = memory handle, 1 = multicast handle
  };
  int lfd = -1;
  std::string name;  // without the leading NUL
  std::thread th;
  std::atomic<bool> stop{false};
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::pair<uint32_t, uint32_t>, int> table;
  int64_t timeout_ms;

  explicit FdServer(int64_t timeout) : timeout_ms(timeout) {
    std::random_device rd;
    char buf[96];
    std::snprintf(buf, sizeof(buf), "mccl-symm-%d-%08x%08x", static_cast<int>(getpid()), rd(), rd());
    name = buf;
    lfd = ::socket(AF_UNIX, SOCK_STREAM, 0);
    MCCL_CHECK_T(lfd >= 0, TransportError, "symm: unix socket() failed: " << std::strerror(errno));
    sockaddr_un addr{};
    socklen_t len = fill(addr, name);
    MCCL_CHECK_T(::bind(lfd, reinterpret_cast<sockaddr*>(&addr), len) == 0, TransportError,
                 "symm: bind of abstract socket failed: " << std::strerror(errno));
    MCCL_CHECK_T(::listen(lfd, 64) == 0, TransportError, "symm: listen failed: " << std::strerror(errno));
    th = std::thread([this] { serve(); });
  }
  ~FdServer() {
    stop = true;
    cv.notify_all();
    if (th.joinable()) th.join();
    if (lfd >= 0) ::close(lfd);
    for (auto& kv : table) ::close(kv.second);
  }
  static socklen_t fill(sockaddr_un& addr, const std::string& n) {
    addr.sun_family = AF_UNIX;
    addr.sun_path[0] = 0;
    std::memcpy(addr.sun_path + 1, n.data(), n.size());
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n.size());
  }
  void publish(uint32_t id, uint32_t kind, int fd) {
    {
      std::lock_guard<std::mutex> g(mu);
      table[{id, kind}] = fd;
    }
    cv.notify_all();
  }
  void retire(uint32_t id) {
    std::lock_guard<std::mutex> g(mu);
    for (auto it = table.begin(); it != table.end();) {
      if (it->first.first == id) {
        ::close(it->second);
        it = table.erase(it);
      } else {
        ++it;
      }
    }
  }
  void serve() {
    while (!stop) {
      pollfd pfd{lfd, POLLIN, 0};
      if (::poll(&pfd, 1, 100) <= 0) continue;
      int cfd = ::accept(lfd, nullptr, nullptr);
      if (cfd < 0) continue;
      Req rq{};
      ssize_t n = ::recv(cfd, &rq, sizeof(rq), MSG_WAITALL);
      int fd = -1;
      if (n == static_cast<ssize_t>(sizeof(rq))) {
        std::unique_lock<std::mutex> g(mu);
        cv.wait_for(g, std::chrono::milliseconds(timeout_ms),
                    [&] { return stop.load() || table.count({rq.id, rq.kind}) != 0; });
        auto it = table.find({rq.id, rq.kind});
        if (it != table.end()) fd = it->second;
      }
      char tag = fd >= 0 ? 'K' : 'E';
      iovec iov{&tag, 1};
      msghdr msg{};
      msg.msg_iov = &iov;
      msg.msg_iovlen = 1;
      alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
      if (fd >= 0) {
        std::memset(ctrl, 0, sizeof(ctrl));
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        cmsghdr* cm = CMSG_FIRSTHDR(&msg);
        cm->cmsg_level = SOL_SOCKET;
        cm->cmsg_type = SCM_RIGHTS;
        cm->cmsg_len = CMSG_LEN(sizeof(int));
        std::memcpy(CMSG_DATA(cm), &fd, sizeof(int));
      }
      ::sendmsg(cfd, &msg, MSG_NOSIGNAL);
      ::close(cfd);
    }
  }
  // Client side: asks the server named `peer_name` for a descriptor.
  static int fetch(const std::string& peer_name, uint32_t id, uint32_t kind, int64_t timeout_ms) {
    auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    int s = -1;
    for (;;) {
      s = ::socket(AF_UNIX, SOCK_STREAM, 0);
      MCCL_CHECK_T(s >= 0, TransportError, "symm: unix socket() failed: " << std::strerror(errno));
      sockaddr_un addr{};
      socklen_t len = fill(addr, peer_name);
      if (::connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) break;
      ::close(s);
      MCCL_CHECK_T(std::chrono::steady_clock::now() < deadline, TimeoutError,
                   "symm: could not reach the handle server '" << peer_name << "'");
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
    Req rq{id, kind};
    MCCL_CHECK_T(::send(s, &rq, sizeof(rq), MSG_NOSIGNAL) == static_cast<ssize_t>(sizeof(rq)), TransportError,
                 "symm: request to handle server failed");
    timeval tv{static_cast<time_t>(timeout_ms / 1000 + 1), 0};
    setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    char tag = 0;
    iovec iov{&tag, 1};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n = ::recvmsg(s, &msg, 0);
    ::close(s);
    MCCL_CHECK_T(n == 1 && tag == 'K', TransportError,
                 "symm: handle server '" << peer_name << "' had no handle for allocation " << id << "/" << kind);
    int fd = -1;
    for (cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm; cm = CMSG_NXTHDR(&msg, cm))
      if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
    MCCL_CHECK_T(fd >= 0, TransportError, "symm: reply from '" << peer_name << "' carried no descriptor");
    return fd;
  }
};

// Bookkeeping released with the last reference to an allocation.
struct SymmAlloc::Priv {
  SymmMesh::Mode mode = SymmMesh::Mode::LOCAL;
  int world = 1, rank = 0;
  size_t mapped = 0;
  CUmemGenericAllocationHandle handles[kSymmMaxRanks] = {};
  bool have_handle[kSymmMaxRanks] = {};
  CUdeviceptr vas[kSymmMaxRanks] = {};
  CUmemGenericAllocationHandle mc_handle = 0;
  bool have_mc = false, mc_bound = false;
  CUdeviceptr mc_va = 0;
  CUdevice cu_dev = 0;
  void* ipc_opened[kSymmMaxRanks] = {};
  void* owned[kSymmMaxRanks] = {};  // cudaMalloc'd blocks (IPC: own block, LOCAL: all)
  int device = -1;                  // CUDA device the mappings belong to

  ~Priv() {
    // Unmapping is immediate, not stream-ordered: kernels this process has queued on the allocation (the views it hands
    // out are ordinary tensors) must have finished first, or they touch unmapped addresses.  A peer that still reads
    // this rank's block keeps it alive through its own imported handle.
    if (device >= 0) {
      int cur = -1;
      if (cudaGetDevice(&cur) == cudaSuccess) {
        if (cur != device) cudaSetDevice(device);
        cudaDeviceSynchronize();
        if (cur != device && cur >= 0) cudaSetDevice(cur);
      }
    }
    // Teardown is best effort: the context may already be gone at exit.
    const CuDriver& cu = CuDriver::get();
    if (mode == SymmMesh::Mode::VMM && cu.loaded) {
      if (mc_va) {
        cu.MemUnmap(mc_va, mapped);
        cu.MemAddressFree(mc_va, mapped);
      }
      if (mc_bound) cu.MulticastUnbind(mc_handle, cu_dev, 0, mapped);
      if (have_mc) cu.MemRelease(mc_handle);
      for (int r = 0; r < world; ++r) {
        if (vas[r]) {
          cu.MemUnmap(vas[r], mapped);
          cu.MemAddressFree(vas[r], mapped);
        }
        if (have_handle[r]) cu.MemRelease(handles[r]);
      }
    }
    for (int r = 0; r < kSymmMaxRanks; ++r) {
      if (ipc_opened[r]) cudaIpcCloseMemHandle(ipc_opened[r]);
      if (owned[r]) cudaFree(owned[r]);
    }
  }
};

// ------------------------------------------------------------ construction --
SymmMesh::SymmMesh(int world, int device) : rank_(0), world_(world), device_(device), mode_(Mode::LOCAL) {
  MCCL_CHECK(world >= 1 && world <= kSymmMaxRanks, "symm: world " << world << " outside 1.." << kSymmMaxRanks);
  MCCL_CUDA_CHECK(cudaSetDevice(device));
}

SymmMesh::SymmMesh(KVStore* store, int rank, int world, int device, const std::string& prefix, const EnvConfig& cfg,
                   int64_t timeout_ms)
    : store_(store), rank_(rank), world_(world), device_(device), prefix_(prefix), timeout_ms_(timeout_ms) {
  MCCL_CHECK(world >= 1 && world <= kSymmMaxRanks,
             "symm: a device group spans at most " << kSymmMaxRanks << " GPUs of one NVSwitch domain, got " << world);
  MCCL_CUDA_CHECK(cudaSetDevice(device));
  MCCL_CUDA_CHECK(cudaFree(nullptr));  // make sure the primary context exists

  const CuDriver& cu = CuDriver::get();
  bool vmm_ok = cu.loaded && cfg.symm_mode != "ipc";
  int mc_attr = 0;
  if (vmm_ok) {
    CUdevice dev;
    vmm_ok = cu.DeviceGet(&dev, device) == CUDA_SUCCESS;
    int vmm_attr = 0, fd_attr = 0;
    if (vmm_ok) {
      cu.DeviceGetAttribute(&vmm_attr, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
      cu.DeviceGetAttribute(&fd_attr, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
      if (cu.multicast) cu.DeviceGetAttribute(&mc_attr, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
      vmm_ok = vmm_attr != 0 && fd_attr != 0;
    }
  }
  if (cfg.symm_mode == "vmm")
    MCCL_CHECK_T(vmm_ok, CudaError, "symm: MCCL_SYMM_MODE=vmm but this device cannot export VMM handles (" << cu.why << ")");
  // All ranks must take the same path.
  vmm_ok = all_ranks_agree("vmm", vmm_ok);
  mode_ = vmm_ok ? Mode::VMM : Mode::IPC;
  bool want_mc = vmm_ok && mc_attr != 0 && cfg.nvls != 0 && world > 1;
  multicast_ = all_ranks_agree("mc", want_mc);
  if (cfg.nvls == 1)
    MCCL_CHECK_T(multicast_, CudaError, "symm: MCCL_NVLS=1 but NVLink multicast is not available on every rank");

  if (mode_ == Mode::VMM) {
    server_.reset(new FdServer(timeout_ms));
    store_->set_str(prefix_ + "/uds/" + std::to_string(rank_), server_->name);
  }
  MCCL_INFO("symmetric mesh: rank " << rank << "/" << world << " on cuda:" << device << ", mode " << mode_name()
                                    << ", multicast " << (multicast_ ? "yes" : "no"));
}

SymmMesh::~SymmMesh() = default;

bool SymmMesh::all_ranks_agree(const std::string& what, bool mine) {
  if (world_ <= 1 || !store_) return mine;
  store_->set_str(prefix_ + "/cap/" + what + "/" + std::to_string(rank_), mine ? "1" : "0");
  bool all = mine;
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    all = all && store_->get_str(prefix_ + "/cap/" + what + "/" + std::to_string(r), timeout_ms_) == "1";
  }
  return all;
}

void SymmMesh::store_barrier(const std::string& tag) {
  if (world_ <= 1 || !store_) return;
  Rendezvous rdv(store_, rank_, world_, timeout_ms_, prefix_);
  rdv.barrier(tag);
}

std::shared_ptr<SymmAlloc> SymmMesh::alloc(size_t bytes, bool want_multicast) {
  MCCL_CHECK(bytes > 0, "symm: zero-byte allocation");
  MCCL_CUDA_CHECK(cudaSetDevice(device_));
  switch (mode_) {
    case Mode::VMM: return alloc_vmm(bytes, want_multicast && multicast_);
    case Mode::IPC: return alloc_ipc(bytes);
    default: return alloc_local(bytes);
  }
}

std::shared_ptr<SymmAlloc> SymmMesh::alloc_local(size_t bytes) {
  auto a = std::make_shared<SymmAlloc>();
  a->priv = std::make_shared<SymmAlloc::Priv>();
  a->priv->mode = Mode::LOCAL;
  a->priv->device = device_;
  a->bytes = (bytes + 255) / 256 * 256;
  a->world = world_;
  a->rank = 0;
  a->id = next_id_++;
  for (int r = 0; r < world_; ++r) {
    MCCL_CUDA_CHECK(cudaMalloc(&a->priv->owned[r], a->bytes));
    MCCL_CUDA_CHECK(cudaMemset(a->priv->owned[r], 0, a->bytes));
    a->ptrs[r] = a->priv->owned[r];
  }
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  return a;
}

std::shared_ptr<SymmAlloc> SymmMesh::alloc_ipc(size_t bytes) {
  auto a = std::make_shared<SymmAlloc>();
  a->priv = std::make_shared<SymmAlloc::Priv>();
  a->priv->mode = Mode::IPC;
  a->priv->device = device_;
  a->bytes = (bytes + 255) / 256 * 256;
  a->world = world_;
  a->rank = rank_;
  a->id = next_id_++;
  void* mine = nullptr;
  MCCL_CUDA_CHECK(cudaMalloc(&mine, a->bytes));
  a->priv->owned[rank_] = mine;
  a->ptrs[rank_] = mine;
  MCCL_CUDA_CHECK(cudaMemset(mine, 0, a->bytes));
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  MCCL_CUDA_CHECK(cudaIpcGetMemHandle(&h, mine));
  const std::string base = prefix_ + "/ipc/" + std::to_string(a->id) + "/";
  store_->set(base + std::to_string(rank_), std::vector<uint8_t>(reinterpret_cast<uint8_t*>(&h), reinterpret_cast<uint8_t*>(&h) + sizeof(h)));
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    auto raw = store_->get(base + std::to_string(r), timeout_ms_);
    MCCL_CHECK_T(raw.size() == sizeof(h), ProtocolError, "symm: malformed IPC handle from rank " << r);
    cudaIpcMemHandle_t ph;
    std::memcpy(&ph, raw.data(), sizeof(ph));
    void* p = nullptr;
    MCCL_CUDA_CHECK(cudaIpcOpenMemHandle(&p, ph, cudaIpcMemLazyEnablePeerAccess));
    a->priv->ipc_opened[r] = p;
    a->ptrs[r] = p;
  }
  store_barrier("ipc-mapped-" + std::to_string(a->id));
  return a;
}

std::shared_ptr<SymmAlloc> SymmMesh::alloc_vmm(size_t bytes, bool want_mc) {
  const CuDriver& cu = CuDriver::get();
  auto a = std::make_shared<SymmAlloc>();
  a->priv = std::make_shared<SymmAlloc::Priv>();
  SymmAlloc::Priv& pv = *a->priv;
  pv.mode = Mode::VMM;
  pv.device = device_;
  pv.world = world_;
  pv.rank = rank_;
  a->world = world_;
  a->rank = rank_;
  a->id = next_id_++;
  const std::string idstr = std::to_string(a->id);
  MCCL_CU_CHECK(cu.DeviceGet(&pv.cu_dev, device_));

  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  MCCL_CU_CHECK(cu.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  CUmulticastObjectProp mcprop{};
  if (want_mc) {
    mcprop.numDevices = static_cast<unsigned>(world_);
    mcprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcprop.flags = 0;
    mcprop.size = (bytes + gran - 1) / gran * gran;
    size_t mcgran = 0;
    if (cu.MulticastGetGranularity(&mcgran, &mcprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mcgran > gran)
      gran = mcgran;
  }
  const size_t size = (bytes + gran - 1) / gran * gran;
  pv.mapped = size;
  a->bytes = size;
  mcprop.size = size;

  // 1. create + export my block
  MCCL_CU_CHECK(cu.MemCreate(&pv.handles[rank_], size, &prop, 0));
  pv.have_handle[rank_] = true;
  int my_fd = -1;
  MCCL_CU_CHECK(cu.MemExportToShareableHandle(&my_fd, pv.handles[rank_], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  server_->publish(a->id, 0, my_fd);

  // 2. import every peer's block
  // the peers' socket names never change: asked from the store once per mesh, not once per allocation
  if (peer_names_.empty()) {
    std::vector<std::string> fetched(world_);
    for (int r = 0; r < world_; ++r)
      if (r != rank_) fetched[r] = store_->get_str(prefix_ + "/uds/" + std::to_string(r), timeout_ms_);
    peer_names_ = std::move(fetched);
  }
  const std::vector<std::string>& names = peer_names_;
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    int fd = FdServer::fetch(names[r], a->id, 0, timeout_ms_);
    CUresult rc = cu.MemImportFromShareableHandle(&pv.handles[r], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    MCCL_CHECK_T(rc == CUDA_SUCCESS, CudaError, "symm: import of rank " << r << "'s block failed: " << cu.error_string(rc));
    pv.have_handle[r] = true;
  }

  // 3. map all blocks read/write for this device
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < world_; ++r) {
    MCCL_CU_CHECK(cu.MemAddressReserve(&pv.vas[r], size, gran, 0, 0));
    MCCL_CU_CHECK(cu.MemMap(pv.vas[r], size, 0, pv.handles[r], 0));
    MCCL_CU_CHECK(cu.MemSetAccess(pv.vas[r], size, &access, 1));
    a->ptrs[r] = reinterpret_cast<void*>(pv.vas[r]);
  }

  // 4. optional multicast object.  Failures are recorded, not thrown, until
  // every rank has passed the same store barriers.
  bool mc_ok = want_mc;
  if (want_mc) {
    if (rank_ == 0) {
      CUresult rc = cu.MulticastCreate(&pv.mc_handle, &mcprop);
      int mfd = -1;
      if (rc == CUDA_SUCCESS) {
        pv.have_mc = true;
        rc = cu.MemExportToShareableHandle(&mfd, pv.mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      }
      if (rc != CUDA_SUCCESS) {
        MCCL_WARN("symm: multicast object creation failed: " << cu.error_string(rc));
        mc_ok = false;
      }
      store_->set_str(prefix_ + "/mc/" + idstr + "/created", mc_ok ? "1" : "0");
      if (mc_ok) server_->publish(a->id, 1, mfd);
    } else {
      mc_ok = store_->get_str(prefix_ + "/mc/" + idstr + "/created", timeout_ms_) == "1";
      if (mc_ok) {
        try {
          int mfd = FdServer::fetch(names[0], a->id, 1, timeout_ms_);
          CUresult rc = cu.MemImportFromShareableHandle(&pv.mc_handle, reinterpret_cast<void*>(static_cast<uintptr_t>(mfd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
          ::close(mfd);
          if (rc == CUDA_SUCCESS) pv.have_mc = true;
          else mc_ok = false;
        } catch (const std::exception& e) {
          MCCL_WARN("symm: multicast handle fetch failed: " << e.what());
          mc_ok = false;
        }
      }
    }
    if (mc_ok && cu.MulticastAddDevice(pv.mc_handle, pv.cu_dev) != CUDA_SUCCESS) mc_ok = false;
    mc_ok = all_ranks_agree("mc-added-" + idstr, mc_ok);  // doubles as the "all devices added" barrier
    if (mc_ok) {
      CUresult rc = cu.MulticastBindMem(pv.mc_handle, 0, pv.handles[rank_], 0, size, 0);
      if (rc == CUDA_SUCCESS) pv.mc_bound = true;
      else {
        MCCL_WARN("symm: cuMulticastBindMem failed: " << cu.error_string(rc));
        mc_ok = false;
      }
    }
    if (mc_ok) {
      CUresult rc = cu.MemAddressReserve(&pv.mc_va, size, gran, 0, 0);
      if (rc == CUDA_SUCCESS) rc = cu.MemMap(pv.mc_va, size, 0, pv.mc_handle, 0);
      if (rc == CUDA_SUCCESS) rc = cu.MemSetAccess(pv.mc_va, size, &access, 1);
      if (rc != CUDA_SUCCESS) {
        MCCL_WARN("symm: mapping the multicast object failed: " << cu.error_string(rc));
        mc_ok = false;
      }
    }
    mc_ok = all_ranks_agree("mc-bound-" + idstr, mc_ok);
    if (mc_ok) a->mc_ptr = reinterpret_cast<void*>(pv.mc_va);
  }

  // 5. zero my block, then meet so that nobody touches a block before it is
  // zeroed and nobody closes a descriptor a peer still has to fetch.
  MCCL_CUDA_CHECK(cudaMemset(a->ptrs[rank_], 0, size));
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  store_barrier("vmm-ready-" + idstr);
  server_->retire(a->id);
  return a;
}

}  // namespace mccl
