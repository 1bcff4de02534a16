// Python bindings of the distributed runtime: distributed memory (dmem),
// coherence, scheduler, cluster manager, node agent and kernel dispatch.
//
// The module-level dmem functions answer the names the reference's Python
// layer imports from its extension but never got (register_region,
// unregister_region, put, get, poll_completion, drain_pending, metal_sync,
// init_dmem, shutdown_dmem, get_stats: mccl/distributed/tensor.py:19-27,
// mccl/cli.py:34-54).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "../cluster/agent.hpp"
#include "../cluster/cluster_manager.hpp"
#include "../cluster/scheduler.hpp"
#include "../coherence/coherence.hpp"
#include "../core/errors.hpp"
#include "../dmem/dmem_kernels.hpp"
#include "../dmem/dmem_manager.hpp"
#include "../dmem/shm_domain.hpp"
#include "../dmem/symm_fabric.hpp"
#include "../pg/process_group.hpp"
#include "../pg/device_comm.hpp"
#include "../runtime/kernel_dispatch.hpp"
#include "../symm/symm_mesh.hpp"
#include "bind.hpp"

namespace py = pybind11;

namespace mccl {

namespace {

py::dict job_to_dict(const Job& j) {
  py::dict d;
  d["id"] = j.id;
  d["name"] = j.spec.name;
  d["tenant"] = j.spec.tenant;
  d["priority"] = job_priority_name(j.spec.priority);
  d["nodes_required"] = j.spec.nodes_required;
  d["memory_per_node"] = j.spec.memory_per_node;
  d["command"] = j.spec.command;
  d["state"] = job_state_name(j.state);
  d["nodes"] = j.nodes;
  d["preemptions"] = j.preemptions;
  d["reason"] = j.reason;
  return d;
}

JobPriority parse_priority(const std::string& s) {
  if (s == "LOW" || s == "low") return JobPriority::LOW;
  if (s == "NORMAL" || s == "normal") return JobPriority::NORMAL;
  if (s == "HIGH" || s == "high") return JobPriority::HIGH;
  if (s == "CRITICAL" || s == "critical") return JobPriority::CRITICAL;
  MCCL_CHECK(false, "unknown priority '" << s << "'");
  return JobPriority::NORMAL;
}

JobSpec make_spec(const std::string& name, const std::string& tenant, const std::string& priority, int nodes, uint64_t mem,
                  const std::string& command) {
  JobSpec s;
  s.name = name;
  s.tenant = tenant;
  s.priority = parse_priority(priority);
  s.nodes_required = nodes;
  s.memory_per_node = mem;
  s.command = command;
  return s;
}

py::dict tick_to_dict(const TickResult& r) {
  py::list started;
  for (auto& p : r.started) started.append(py::make_tuple(p.job_id, p.nodes));
  py::dict d;
  d["started"] = started;
  d["preempted"] = r.preempted;
  return d;
}

std::vector<NodeLoad> loads_from(const std::vector<std::tuple<int, bool, uint64_t, uint64_t>>& in) {
  std::vector<NodeLoad> out;
  for (auto& t : in) {
    NodeLoad l;
    l.node_id = std::get<0>(t);
    l.online = std::get<1>(t);
    l.memory_total = std::get<2>(t);
    l.memory_used = std::get<3>(t);
    out.push_back(l);
  }
  return out;
}

py::dict dmem_stats_dict(const DmemStats& s) {
  py::dict d;
  d["total_put_bytes"] = s.total_put_bytes;
  d["total_get_bytes"] = s.total_get_bytes;
  d["total_put_ops"] = s.total_put_ops;
  d["total_get_ops"] = s.total_get_ops;
  d["total_errors"] = s.total_errors;
  d["regions"] = s.regions;
  d["pending"] = s.pending;
  return d;
}

// Process-wide manager behind the module-level dmem functions.
struct GlobalDmem {
  std::shared_ptr<DmemFabric> fabric;
  std::shared_ptr<ShmFabric> shm;   // set when the peers are other processes of this box
  std::shared_ptr<SymmFabric> symm; // set when the peers are the GPUs of a process group (regions in the symmetric heap)
  std::shared_ptr<DeviceComm> comm; // the group's device communicator (symm only)
  c10::intrusive_ptr<ProcessGroupMCCL> pg;  // keeps the store alive (symm only)
  std::vector<std::unique_ptr<DistributedMemoryManager>> nodes;  // in-process emulation: one per node; otherwise only this node
  int self = 0;
};
GlobalDmem& gd() {
  static GlobalDmem g;
  return g;
}
DistributedMemoryManager& self_mgr() {
  MCCL_CHECK(!gd().nodes.empty(), "dmem is not initialised; call init_dmem(node_id, num_peers) first");
  return *gd().nodes[(gd().shm || gd().symm) ? 0 : static_cast<size_t>(gd().self)];
}
// Stream the module-level device copies run on: the current stream of the communicator's GPU.
void* dmem_stream() {
  if (!gd().comm) return nullptr;
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(gd().comm->device())).stream());
}

// Stream-ordered acquire / release between the GPUs of a device communicator.
class GpuCoherence {
 public:
  explicit GpuCoherence(std::shared_ptr<DeviceComm> comm) : comm_(std::move(comm)) {
    MCCL_CHECK(comm_->nlocal() == 1, "gpu coherence needs one process per GPU");
    pads_ = comm_->symm_alloc(4096);
    const int w = comm_->world();
    std::vector<unsigned int*> host(static_cast<size_t>(w));
    for (int r = 0; r < w; ++r) host[static_cast<size_t>(r)] = static_cast<unsigned int*>(pads_->ptrs[r]);
    MCCL_CHECK_T(cudaMalloc(&table_, sizeof(unsigned int*) * w) == cudaSuccess, CudaError, "cudaMalloc failed");
    cudaMemcpy(table_, host.data(), sizeof(unsigned int*) * w, cudaMemcpyHostToDevice);
    MCCL_CHECK_T(cudaHostAlloc(&status_, sizeof(int), cudaHostAllocMapped) == cudaSuccess, CudaError, "cudaHostAlloc failed");
    *status_ = 0;
    cudaHostGetDevicePointer(&status_dev_, status_, 0);
  }
  ~GpuCoherence() {
    if (table_) cudaFree(table_);
    if (status_) cudaFreeHost(status_);
  }
  // Everything this stream wrote so far becomes visible to peers that acquire `epoch`.
  unsigned int release(void* stream) {
    ++epoch_;
    cudaError_t rc = launch_coherence_release(table_, comm_->world(), comm_->rank(), epoch_, static_cast<cudaStream_t>(stream));
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "gpu_release launch failed: " << cudaGetErrorString(rc));
    return epoch_;
  }
  // Later work on the stream runs after every peer has released `epoch`.
  void acquire(unsigned int epoch, int64_t timeout_ms, void* stream) {
    cudaError_t rc = launch_coherence_acquire(static_cast<unsigned int*>(pads_->ptrs[comm_->rank()]), comm_->world(), comm_->rank(),
                                              epoch, static_cast<unsigned long long>(timeout_ms) * 1000000ull, status_dev_,
                                              static_cast<cudaStream_t>(stream));
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "gpu_acquire launch failed: " << cudaGetErrorString(rc));
  }
  int status() const { return *reinterpret_cast<volatile int*>(status_); }
  void clear_status() { *status_ = 0; }
  unsigned int epoch() const { return epoch_; }

 private:
  std::shared_ptr<DeviceComm> comm_;
  std::shared_ptr<SymmAlloc> pads_;
  unsigned int** table_ = nullptr;
  int* status_ = nullptr;
  int* status_dev_ = nullptr;
  unsigned int epoch_ = 0;
};

}  // namespace

void bind_runtime(py::module_& m) {
  // ------------------------------------------------------------- scheduler --
  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init([] { return new Scheduler(); }))
      .def("submit",
           [](Scheduler& s, const std::string& name, const std::string& tenant, const std::string& priority, int nodes,
              uint64_t mem, const std::string& command) { return s.submit(make_spec(name, tenant, priority, nodes, mem, command)); },
           py::arg("name"), py::arg("tenant") = "default", py::arg("priority") = "NORMAL", py::arg("nodes") = 1,
           py::arg("memory_per_node") = 0, py::arg("command") = "")
      .def("cancel", &Scheduler::cancel)
      .def("complete", &Scheduler::complete, py::arg("job_id"), py::arg("ok") = true, py::arg("reason") = "")
      .def("schedule_tick",
           [](Scheduler& s, const std::vector<std::tuple<int, bool, uint64_t, uint64_t>>& loads) {
             return tick_to_dict(s.schedule_tick(loads_from(loads)));
           },
           "loads: list of (node_id, online, memory_total, memory_used)")
      .def("evict_node", &Scheduler::evict_node)
      .def("get",
           [](Scheduler& s, uint64_t id) -> py::object {
             Job j;
             if (!s.get(id, &j)) return py::none();
             return job_to_dict(j);
           })
      .def("jobs",
           [](Scheduler& s) {
             py::list out;
             for (auto& j : s.jobs()) out.append(job_to_dict(j));
             return out;
           })
      .def("queue",
           [](Scheduler& s) {
             py::list out;
             for (auto& j : s.queue()) out.append(job_to_dict(j));
             return out;
           })
      .def("tenant_node_seconds", &Scheduler::tenant_node_seconds)
      .def("set_tenant_weight", &Scheduler::set_tenant_weight)
      .def("running_count", &Scheduler::running_count);

  // ----------------------------------------------------------------- agent --
  py::class_<AgentServer>(m, "AgentServer")
      .def(py::init<>())
      .def("start", &AgentServer::start, py::arg("port") = 0, py::arg("any") = false)
      .def("stop", &AgentServer::stop, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("port", &AgentServer::port)
      .def_property_readonly("running", &AgentServer::running)
      .def_property_readonly("pings", &AgentServer::pings)
      .def_property_readonly("runs", &AgentServer::runs)
      .def("regions", &AgentServer::regions)
      .def("set_unresponsive", &AgentServer::set_unresponsive)
      .def("set_run_handler", [](AgentServer& a, py::function fn) {
        auto holder = std::shared_ptr<py::function>(new py::function(std::move(fn)), [](py::function* f) {
          f->release();
          delete f;
        });
        a.set_run_handler([holder](const std::string& k, uint64_t off, uint64_t cnt) {
          py::gil_scoped_acquire gil;
          return (*holder)(k, off, cnt).cast<int>();
        });
      });
  m.def(
      "agent_request",
      [](const std::string& host, int port, int cmd, py::bytes payload, int timeout_ms) {
        std::string p = payload;
        AgentReply r;
        {
          py::gil_scoped_release rel;
          r = agent_request(host, port, static_cast<AgentCmd>(cmd), std::vector<uint8_t>(p.begin(), p.end()), timeout_ms);
        }
        return py::make_tuple(r.ok, static_cast<int>(r.status), py::bytes(std::string(r.payload.begin(), r.payload.end())), r.error);
      },
      py::arg("host"), py::arg("port"), py::arg("cmd"), py::arg("payload") = py::bytes(), py::arg("timeout_ms") = 1000);
  m.attr("AGENT_PING") = static_cast<int>(AgentCmd::PING);
  m.attr("AGENT_REGISTER") = static_cast<int>(AgentCmd::REGISTER);
  m.attr("AGENT_DEREGISTER") = static_cast<int>(AgentCmd::DEREGISTER);
  m.attr("AGENT_KERNEL_LOAD") = static_cast<int>(AgentCmd::KERNEL_LOAD);
  m.attr("AGENT_KERNEL_RUN") = static_cast<int>(AgentCmd::KERNEL_RUN);
  m.attr("AGENT_KERNEL_SYNC") = static_cast<int>(AgentCmd::KERNEL_SYNC);
  m.attr("AGENT_STATS") = static_cast<int>(AgentCmd::STATS);
  m.attr("AGENT_SHUTDOWN") = static_cast<int>(AgentCmd::SHUTDOWN);

  // ------------------------------------------------------- cluster manager --
  py::class_<ClusterManager>(m, "ClusterManager")
      .def(py::init([](int self, int hb_ms, int timeout_ms, int ping_ms, int tick_ms) {
             ClusterTimings t;
             t.heartbeat_interval_ms = hb_ms;
             t.heartbeat_timeout_ms = timeout_ms;
             t.ping_socket_timeout_ms = ping_ms;
             t.scheduler_tick_ms = tick_ms;
             return new ClusterManager(self, t);
           }),
           py::arg("self_node") = 0, py::arg("heartbeat_interval_ms") = 500, py::arg("heartbeat_timeout_ms") = 2000,
           py::arg("ping_socket_timeout_ms") = 1000, py::arg("scheduler_tick_ms") = 1000)
      .def("join",
           [](ClusterManager& c, int node, const std::string& host, int port, uint64_t mem_total) {
             NodeInfo n;
             n.node_id = node;
             n.host = host;
             n.agent_port = port;
             n.memory_total = mem_total;
             return c.handle_join(n);
           },
           py::arg("node_id"), py::arg("host") = "127.0.0.1", py::arg("agent_port") = 0, py::arg("memory_total") = 0)
      .def("leave", &ClusterManager::handle_leave)
      .def("heartbeat", &ClusterManager::handle_heartbeat, py::arg("node_id"), py::arg("memory_used") = 0)
      .def("node_failure", &ClusterManager::handle_node_failure)
      .def("leader", &ClusterManager::leader)
      .def("is_leader", &ClusterManager::is_leader)
      .def("online_count", &ClusterManager::online_count)
      .def("version", &ClusterManager::version)
      .def("nodes",
           [](ClusterManager& c) {
             py::list out;
             for (auto& n : c.nodes()) {
               py::dict d;
               d["node_id"] = n.node_id;
               d["host"] = n.host;
               d["agent_port"] = n.agent_port;
               d["status"] = n.status == NodeStatus::ONLINE ? "ONLINE" : (n.status == NodeStatus::SUSPECT ? "SUSPECT" : "OFFLINE");
               d["heartbeats"] = n.heartbeats;
               d["memory_total"] = n.memory_total;
               d["memory_used"] = n.memory_used;
               out.append(d);
             }
             return out;
           })
      .def("start", &ClusterManager::start)
      .def("stop", &ClusterManager::stop, py::call_guard<py::gil_scoped_release>())
      .def("scheduler", &ClusterManager::scheduler, py::return_value_policy::reference_internal)
      .def("catalog_size", [](ClusterManager& c) { return c.catalog().size(); })
      .def("publish_region",
           [](ClusterManager& c, int node, uint32_t region, uint64_t addr, uint64_t len) {
             RegionDirectoryEntry e;
             e.local_addr = addr;
             e.length = len;
             return c.publish_region(node, region, e);
           })
      .def("lookup_region", [](ClusterManager& c, int node, uint32_t region) -> py::object {
        RegionDirectoryEntry e;
        if (!c.lookup_region(node, region, &e)) return py::none();
        return py::make_tuple(e.local_addr, e.length);
      });

  // ------------------------------------------------------------------ dmem --
  py::class_<DmemFabric, std::shared_ptr<DmemFabric>>(m, "DmemFabric");
  py::class_<LocalFabric, DmemFabric, std::shared_ptr<LocalFabric>>(m, "LocalFabric").def(py::init<int>(), py::arg("num_nodes"));
  py::class_<ShmFabric, DmemFabric, std::shared_ptr<ShmFabric>>(m, "ShmFabric")
      .def(py::init<const std::string&, int, int, int>(), py::arg("name"), py::arg("node"), py::arg("num_nodes"),
           py::arg("timeout_ms") = 10000, py::call_guard<py::gil_scoped_release>(),
           "Fabric of one process of a job on this box: region directory, immediates and coherence mailboxes in POSIX "
           "shared memory (node 0 creates them), host regions in shared heaps.")
      .def("alloc_heap",
           [](ShmFabric& f, uint64_t bytes) {
             auto r = f.alloc_heap(bytes);
             return py::make_tuple(r.first, reinterpret_cast<uintptr_t>(r.second));
           },
           py::arg("nbytes"), "Returns (heap id, address) of a zeroed heap every process of the job can map.")
      .def("collect_imm", [](ShmFabric& f) {
        py::list out;
        for (auto& r : f.collect_imm()) out.append(py::make_tuple(r.src_node, r.region_id, r.offset, r.length, r.imm));
        return out;
      });
  m.attr("REGION_HOST_HEAP") = static_cast<uint32_t>(REGION_HOST_HEAP);
  py::class_<DistributedMemoryManager>(m, "DmemManager")
      .def(py::init([](int node, std::shared_ptr<DmemFabric> f) { return new DistributedMemoryManager(static_cast<uint16_t>(node), f); }),
           py::arg("node_id"), py::arg("fabric"), py::keep_alive<1, 3>())
      .def_property_readonly("node_id", &DistributedMemoryManager::node_id)
      .def("register_region",
           [](DistributedMemoryManager& d, uintptr_t ptr, uint64_t n, uint32_t flags, uint32_t heap_id, uint64_t heap_offset) {
             if (heap_id != 0 && !(flags & REGION_DEVICE)) flags |= REGION_HOST_HEAP;
             return d.register_region(reinterpret_cast<void*>(ptr), n, flags, heap_id, heap_offset);
           },
           py::arg("ptr"), py::arg("nbytes"), py::arg("flags") = static_cast<uint32_t>(REGION_READABLE | REGION_WRITABLE | REGION_SHARED),
           py::arg("heap_id") = 0, py::arg("heap_offset") = 0,
           "heap_id / heap_offset: the shared heap (ShmFabric.alloc_heap) the memory was carved from and its offset inside it.")
      .def("unregister_region", &DistributedMemoryManager::unregister_region)
      .def("put",
           [](DistributedMemoryManager& d, int node, uint32_t region, uint64_t off, uintptr_t src, uint64_t len) {
             return d.put(GlobalAddress(static_cast<uint16_t>(node), region, off), reinterpret_cast<const void*>(src), len);
           })
      .def("get",
           [](DistributedMemoryManager& d, int node, uint32_t region, uint64_t off, uintptr_t dst, uint64_t len) {
             return d.get(reinterpret_cast<void*>(dst), GlobalAddress(static_cast<uint16_t>(node), region, off), len);
           })
      .def("put_with_imm",
           [](DistributedMemoryManager& d, int node, uint32_t region, uint64_t off, uintptr_t src, uint64_t len, uint32_t imm) {
             return d.put_with_imm(GlobalAddress(static_cast<uint16_t>(node), region, off), reinterpret_cast<const void*>(src), len, imm);
           })
      .def("fence", [](DistributedMemoryManager& d) { d.fence(); })
      .def("poll_completion", &DistributedMemoryManager::poll_completion, py::arg("wr_id"), py::arg("timeout_ms") = 5000)
      .def("drain_pending", &DistributedMemoryManager::drain_pending)
      .def("take_immediates",
           [](DistributedMemoryManager& d) {
             py::list out;
             for (auto& r : d.take_immediates()) out.append(py::make_tuple(r.src_node, r.region_id, r.offset, r.length, r.imm));
             return out;
           })
      .def("stats", [](DistributedMemoryManager& d) { return dmem_stats_dict(d.stats()); })
      .def("catalog_size", [](DistributedMemoryManager& d) { return d.catalog().size(); })
      .def("catalog_roundtrip", [](DistributedMemoryManager& d) {
        MemoryCatalog c2;
        int n = c2.deserialize(d.catalog().serialize());
        return py::make_tuple(n, c2.size());
      });

  m.def(
      "init_dmem",
      [](int node_id, int num_peers, const std::string& shm_name) {
        GlobalDmem& g = gd();
        MCCL_CHECK(g.nodes.empty(), "dmem is already initialised");
        const int n = num_peers + 1;
        MCCL_CHECK(node_id >= 0 && node_id < n && n <= kDmemMaxNodes, "init_dmem: bad node_id / num_peers");
        g.self = node_id;
        if (!shm_name.empty()) {
          // the peers are other processes of this box: directory and heaps in shared memory
          g.shm = std::make_shared<ShmFabric>(shm_name, node_id, n);
          g.fabric = g.shm;
          g.nodes.emplace_back(new DistributedMemoryManager(static_cast<uint16_t>(node_id), g.fabric));
          return;
        }
        auto local = std::make_shared<LocalFabric>(n);
        g.fabric = local;
        for (int i = 0; i < n; ++i) g.nodes.emplace_back(new DistributedMemoryManager(static_cast<uint16_t>(i), g.fabric));
      },
      py::arg("node_id") = 0, py::arg("num_peers") = 0, py::arg("shm_name") = "", py::call_guard<py::gil_scoped_release>(),
      "Without shm_name all nodes are emulated inside this process; with it the nodes are the processes of one box that "
      "pass the same name (node 0 creates the shared directory).");
  m.def(
      "init_dmem_symm",
      [](ProcessGroupMCCL& pg_ref, int device_index) {
        // the Python object owns the group; share that ownership for as long as dmem is initialised
        c10::intrusive_ptr<ProcessGroupMCCL> pg = c10::intrusive_ptr<ProcessGroupMCCL>::reclaim_copy(&pg_ref);
        GlobalDmem& g = gd();
        MCCL_CHECK(g.nodes.empty(), "dmem is already initialised");
        MCCL_CHECK(pg->getSize() <= kDmemMaxNodes, "init_dmem_symm: group too large");
        g.comm = pg->deviceComm(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device_index)));
        g.pg = pg;
        g.self = pg->getRank();
        auto rings = g.comm->symm_alloc(SymmFabric::ring_bytes(pg->getSize()));
        g.symm = std::make_shared<SymmFabric>(pg->kv(), pg->getRank(), pg->getSize(), "mccl/dmem", pg->timeoutMs(), rings);
        g.fabric = g.symm;
        g.nodes.emplace_back(new DistributedMemoryManager(static_cast<uint16_t>(pg->getRank()), g.fabric));
      },
      py::arg("process_group"), py::arg("device_index"), py::call_guard<py::gil_scoped_release>(),
      "Collective over a backend='mccl' group with one GPU per rank: the nodes are the ranks, regions live in symmetric "
      "heaps (alloc_symm_heap) that every rank maps over NVLink, and put / get / put_with_imm run on the current CUDA stream.");
  m.def(
      "alloc_symm_heap",
      [](uint64_t nbytes) {
        MCCL_CHECK(gd().symm != nullptr, "alloc_symm_heap needs init_dmem_symm(process_group, device)");
        std::shared_ptr<SymmAlloc> a;
        {
          py::gil_scoped_release nogil;   // collective: may wait for the peers
          a = gd().comm->symm_alloc(nbytes);
        }
        const uint32_t heap_id = a->id + 1;   // 0 means "not in a heap"
        gd().symm->add_heap(heap_id, a);
        return py::make_tuple(heap_id, a);
      },
      py::arg("nbytes"),
      "Collective.  Returns (heap id, SymmAlloc): device memory of `nbytes` on every rank, each block mapped in every process.");
  m.def("shutdown_dmem", [] {
    gd().nodes.clear();
    gd().fabric.reset();
    gd().shm.reset();
    gd().symm.reset();
    gd().comm.reset();
    gd().pg.reset();
  });
  m.def("alloc_dmem_heap", [](uint64_t nbytes) {
    MCCL_CHECK(gd().shm != nullptr, "alloc_dmem_heap needs init_dmem(..., shm_name=...)");
    auto r = gd().shm->alloc_heap(nbytes);
    return py::make_tuple(r.first, reinterpret_cast<uintptr_t>(r.second));
  }, py::arg("nbytes"), "Returns (heap id, address) of a zeroed host heap that the other processes of the job can reach.");
  m.def("dmem_initialised", [] { return !gd().nodes.empty(); });
  m.def("get_stats", [] { return gd().nodes.empty() ? dmem_stats_dict(DmemStats()) : dmem_stats_dict(self_mgr().stats()); });
  m.def("register_region", [](uintptr_t ptr, uint64_t n, uint32_t flags, uint32_t heap_id, uint64_t heap_offset) {
          if (heap_id != 0 && !(flags & REGION_DEVICE)) flags |= REGION_HOST_HEAP;
          return self_mgr().register_region(reinterpret_cast<void*>(ptr), n, flags, heap_id, heap_offset);
        },
        py::arg("ptr"), py::arg("nbytes"), py::arg("flags") = static_cast<uint32_t>(REGION_READABLE | REGION_WRITABLE | REGION_SHARED),
        py::arg("heap_id") = 0, py::arg("heap_offset") = 0);
  m.def("register_region_on",
        [](int node, uintptr_t ptr, uint64_t n) {
          MCCL_CHECK(node >= 0 && node < static_cast<int>(gd().nodes.size()), "no such in-process node");
          return gd().nodes[static_cast<size_t>(node)]->register_region(reinterpret_cast<void*>(ptr), n);
        },
        "Registers memory on behalf of an in-process peer node (single-process emulation of a cluster).");
  m.def("unregister_region", [](uint32_t id) { return self_mgr().unregister_region(id); });
  m.def("put", [](int node, uint32_t region, uint64_t off, uintptr_t src, uint64_t len) {
    return self_mgr().put(GlobalAddress(static_cast<uint16_t>(node), region, off), reinterpret_cast<const void*>(src), len, dmem_stream());
  });
  m.def("get", [](int node, uint32_t region, uint64_t off, uintptr_t dst, uint64_t len) {
    return self_mgr().get(reinterpret_cast<void*>(dst), GlobalAddress(static_cast<uint16_t>(node), region, off), len, dmem_stream());
  });
  m.def("put_with_imm", [](int node, uint32_t region, uint64_t off, uintptr_t src, uint64_t len, uint32_t imm) {
    return self_mgr().put_with_imm(GlobalAddress(static_cast<uint16_t>(node), region, off), reinterpret_cast<const void*>(src), len, imm,
                                   dmem_stream());
  });
  m.def("take_immediates", [] {
    // immediates that peers posted into this rank's rings (symmetric-heap fabric) join the local queue first
    if (gd().symm)
      for (auto& r : gd().symm->collect_imm()) self_mgr().push_immediate(r);
    if (gd().shm)
      for (auto& r : gd().shm->collect_imm()) self_mgr().push_immediate(r);
    py::list out;
    for (auto& r : self_mgr().take_immediates()) out.append(py::make_tuple(r.src_node, r.region_id, r.offset, r.length, r.imm));
    return out;
  }, "List of (source node, region, offset, length, immediate) delivered to this node since the last call.");
  m.def("dmem_fence", [] { self_mgr().fence(dmem_stream()); },
        "Orders every copy issued so far before later work on the current stream.");
  m.def("poll_completion", [](uint64_t wr) { return self_mgr().poll_completion(wr); });
  m.def("drain_pending", [] { return self_mgr().drain_pending(); });
  m.def("device_sync", [] {
    if (at::cuda::is_available()) cudaDeviceSynchronize();
  });
  m.attr("metal_sync") = m.attr("device_sync");  // name used by code written against the reference

  m.attr("REGION_READABLE") = static_cast<uint32_t>(REGION_READABLE);
  m.attr("REGION_WRITABLE") = static_cast<uint32_t>(REGION_WRITABLE);
  m.attr("REGION_SHARED") = static_cast<uint32_t>(REGION_SHARED);
  m.attr("REGION_PRIVATE") = static_cast<uint32_t>(REGION_PRIVATE);
  m.attr("REGION_DEVICE") = static_cast<uint32_t>(REGION_DEVICE);
  m.def("global_address_wire", [](int node, uint32_t region, uint64_t off) {
    uint8_t buf[GlobalAddress::kWireBytes];
    GlobalAddress g(static_cast<uint16_t>(node), region, off);
    g.to_wire(buf);
    GlobalAddress b = GlobalAddress::from_wire(buf);
    return py::make_tuple(py::bytes(reinterpret_cast<char*>(buf), sizeof(buf)), b.node_id, b.region_id, b.offset, g.pack());
  });

  // ------------------------------------------------------------- coherence --
  py::class_<CoherenceBus, std::shared_ptr<CoherenceBus>>(m, "CoherenceBus");
  py::class_<ShmBus, CoherenceBus, std::shared_ptr<ShmBus>>(m, "ShmBus")
      .def(py::init<std::shared_ptr<ShmFabric>>(), py::arg("fabric"), "Coherence mailboxes of the job in shared memory.");
  py::class_<LocalBus, CoherenceBus, std::shared_ptr<LocalBus>>(m, "LocalBus")
      .def(py::init<int>(), py::arg("num_nodes"))
      .def("drop_op", [](LocalBus& b, int op, int dst) {
        b.set_drop([op, dst](int d, const CoherenceMessage& msg) { return (op < 0 || msg.op == op) && (dst < 0 || d == dst); });
      }, py::arg("op"), py::arg("dst") = -1, "Test hook: drop messages with this opcode (-1 = any) sent to dst (-1 = anyone).")
      .def("drop_nothing", [](LocalBus& b) { b.set_drop(nullptr); });
  py::class_<CoherenceProtocol>(m, "CoherenceProtocol")
      .def(py::init([](int node, std::shared_ptr<CoherenceBus> bus, DistributedMemoryManager* d, int timeout_ms) {
             return new CoherenceProtocol(node, bus, d, timeout_ms);
           }),
           py::arg("node"), py::arg("bus"), py::arg("dmem"), py::arg("timeout_ms") = 5000, py::keep_alive<1, 3>(), py::keep_alive<1, 4>())
      .def("start", &CoherenceProtocol::start)
      .def("shutdown", &CoherenceProtocol::shutdown, py::call_guard<py::gil_scoped_release>())
      .def("acquire", &CoherenceProtocol::acquire, py::call_guard<py::gil_scoped_release>())
      .def("release", &CoherenceProtocol::release, py::call_guard<py::gil_scoped_release>())
      .def("fence", &CoherenceProtocol::fence, py::call_guard<py::gil_scoped_release>())
      .def("barrier_all", &CoherenceProtocol::barrier_all, py::call_guard<py::gil_scoped_release>())
      .def("read_page",
           [](CoherenceProtocol& c, int node, uint32_t region, uint64_t off, bool write) {
             void* p;
             {
               py::gil_scoped_release rel;
               p = c.read_page(GlobalAddress(static_cast<uint16_t>(node), region, off), write);
             }
             return reinterpret_cast<uintptr_t>(p);
           },
           py::arg("node"), py::arg("region"), py::arg("offset"), py::arg("write") = false)
      .def("write_page_done", [](CoherenceProtocol& c, int node, uint32_t region, uint64_t off) {
        c.write_page_done(GlobalAddress(static_cast<uint16_t>(node), region, off));
      })
      .def("local_state", [](CoherenceProtocol& c, int node, uint32_t region, uint64_t off) {
        return static_cast<int>(c.local_state(GlobalAddress(static_cast<uint16_t>(node), region, off)));
      })
      .def("directory_lookup", [](CoherenceProtocol& c, uint32_t region, uint64_t page) -> py::object {
        DirectoryEntry e;
        if (!c.directory_lookup(region, page, &e)) return py::none();
        return py::make_tuple(static_cast<int>(e.state), static_cast<int>(e.sharers), static_cast<int>(e.exclusive_owner), e.epoch);
      })
      .def("global_epoch", &CoherenceProtocol::global_epoch)
      .def("stats", [](CoherenceProtocol& c) {
        CoherenceStats s = c.stats();
        py::dict d;
        d["messages_sent"] = s.messages_sent;
        d["messages_handled"] = s.messages_handled;
        d["read_misses"] = s.read_misses;
        d["write_misses"] = s.write_misses;
        d["invalidations"] = s.invalidations;
        d["writebacks"] = s.writebacks;
        d["timeouts"] = s.timeouts;
        return d;
      });
  m.attr("COHERENCE_PAGE_SIZE") = COHERENCE_PAGE_SIZE;

  py::class_<GpuCoherence>(m, "GpuCoherence")
      .def(py::init<std::shared_ptr<DeviceComm>>(), py::call_guard<py::gil_scoped_release>())
      .def("gpu_release",
           [](GpuCoherence& g, int device) {
             return g.release(static_cast<void*>(at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream()));
           },
           py::arg("device"))
      .def("gpu_acquire",
           [](GpuCoherence& g, unsigned int epoch, int64_t timeout_ms, int device) {
             g.acquire(epoch, timeout_ms, static_cast<void*>(at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream()));
           },
           py::arg("epoch"), py::arg("timeout_ms") = 10000, py::arg("device") = 0)
      .def("status", &GpuCoherence::status)
      .def("clear_status", &GpuCoherence::clear_status)
      .def_property_readonly("epoch", &GpuCoherence::epoch);

  m.def("dmem_copy", [](uintptr_t dst, uintptr_t src, uint64_t n, int device) {
    c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
    cudaError_t rc = launch_dmem_copy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), n,
                                      at::cuda::getCurrentCUDAStream().stream());
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "dmem_copy failed: " << cudaGetErrorString(rc));
  }, py::arg("dst"), py::arg("src"), py::arg("nbytes"), py::arg("device") = 0, "SM-driven copy; either pointer may be a peer mapping.");
  m.def("dmem_atomic_selftest", [](at::Tensor counter, at::Tensor slot, at::Tensor sum, int adds) {
    c10::cuda::CUDAGuard g(counter.device());
    cudaError_t rc = launch_dmem_atomic_selftest(reinterpret_cast<unsigned int*>(counter.data_ptr()),
                                                 reinterpret_cast<unsigned long long*>(slot.data_ptr()), sum.data_ptr<float>(), adds,
                                                 at::cuda::getCurrentCUDAStream().stream());
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "dmem selftest failed: " << cudaGetErrorString(rc));
  });

  // ------------------------------------------------------- kernel dispatch --
  m.def("data_parallel_split", [](uint64_t total, int nodes) {
    py::list out;
    for (auto& w : KernelDispatch::data_parallel(total, nodes)) out.append(py::make_tuple(w.node, w.offset, w.count));
    return out;
  });
  m.def("pipeline_schedule", [](int stages, uint64_t micro_batches) {
    py::list out;
    for (auto& s : pipeline_schedule(stages, micro_batches)) out.append(py::make_tuple(s.time, s.stage, s.micro_batch));
    return out;
  });
}

}  // namespace mccl
