// C++ unit tests without torch for the threaded parts of the runtime: distributed memory over the
// in-process fabric, the coherence protocol with one service thread per node, the scheduler and the
// cluster manager's heartbeat bookkeeping.  The program exists so that the host code can run under
// ThreadSanitizer / AddressSanitizer (tests/test_sanitizers.py): every test drives the component from
// several threads at once.  The reference documents its own data-race handling for the overlapped
// receive / reduce buffers at csrc/backend/AllreduceAlgos.hpp:13-16; there is no sanitizer job in it.
#include <atomic>
#include <chrono>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#include "../../csrc/cluster/cluster_manager.hpp"
#include "../../csrc/cluster/scheduler.hpp"
#include "../../csrc/coherence/coherence.hpp"
#include "../../csrc/dmem/dmem_manager.hpp"
#include "_test.h"

using namespace mccl;

TEST_CASE(dmem_concurrent_puts_and_gets_between_in_process_nodes) {
  const int N = 4;
  auto fabric = std::make_shared<LocalFabric>(N);
  std::vector<std::unique_ptr<DistributedMemoryManager>> nodes;
  for (int i = 0; i < N; ++i) nodes.emplace_back(new DistributedMemoryManager(static_cast<uint16_t>(i), fabric));
  std::vector<std::vector<uint8_t>> mem(N, std::vector<uint8_t>(N * 4096, 0));
  std::vector<uint32_t> region(N);
  for (int i = 0; i < N; ++i) region[i] = nodes[i]->register_region(mem[i].data(), mem[i].size());
  // every node writes its slot of every other node's region, all at once
  std::vector<std::thread> ts;
  for (int i = 0; i < N; ++i)
    ts.emplace_back([&, i] {
      std::vector<uint8_t> src(4096, static_cast<uint8_t>(i + 1));
      for (int rep = 0; rep < 20; ++rep)
        for (int p = 0; p < N; ++p) {
          if (p == i) continue;
          uint64_t wr = nodes[i]->put_with_imm(GlobalAddress(static_cast<uint16_t>(p), region[p], static_cast<uint64_t>(i) * 4096), src.data(),
                                               src.size(), static_cast<uint32_t>(100 * i + rep));
          CHECK(wr > 0 && nodes[i]->poll_completion(wr));
        }
    });
  for (auto& t : ts) t.join();
  for (int p = 0; p < N; ++p) {
    for (int i = 0; i < N; ++i)
      if (i != p) CHECK(mem[p][static_cast<size_t>(i) * 4096] == i + 1 && mem[p][static_cast<size_t>(i) * 4096 + 4095] == i + 1);
    CHECK(nodes[p]->take_immediates().size() == static_cast<size_t>(20 * (N - 1)));
  }
  // concurrent readers of one region
  ts.clear();
  std::atomic<int> good{0};
  for (int i = 1; i < N; ++i)
    ts.emplace_back([&, i] {
      std::vector<uint8_t> dst(4096);
      for (int rep = 0; rep < 50; ++rep) {
        uint64_t wr = nodes[i]->get(dst.data(), GlobalAddress(0, region[0], 4096), 4096);
        if (wr > 0 && dst[0] == 2 && dst[4095] == 2) ++good;
      }
    });
  for (auto& t : ts) t.join();
  CHECK(good == 50 * (N - 1));
  CHECK(nodes[0]->stats().total_put_ops == static_cast<uint64_t>(20 * (N - 1)));
}

TEST_CASE(coherence_three_nodes_contend_for_pages_from_threads) {
  const int N = 3;
  auto fabric = std::make_shared<LocalFabric>(N);
  auto bus = std::make_shared<LocalBus>(N);
  std::vector<std::unique_ptr<DistributedMemoryManager>> dm;
  std::vector<std::unique_ptr<CoherenceProtocol>> co;
  for (int i = 0; i < N; ++i) dm.emplace_back(new DistributedMemoryManager(static_cast<uint16_t>(i), fabric));
  for (int i = 0; i < N; ++i) co.emplace_back(new CoherenceProtocol(i, bus, dm[i].get(), 5000));
  for (auto& c : co) c->start();
  const uint64_t page = COHERENCE_PAGE_SIZE;
  std::vector<uint8_t> home(4 * page, 0);
  const uint32_t rid = dm[0]->register_region(home.data(), home.size());
  // nodes 1 and 2 take turns writing "their" counter byte on pages they both touch; the home reads.
  std::vector<std::thread> ts;
  for (int n = 1; n < N; ++n)
    ts.emplace_back([&, n] {
      for (int rep = 0; rep < 30; ++rep) {
        for (uint64_t pg = 0; pg < 4; ++pg) {
          GlobalAddress g(0, rid, pg * page + static_cast<uint64_t>(n));
          uint8_t* w = static_cast<uint8_t*>(co[n]->read_page(g, /*write=*/true));   // start of the cached page
          w[n] = static_cast<uint8_t>(w[n] + 1);
          co[n]->write_page_done(g);
        }
        co[n]->release();
      }
    });
  ts.emplace_back([&] {
    for (int rep = 0; rep < 30; ++rep) {
      co[0]->acquire();
      for (uint64_t pg = 0; pg < 4; ++pg) (void)co[0]->read_page(GlobalAddress(0, rid, pg * page), false);
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
  });
  for (auto& t : ts) t.join();
  for (auto& c : co) c->fence();
  for (uint64_t pg = 0; pg < 4; ++pg) {
    (void)co[0]->read_page(GlobalAddress(0, rid, pg * page), false);   // pulls any dirty copy home
    CHECK(home[pg * page + 1] == 30 && home[pg * page + 2] == 30);
  }
  std::vector<std::thread> bs;
  for (auto& c : co) bs.emplace_back([&c] { c->barrier_all(); });
  for (auto& t : bs) t.join();
  for (auto& c : co) c->shutdown();
}

TEST_CASE(scheduler_is_safe_under_concurrent_submit_tick_cancel) {
  Scheduler s;
  std::atomic<bool> stop{false};
  std::vector<std::thread> ts;
  std::vector<uint64_t> ids[3];
  for (int t = 0; t < 3; ++t)
    ts.emplace_back([&, t] {
      for (int i = 0; i < 200; ++i) {
        JobSpec spec;
        spec.name = "job";
        spec.tenant = "tenant" + std::to_string(t);
        spec.priority = static_cast<JobPriority>(i % 4);
        spec.nodes_required = 1 + i % 2;
        ids[t].push_back(s.submit(spec));
        if (i % 7 == 0) s.cancel(ids[t][static_cast<size_t>(i / 2)]);
      }
    });
  std::thread ticker([&] {
    std::vector<NodeLoad> loads(4);
    for (int n = 0; n < 4; ++n) {
      loads[n].node_id = n;
      loads[n].online = true;
      loads[n].memory_total = 1 << 30;
    }
    while (!stop) {
      TickResult r = s.schedule_tick(loads);
      for (auto& p : r.started) s.complete(p.job_id, true, "");
    }
  });
  for (auto& t : ts) t.join();
  stop = true;
  ticker.join();
  CHECK(s.jobs().size() == 600);
}

TEST_CASE(cluster_manager_heartbeats_from_threads_and_eviction) {
  ClusterTimings t;
  t.heartbeat_interval_ms = 10;
  t.heartbeat_timeout_ms = 80;
  t.scheduler_tick_ms = 20;
  ClusterManager cm(0, t);
  std::atomic<int> failed_node{-1};
  cm.on_failure([&](int n) { failed_node = n; });
  for (int n = 0; n < 4; ++n) {
    NodeInfo info;
    info.node_id = n;
    info.agent_port = 1;   // nobody listens there: pings are refused at once, liveness comes from the heartbeats below
    info.memory_total = 1ull << 30;
    CHECK(cm.handle_join(info));
  }
  cm.start();
  std::atomic<bool> stop{false};
  std::vector<std::thread> beats;
  for (int n = 0; n < 3; ++n)   // node 3 never reports
    beats.emplace_back([&, n] {
      while (!stop) {
        cm.handle_heartbeat(n, 1000 + n);
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
      }
    });
  std::thread reader([&] {
    while (!stop) {
      (void)cm.nodes();
      (void)cm.leader();
      (void)cm.online_count();
    }
  });
  for (int i = 0; i < 100 && failed_node.load() != 3; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
  stop = true;
  for (auto& th : beats) th.join();
  reader.join();
  cm.stop();
  CHECK(failed_node.load() == 3);
  CHECK(cm.leader() == 0);
  int online = 0;
  for (auto& n : cm.nodes()) online += n.status == NodeStatus::ONLINE ? 1 : 0;
  CHECK(online >= 1 && online <= 3);
}

int main() { return run_all_tests(); }
