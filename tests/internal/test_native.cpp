// C++ unit tests without torch: FIFO progress engine, chunking, host collectives
// between threads over loopback TCP, host pool, metrics.
// Mirrors the reference's internal tests (tests/internal/test_progress.cpp: FIFO order of
// 100 tasks, destructor drains, idempotent shutdown, a throwing task does not poison the
// engine, submit stays fast while the engine is busy; tests/internal/test_ring_chunks.cpp:
// chunks cover the buffer exactly, are contiguous, wrap around the ring, numel < world).
#include <atomic>
#include <chrono>
#include <cmath>
#include <thread>

#include "../../csrc/engine/host_pool.hpp"
#include "../../csrc/engine/metrics.hpp"
#include "../../csrc/engine/progress.hpp"
#include "../../csrc/net/tcp_mesh.hpp"
#include "../../csrc/pg/cpu_algos.hpp"
#include "_test.h"

using namespace mccl;

TEST_CASE(progress_runs_tasks_in_submission_order) {
  Progress p;
  std::vector<int> seen;
  std::mutex mu;
  for (int i = 0; i < 100; ++i) p.submit([&, i] { std::lock_guard<std::mutex> g(mu); seen.push_back(i); });
  p.drain();
  CHECK(seen.size() == 100);
  for (int i = 0; i < 100; ++i) CHECK(seen[i] == i);
}

TEST_CASE(progress_destructor_drains_and_shutdown_is_idempotent) {
  std::atomic<int> ran{0};
  {
    Progress p;
    for (int i = 0; i < 20; ++i) p.submit([&] { std::this_thread::sleep_for(std::chrono::milliseconds(1)); ++ran; });
  }
  CHECK(ran == 20);
  Progress q;
  q.shutdown();
  q.shutdown();
  bool rejected = false;
  ProgressTask t;
  t.execute = [] {};
  t.on_error = [&](std::exception_ptr) { rejected = true; };
  CHECK(q.submit(std::move(t)) == 0 && rejected);
}

TEST_CASE(progress_exception_reaches_callback_and_engine_survives) {
  Progress p;
  bool got = false, later = false;
  ProgressTask t;
  t.execute = [] { throw std::runtime_error("boom"); };
  t.on_error = [&](std::exception_ptr e) { try { std::rethrow_exception(e); } catch (const std::runtime_error& x) { got = std::string(x.what()) == "boom"; } };
  p.submit(std::move(t));
  p.submit([&] { later = true; });
  p.drain();
  CHECK(got && later);
}

TEST_CASE(progress_submit_is_fast_while_busy_and_queue_is_bounded) {
  Progress p(4);
  std::atomic<bool> release{false};
  p.submit([&] { while (!release) std::this_thread::sleep_for(std::chrono::milliseconds(1)); });
  auto t0 = std::chrono::steady_clock::now();
  p.submit([] {});
  double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  CHECK(ms < 5.0);
  for (int i = 0; i < 3; ++i) p.submit([] {});
  CHECK(p.depth() == 4);
  std::thread blocked([&] { p.submit([] {}); });           // the fifth waits for space
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  CHECK(p.depth() == 4);
  release = true;
  blocked.join();
  p.drain();
  CHECK(p.completed() == 6);
}

TEST_CASE(chunks_cover_exactly_and_wrap) {
  for (size_t numel : {size_t(1), size_t(7), size_t(8), size_t(1000), size_t(1001)}) {
    for (int world : {1, 2, 3, 4, 8}) {
      Chunks ch(numel, world);
      size_t covered = 0;
      for (int i = 0; i < world; ++i) {
        CHECK(ch.offset(i) == covered || ch.len(i) == 0);
        covered += ch.len(i);
        CHECK(ch.len(i) <= ch.per);
      }
      CHECK(covered == numel);
    }
  }
  Chunks tiny(2, 4);      // numel < world: tail chunks are empty
  CHECK(tiny.len(0) == 1 && tiny.len(1) == 1 && tiny.len(2) == 0 && tiny.len(3) == 0);
  CHECK(resolve_cpu_algo(Algo::RING, 2, 8, 4, 262144) == Algo::TREE);
  CHECK(resolve_cpu_algo(Algo::AUTO, 1 << 20, 4 << 20, 4, 262144) == Algo::RING);
  CHECK(resolve_cpu_algo(Algo::AUTO, 65536, 262144, 4, 262144) == Algo::TREE);   // inclusive bound
}

TEST_CASE(bf16_and_fp16_conversions_round_to_nearest_even) {
  CHECK(f32_to_bf16_bits(1.0f) == 0x3f80);
  CHECK(bf16_bits_to_f32(f32_to_bf16_bits(3.14159f)) == 3.140625f);
  CHECK(f32_to_bf16_bits(1.00390625f) == 0x3f80);        // tie → even
  CHECK(f32_to_bf16_bits(1.01171875f) == 0x3f82);        // tie → even (up)
  CHECK(f16_bits_to_f32(f32_to_f16_bits(0.333251953125f)) == 0.333251953125f);
  CHECK(f32_to_f16_bits(65520.0f) == 0x7c00);            // overflows to inf
  CHECK(f16_bits_to_f32(0x0001) == std::ldexp(1.0f, -24));
  CHECK(f32_to_f16_bits(std::ldexp(1.0f, -24)) == 0x0001);
}

static void run_ranks(int world, const std::function<void(TcpMesh&, int)>& body) {
  MemoryKVStore store;
  EnvConfig cfg;
  std::vector<std::thread> ts;
  std::vector<std::string> errors(world);
  for (int r = 0; r < world; ++r)
    ts.emplace_back([&, r] {
      try {
        TcpMesh mesh(&store, r, world, 10000, "t", cfg);
        body(mesh, r);
      } catch (const std::exception& e) { errors[r] = e.what(); }
    });
  for (auto& t : ts) t.join();
  for (auto& e : errors) { if (!e.empty()) std::fprintf(stderr, "  rank error: %s\n", e.c_str()); CHECK(e.empty()); }
}

TEST_CASE(allreduce_schedules_agree_over_loopback) {
  for (int world : {2, 3, 4}) {
    for (Algo algo : {Algo::RING, Algo::TREE, Algo::BUTTERFLY}) {
      for (WireDtype wire : {WireDtype::NATIVE, WireDtype::BF16}) {
        run_ranks(world, [&](TcpMesh& mesh, int r) {
          const size_t n = 1003;
          std::vector<float> v(n);
          for (size_t i = 0; i < n; ++i) v[i] = static_cast<float>((i % 7) + r + 1);
          AllreduceArgs a;
          a.data = v.data(); a.numel = n; a.dtype = DType::F32; a.op = RedOp::AVG; a.wire = wire;
          allreduce(mesh, a, algo);
          for (size_t i = 0; i < n; ++i) {
            float want = 0;
            for (int q = 0; q < world; ++q) want += static_cast<float>((i % 7) + q + 1);
            want /= world;
            CHECK(std::fabs(v[i] - want) <= (wire == WireDtype::BF16 ? 0.05f : 1e-5f));
          }
        });
      }
    }
  }
}

TEST_CASE(other_collectives_over_loopback) {
  run_ranks(3, [&](TcpMesh& mesh, int r) {
    const int N = 3;
    std::vector<int32_t> mine(5, r + 1), all(15);
    allgather(mesh, mine.data(), all.data(), 5 * 4);
    for (int p = 0; p < N; ++p) for (int i = 0; i < 5; ++i) CHECK(all[p * 5 + i] == p + 1);
    std::vector<int32_t> in(6), out(2);
    for (int i = 0; i < 6; ++i) in[i] = (r + 1) * 10 + i;
    reduce_scatter(mesh, in.data(), out.data(), 2, DType::I32, RedOp::SUM);
    CHECK(out[0] == 60 + 3 * (2 * r) && out[1] == 60 + 3 * (2 * r + 1));
    std::vector<uint8_t> b(9, static_cast<uint8_t>(r == 2 ? 42 : 0));
    broadcast(mesh, b.data(), 9, 2);
    CHECK(b[0] == 42 && b[8] == 42);
    if (r == 0) { int x = 77; send_tagged(mesh, 1, &x, 4, 5); }
    if (r == 1) { int x = 0; recv_tagged(mesh, 0, &x, 4, -1); CHECK(x == 77); }
  });
}

TEST_CASE(closed_peer_surfaces_as_transport_error) {
  MemoryKVStore store;
  EnvConfig cfg;
  std::string err;
  std::thread a([&] { TcpMesh mesh(&store, 0, 2, 5000, "x", cfg); /* leaves at once: sockets close */ });
  std::thread b([&] {
    TcpMesh mesh(&store, 1, 2, 5000, "x", cfg);
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    char buf[8];
    try { mesh.recv(0, buf, 8); } catch (const TransportError& e) { err = e.what(); }
  });
  a.join();
  b.join();
  CHECK(!err.empty());
}

TEST_CASE(host_pool_reuses_best_fit_and_metrics_summarise) {
  HostPool pool;
  void* first;
  { PooledBuffer x = pool.acquire(1000); first = x.data(); CHECK(x.capacity() >= 1250); }
  { PooledBuffer y = pool.acquire(1100); CHECK(y.data() == first); }   // fits in the 25 % slack
  CHECK(pool.hits() == 1 && pool.misses() == 1);
  Metrics m;
  for (int i = 0; i < 10; ++i) { uint64_t s = m.op_start("allreduce", 1000, "ring"); m.record_phase(s, "network", 1.5); m.op_end(s); }
  uint64_t bad = m.op_start("broadcast", 10);
  m.op_end(bad, true);
  MetricsSummary sum = m.summarize();
  CHECK(sum.total_ops == 11 && sum.total_errors == 1 && sum.total_bytes == 10010);
  CHECK(std::fabs(sum.avg_network_ms - 15.0 / 11) < 1e-9 && sum.ops_by_name["allreduce"] == 10 && sum.bytes_by_algo["ring"] == 10000);
}

int main() { return run_all_tests(); }
