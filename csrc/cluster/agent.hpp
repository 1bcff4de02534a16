// Node agent: a small TCP server that answers the cluster manager's pings,
// keeps a table of registered regions and loaded kernels, runs kernel slices
// through a pluggable handler and reports counters.
//
// Parity: the reference's agent is a stand-alone binary with a thread per
// connection (csrc/agent/Agent.cpp:72-242) whose SHADER_RUN handler only
// acknowledges.  Here the same server is a class (so tests and `mccl status`
// can run one in-process) and a binary (csrc/agent/agent_main.cpp); KERNEL_RUN
// calls the handler the embedding process installs, which on a GPU rank
// launches its slice of a registered kernel.
#pragma once

#include <atomic>
#include <cstdint>
#include <functional>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "agent_protocol.hpp"

namespace mccl {

class AgentServer {
 public:
  // (kernel name, first element, element count) -> 0 on success
  using RunHandler = std::function<int(const std::string&, uint64_t, uint64_t)>;

  AgentServer();
  ~AgentServer();
  AgentServer(const AgentServer&) = delete;
  AgentServer& operator=(const AgentServer&) = delete;

  // Binds 127.0.0.1 or 0.0.0.0 (`any`) on `port` (0 = ephemeral) and starts serving.
  // Returns the bound port; throws TransportError on failure.
  int start(int port = 0, bool any = false);
  void stop();
  bool running() const { return running_.load(); }
  int port() const { return port_; }
  void set_run_handler(RunHandler h);
  // Test hook: stop answering (connections are accepted and dropped) to simulate a hung node.
  void set_unresponsive(bool v) { unresponsive_.store(v); }

  uint64_t pings() const { return pings_.load(); }
  uint64_t runs() const { return runs_.load(); }
  std::map<uint32_t, uint64_t> regions() const;

 private:
  void accept_loop();
  void serve(int fd);
  int lfd_ = -1, port_ = 0;
  std::atomic<bool> running_{false}, unresponsive_{false};
  std::thread acceptor_;
  std::mutex mu_;
  std::vector<std::thread> workers_;
  std::map<uint32_t, uint64_t> regions_;
  std::set<std::string> kernels_;
  RunHandler handler_;
  std::atomic<uint64_t> pings_{0}, runs_{0}, errors_{0}, requests_{0};
};

// Blocking client for one request/reply exchange per connection.
struct AgentReply {
  bool ok = false;               // transport-level success
  AgentStatus status = AgentStatus::ERROR;
  std::vector<uint8_t> payload;
  std::string error;
};
AgentReply agent_request(const std::string& host, int port, AgentCmd cmd, const std::vector<uint8_t>& payload, int timeout_ms);

}  // namespace mccl
