// Full-mesh TCP transport between the ranks of one process group.
//
// Role: data plane for CPU tensors and bootstrap channel for everything else.
// Parity: the reference's PeerMesh (csrc/backend/PeerMesh.cpp:109-301) opens
// one socket per peer, lower rank connecting to higher, publishes
// "ip,ip:port" under mccl/peer/<rank> in the c10d store, and filters candidate
// addresses by MCCL_IFACE_PRIORITY prefixes.  Differences chosen for Linux
// hosts: loopback is a legal route (single-box runs use 127.0.0.1), the
// prefix filter only applies when the variable is set, sockets are
// non-blocking and every transfer is a poll() loop with a deadline, and a
// scatter/gather `exchange` moves data with many peers at once from a single
// thread instead of spawning a thread per peer per step.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../core/config.hpp"
#include "kv_store.hpp"

namespace mccl {

struct IoSpan {
  int peer = -1;
  void* ptr = nullptr;       // send spans are only read
  size_t len = 0;
};

class TcpMesh {
 public:
  TcpMesh(KVStore* store, int rank, int world, int64_t timeout_ms, const std::string& prefix,
          const EnvConfig& cfg);
  ~TcpMesh();
  TcpMesh(const TcpMesh&) = delete;
  TcpMesh& operator=(const TcpMesh&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }

  // Blocking, full-length.  Throw TransportError on EOF/reset and
  // TimeoutError when no byte moves for timeout_ms.
  void send(int peer, const void* buf, size_t len);
  void recv(int peer, void* buf, size_t len);

  // Runs all sends and receives concurrently until every span is complete.
  // Spans for the same peer and direction are processed in list order.
  void exchange(const std::vector<IoSpan>& sends, const std::vector<IoSpan>& recvs);

  // Convenience: one send and one receive (possibly different peers).
  void sendrecv(int to, const void* sbuf, size_t slen, int from, void* rbuf, size_t rlen);

  // Closes every socket; later calls throw TransportError.  Used by abort().
  void close_all();

  // Route chosen for a peer ("ip:port"), for logs and `mccl status`.
  const std::string& route(int peer) const { return routes_[peer]; }

  uint64_t bytes_sent() const { return bytes_sent_; }
  uint64_t bytes_received() const { return bytes_recv_; }

  // Local IPv4 addresses that pass the interface filters (loopback last).
  static std::vector<std::string> local_ipv4(const EnvConfig& cfg);

 private:
  int fd_of(int peer) const;
  int rank_, world_;
  int64_t timeout_ms_;
  std::vector<int> fds_;
  std::vector<std::string> routes_;
  std::vector<std::unique_ptr<std::mutex>> io_mu_;  // one per peer; exchange takes all it needs in rank order
  uint64_t bytes_sent_ = 0, bytes_recv_ = 0;
  bool closed_ = false;
};

}  // namespace mccl
