#include "tcp_mesh.hpp"

#include <arpa/inet.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <set>
#include <thread>

#include "../core/errors.hpp"
#include "../core/log.hpp"
#include "../core/version.hpp"

namespace mccl {

namespace {

using Clock = std::chrono::steady_clock;

constexpr uint32_t kHelloMagic = 0x4d43434cu;  // 'MCCL'

struct Hello {
  uint32_t magic;
  uint32_t protocol;
  int32_t rank;
};

int64_t ms_left(Clock::time_point deadline) {
  return std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
}

void set_nonblocking(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}

void tune_socket(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 16 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

// Full-length transfer on a non-blocking fd with an inactivity deadline.
void io_all(int fd, void* buf, size_t len, bool is_send, int64_t timeout_ms, int peer) {
  char* p = static_cast<char*>(buf);
  size_t done = 0;
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  while (done < len) {
    ssize_t n = is_send ? ::send(fd, p + done, len - done, MSG_NOSIGNAL) : ::recv(fd, p + done, len - done, 0);
    if (n > 0) {
      done += static_cast<size_t>(n);
      deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
      continue;
    }
    if (n == 0 && !is_send)
      MCCL_CHECK_T(false, TransportError, "tcp: peer " << peer << " closed the connection");
    if (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)
      MCCL_CHECK_T(false, TransportError,
                   "tcp: " << (is_send ? "send to" : "recv from") << " peer " << peer << " failed: "
                           << std::strerror(errno));
    int64_t left = ms_left(deadline);
    MCCL_CHECK_T(left > 0, TimeoutError,
                 "tcp: no progress " << (is_send ? "sending to" : "receiving from") << " peer " << peer
                                     << " for " << timeout_ms << " ms");
    pollfd pfd{fd, static_cast<short>(is_send ? POLLOUT : POLLIN), 0};
    ::poll(&pfd, 1, static_cast<int>(std::min<int64_t>(left, 1000)));
  }
}

bool has_prefix(const std::string& ip, const std::vector<std::string>& prefixes) {
  for (auto& p : prefixes)
    if (ip.compare(0, p.size(), p) == 0) return true;
  return false;
}

}  // namespace

std::vector<std::string> TcpMesh::local_ipv4(const EnvConfig& cfg) {
  std::vector<std::string> preferred, others, loop;
  ifaddrs* ifa = nullptr;
  if (getifaddrs(&ifa) == 0) {
    for (ifaddrs* it = ifa; it; it = it->ifa_next) {
      if (!it->ifa_addr || it->ifa_addr->sa_family != AF_INET) continue;
      if (!(it->ifa_flags & IFF_UP)) continue;
      if (!cfg.socket_ifname.empty() && cfg.socket_ifname != it->ifa_name) continue;
      char buf[INET_ADDRSTRLEN];
      auto* sin = reinterpret_cast<sockaddr_in*>(it->ifa_addr);
      inet_ntop(AF_INET, &sin->sin_addr, buf, sizeof(buf));
      std::string ip(buf);
      if (it->ifa_flags & IFF_LOOPBACK)
        loop.push_back(ip);
      else if (!cfg.iface_priority.empty() && has_prefix(ip, cfg.iface_priority))
        preferred.push_back(ip);
      else
        others.push_back(ip);
    }
    freeifaddrs(ifa);
  }
  std::vector<std::string> out = preferred;
  // A priority list is a hard filter for non-loopback addresses, as in the
  // reference (PeerMesh.cpp:213-236); loopback stays so one-box runs work.
  if (cfg.iface_priority.empty()) out.insert(out.end(), others.begin(), others.end());
  out.insert(out.end(), loop.begin(), loop.end());
  if (out.empty()) out.push_back("127.0.0.1");
  return out;
}

TcpMesh::TcpMesh(KVStore* store, int rank, int world, int64_t timeout_ms, const std::string& prefix,
                 const EnvConfig& cfg)
    : rank_(rank), world_(world), timeout_ms_(timeout_ms), fds_(world, -1), routes_(world) {
  for (int i = 0; i < world; ++i) io_mu_.emplace_back(new std::mutex());
  if (world <= 1) return;

  int lfd = ::socket(AF_INET, SOCK_STREAM, 0);
  MCCL_CHECK_T(lfd >= 0, TransportError, "tcp: socket() failed: " << std::strerror(errno));
  int one = 1;
  setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = 0;
  MCCL_CHECK_T(::bind(lfd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0, TransportError,
               "tcp: bind failed: " << std::strerror(errno));
  MCCL_CHECK_T(::listen(lfd, world) == 0, TransportError, "tcp: listen failed: " << std::strerror(errno));
  socklen_t alen = sizeof(addr);
  getsockname(lfd, reinterpret_cast<sockaddr*>(&addr), &alen);
  int port = ntohs(addr.sin_port);

  auto ips = local_ipv4(cfg);
  std::string mine;
  for (size_t i = 0; i < ips.size(); ++i) mine += (i ? "," : "") + ips[i];
  mine += ":" + std::to_string(port);
  Rendezvous rdv(store, rank, world, timeout_ms, prefix);
  auto endpoints = rdv.exchange_endpoints(mine, "peer");
  MCCL_INFO("tcp mesh: rank " << rank << " listening on " << mine);

  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  std::string accept_error;

  // Lower ranks connect to us; accept them on a helper thread while this
  // thread connects to the higher ranks.
  std::thread acceptor([&] {
    try {
      set_nonblocking(lfd);
      int need = rank;  // ranks 0..rank-1
      while (need > 0) {
        int64_t left = ms_left(deadline);
        MCCL_CHECK_T(left > 0, TimeoutError, "tcp: timed out waiting for " << need << " lower rank(s) to connect");
        pollfd pfd{lfd, POLLIN, 0};
        if (::poll(&pfd, 1, static_cast<int>(std::min<int64_t>(left, 200))) <= 0) continue;
        int fd = ::accept(lfd, nullptr, nullptr);
        if (fd < 0) continue;
        set_nonblocking(fd);
        tune_socket(fd);
        Hello in{};
        io_all(fd, &in, sizeof(in), false, std::max<int64_t>(left, 1), -1);
        MCCL_CHECK_T(in.magic == kHelloMagic && in.protocol == MCCL_PROTOCOL_VERSION, ProtocolError,
                     "tcp: bad handshake (magic " << in.magic << ", protocol " << in.protocol << ")");
        MCCL_CHECK_T(in.rank >= 0 && in.rank < rank && fds_[in.rank] < 0, ProtocolError,
                     "tcp: unexpected rank " << in.rank << " in handshake");
        Hello out{kHelloMagic, MCCL_PROTOCOL_VERSION, rank};
        io_all(fd, &out, sizeof(out), true, std::max<int64_t>(left, 1), in.rank);
        fds_[in.rank] = fd;
        routes_[in.rank] = "accepted";
        --need;
      }
    } catch (const std::exception& e) {
      accept_error = e.what();
    }
  });

  std::string connect_error;
  try {
    for (int p = rank + 1; p < world; ++p) {
      const std::string& ep = endpoints[p];
      size_t colon = ep.rfind(':');
      MCCL_CHECK_T(colon != std::string::npos, ProtocolError, "tcp: malformed endpoint '" << ep << "'");
      int pport = std::stoi(ep.substr(colon + 1));
      std::vector<std::string> cand;
      {
        std::string list = ep.substr(0, colon);
        size_t b = 0;
        while (b <= list.size()) {
          size_t e = list.find(',', b);
          if (e == std::string::npos) e = list.size();
          if (e > b) cand.push_back(list.substr(b, e - b));
          b = e + 1;
        }
      }
      // Prefer an address both sides own (same host → loopback or same NIC),
      // then the rest in the order the peer listed them.
      std::set<std::string> local(ips.begin(), ips.end());
      std::stable_sort(cand.begin(), cand.end(), [&](const std::string& a, const std::string& b) {
        return local.count(a) > local.count(b);
      });
      int fd = -1;
      while (fd < 0) {
        MCCL_CHECK_T(ms_left(deadline) > 0, TimeoutError,
                     "tcp: could not connect to rank " << p << " at " << ep << " within " << timeout_ms << " ms");
        for (auto& ip : cand) {
          int s = ::socket(AF_INET, SOCK_STREAM, 0);
          if (s < 0) continue;
          set_nonblocking(s);
          sockaddr_in pa{};
          pa.sin_family = AF_INET;
          pa.sin_port = htons(static_cast<uint16_t>(pport));
          if (inet_pton(AF_INET, ip.c_str(), &pa.sin_addr) != 1) {
            ::close(s);
            continue;
          }
          int rc = ::connect(s, reinterpret_cast<sockaddr*>(&pa), sizeof(pa));
          if (rc != 0 && errno == EINPROGRESS) {
            pollfd pfd{s, POLLOUT, 0};
            if (::poll(&pfd, 1, 1000) == 1) {
              int err = 0;
              socklen_t el = sizeof(err);
              getsockopt(s, SOL_SOCKET, SO_ERROR, &err, &el);
              rc = err == 0 ? 0 : -1;
            } else {
              rc = -1;
            }
          }
          if (rc == 0) {
            fd = s;
            routes_[p] = ip + ":" + std::to_string(pport);
            break;
          }
          ::close(s);
        }
        if (fd < 0) std::this_thread::sleep_for(std::chrono::milliseconds(50));
      }
      tune_socket(fd);
      Hello out{kHelloMagic, MCCL_PROTOCOL_VERSION, rank};
      io_all(fd, &out, sizeof(out), true, timeout_ms, p);
      Hello in{};
      io_all(fd, &in, sizeof(in), false, timeout_ms, p);
      MCCL_CHECK_T(in.magic == kHelloMagic && in.protocol == MCCL_PROTOCOL_VERSION && in.rank == p, ProtocolError,
                   "tcp: handshake with rank " << p << " answered by rank " << in.rank);
      fds_[p] = fd;
      MCCL_INFO("tcp mesh: rank " << rank << " -> rank " << p << " via " << routes_[p]);
    }
  } catch (const std::exception& e) {
    connect_error = e.what();
    deadline = Clock::now();  // let the acceptor give up promptly
  }
  acceptor.join();
  ::close(lfd);
  if (!connect_error.empty() || !accept_error.empty()) {
    close_all();
    MCCL_CHECK_T(false, TransportError,
                 "tcp mesh setup failed: " << (connect_error.empty() ? accept_error : connect_error));
  }
  closed_ = false;
}

TcpMesh::~TcpMesh() { close_all(); }

void TcpMesh::close_all() {
  for (auto& fd : fds_) {
    if (fd >= 0) {
      ::shutdown(fd, SHUT_RDWR);
      ::close(fd);
      fd = -1;
    }
  }
  closed_ = true;
}

int TcpMesh::fd_of(int peer) const {
  MCCL_CHECK_T(peer >= 0 && peer < world_ && peer != rank_, TransportError, "tcp: bad peer " << peer);
  int fd = fds_[peer];
  MCCL_CHECK_T(fd >= 0, TransportError, "tcp: connection to peer " << peer << " is closed");
  return fd;
}

void TcpMesh::send(int peer, const void* buf, size_t len) {
  int fd = fd_of(peer);
  std::lock_guard<std::mutex> g(*io_mu_[peer]);
  io_all(fd, const_cast<void*>(buf), len, true, timeout_ms_, peer);
  bytes_sent_ += len;
}

void TcpMesh::recv(int peer, void* buf, size_t len) {
  int fd = fd_of(peer);
  std::lock_guard<std::mutex> g(*io_mu_[peer]);
  io_all(fd, buf, len, false, timeout_ms_, peer);
  bytes_recv_ += len;
}

void TcpMesh::sendrecv(int to, const void* sbuf, size_t slen, int from, void* rbuf, size_t rlen) {
  std::vector<IoSpan> s, r;
  if (slen) s.push_back({to, const_cast<void*>(sbuf), slen});
  if (rlen) r.push_back({from, rbuf, rlen});
  exchange(s, r);
}

void TcpMesh::exchange(const std::vector<IoSpan>& sends, const std::vector<IoSpan>& recvs) {
  struct Lane {
    std::vector<IoSpan> q;  // in order
    size_t idx = 0, off = 0;
    bool done() const { return idx >= q.size(); }
  };
  std::vector<Lane> tx(world_), rx(world_);
  std::set<int> peers;
  for (auto& s : sends)
    if (s.len) {
      fd_of(s.peer);
      tx[s.peer].q.push_back(s);
      peers.insert(s.peer);
    }
  for (auto& r : recvs)
    if (r.len) {
      fd_of(r.peer);
      rx[r.peer].q.push_back(r);
      peers.insert(r.peer);
    }
  if (peers.empty()) return;
  std::vector<std::unique_lock<std::mutex>> locks;
  for (int p : peers) locks.emplace_back(*io_mu_[p]);  // std::set iterates in rank order

  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms_);
  std::vector<pollfd> pfds;
  std::vector<int> pfd_peer;
  for (;;) {
    pfds.clear();
    pfd_peer.clear();
    for (int p : peers) {
      short ev = 0;
      if (!tx[p].done()) ev |= POLLOUT;
      if (!rx[p].done()) ev |= POLLIN;
      if (ev) {
        pfds.push_back({fds_[p], ev, 0});
        pfd_peer.push_back(p);
      }
    }
    if (pfds.empty()) break;
    int64_t left = ms_left(deadline);
    MCCL_CHECK_T(left > 0, TimeoutError, "tcp: exchange made no progress for " << timeout_ms_ << " ms");
    int n = ::poll(pfds.data(), pfds.size(), static_cast<int>(std::min<int64_t>(left, 1000)));
    if (n <= 0) continue;
    bool progressed = false;
    for (size_t i = 0; i < pfds.size(); ++i) {
      int p = pfd_peer[i];
      if (pfds[i].revents & (POLLOUT | POLLERR | POLLHUP)) {
        Lane& l = tx[p];
        while (!l.done()) {
          IoSpan& sp = l.q[l.idx];
          ssize_t k = ::send(pfds[i].fd, static_cast<char*>(sp.ptr) + l.off, sp.len - l.off, MSG_NOSIGNAL);
          if (k > 0) {
            l.off += static_cast<size_t>(k);
            bytes_sent_ += static_cast<uint64_t>(k);
            progressed = true;
            if (l.off == sp.len) {
              ++l.idx;
              l.off = 0;
            }
          } else if (k < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) {
            break;
          } else {
            MCCL_CHECK_T(false, TransportError, "tcp: send to peer " << p << " failed: " << std::strerror(errno));
          }
        }
      }
      if (pfds[i].revents & (POLLIN | POLLERR | POLLHUP)) {
        Lane& l = rx[p];
        while (!l.done()) {
          IoSpan& sp = l.q[l.idx];
          ssize_t k = ::recv(pfds[i].fd, static_cast<char*>(sp.ptr) + l.off, sp.len - l.off, 0);
          if (k > 0) {
            l.off += static_cast<size_t>(k);
            bytes_recv_ += static_cast<uint64_t>(k);
            progressed = true;
            if (l.off == sp.len) {
              ++l.idx;
              l.off = 0;
            }
          } else if (k == 0) {
            MCCL_CHECK_T(false, TransportError, "tcp: peer " << p << " closed the connection");
          } else if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) {
            break;
          } else {
            MCCL_CHECK_T(false, TransportError, "tcp: recv from peer " << p << " failed: " << std::strerror(errno));
          }
        }
      }
    }
    if (progressed) deadline = Clock::now() + std::chrono::milliseconds(timeout_ms_);
  }
}

}  // namespace mccl
