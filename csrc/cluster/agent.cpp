#include "agent.hpp"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>

#include "../core/errors.hpp"
#include "../core/log.hpp"

namespace mccl {

namespace {

bool io_full(int fd, void* buf, size_t len, bool is_send, int timeout_ms) {
  char* p = static_cast<char*>(buf);
  size_t done = 0;
  while (done < len) {
    pollfd pfd{fd, static_cast<short>(is_send ? POLLOUT : POLLIN), 0};
    int rc = ::poll(&pfd, 1, timeout_ms);
    if (rc <= 0) return false;
    ssize_t n = is_send ? ::send(fd, p + done, len - done, MSG_NOSIGNAL) : ::recv(fd, p + done, len - done, 0);
    if (n <= 0) return false;
    done += static_cast<size_t>(n);
  }
  return true;
}

bool send_frame(int fd, uint16_t cmd, uint16_t status, const std::vector<uint8_t>& payload, int timeout_ms) {
  AgentHeader h{cmd, status, static_cast<uint32_t>(payload.size())};
  if (!io_full(fd, &h, sizeof(h), true, timeout_ms)) return false;
  return payload.empty() || io_full(fd, const_cast<uint8_t*>(payload.data()), payload.size(), true, timeout_ms);
}

}  // namespace

AgentServer::AgentServer() = default;
AgentServer::~AgentServer() { stop(); }

void AgentServer::set_run_handler(RunHandler h) {
  std::lock_guard<std::mutex> g(mu_);
  handler_ = std::move(h);
}

std::map<uint32_t, uint64_t> AgentServer::regions() const {
  std::lock_guard<std::mutex> g(const_cast<std::mutex&>(mu_));
  return regions_;
}

int AgentServer::start(int port, bool any) {
  MCCL_CHECK(!running_, "agent already running");
  lfd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  MCCL_CHECK_T(lfd_ >= 0, TransportError, "agent: socket() failed: " << std::strerror(errno));
  int one = 1;
  setsockopt(lfd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(any ? INADDR_ANY : INADDR_LOOPBACK);
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (::bind(lfd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(lfd_, 64) != 0) {
    std::string why = std::strerror(errno);
    ::close(lfd_);
    lfd_ = -1;
    MCCL_CHECK_T(false, TransportError, "agent: cannot listen on port " << port << ": " << why);
  }
  socklen_t alen = sizeof(addr);
  getsockname(lfd_, reinterpret_cast<sockaddr*>(&addr), &alen);
  port_ = ntohs(addr.sin_port);
  running_ = true;
  acceptor_ = std::thread([this] { accept_loop(); });
  return port_;
}

void AgentServer::stop() {
  if (!running_.exchange(false)) {
    if (acceptor_.joinable()) acceptor_.join();
    return;
  }
  if (acceptor_.joinable()) acceptor_.join();
  if (lfd_ >= 0) ::close(lfd_);
  lfd_ = -1;
  std::vector<std::thread> ws;
  {
    std::lock_guard<std::mutex> g(mu_);
    ws.swap(workers_);
  }
  for (auto& t : ws)
    if (t.joinable()) t.join();
}

void AgentServer::accept_loop() {
  while (running_) {
    pollfd pfd{lfd_, POLLIN, 0};
    if (::poll(&pfd, 1, 100) <= 0) continue;
    int fd = ::accept(lfd_, nullptr, nullptr);
    if (fd < 0) continue;
    if (unresponsive_) {  // simulated hang: take the connection, never answer
      std::lock_guard<std::mutex> g(mu_);
      workers_.emplace_back([this, fd] {
        while (running_ && unresponsive_) ::usleep(20000);
        ::close(fd);
      });
      continue;
    }
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    std::lock_guard<std::mutex> g(mu_);
    workers_.emplace_back([this, fd] { serve(fd); });
  }
}

void AgentServer::serve(int fd) {
  while (running_) {
    AgentHeader h{};
    if (!io_full(fd, &h, sizeof(h), false, 500)) break;
    if (h.payload_len > kAgentMaxPayload) break;
    std::vector<uint8_t> in(h.payload_len);
    if (h.payload_len && !io_full(fd, in.data(), in.size(), false, 2000)) break;
    ++requests_;
    std::vector<uint8_t> out;
    AgentStatus st = AgentStatus::OK;
    bool shutdown = false;
    switch (static_cast<AgentCmd>(h.cmd)) {
      case AgentCmd::PING: ++pings_; break;
      case AgentCmd::REGISTER:
        if (in.size() >= 12) {
          std::lock_guard<std::mutex> g(mu_);
          regions_[get_u32(in.data())] = get_u64(in.data() + 4);
        } else st = AgentStatus::ERROR;
        break;
      case AgentCmd::DEREGISTER:
        if (in.size() >= 4) {
          std::lock_guard<std::mutex> g(mu_);
          st = regions_.erase(get_u32(in.data())) ? AgentStatus::OK : AgentStatus::NOT_FOUND;
        } else st = AgentStatus::ERROR;
        break;
      case AgentCmd::KERNEL_LOAD: {
        std::lock_guard<std::mutex> g(mu_);
        kernels_.insert(std::string(in.begin(), in.end()));
        break;
      }
      case AgentCmd::KERNEL_RUN: {
        if (in.size() < 2 || in.size() < 2u + get_u16(in.data()) + 16u) { st = AgentStatus::ERROR; break; }
        const uint16_t nl = get_u16(in.data());
        std::string name(in.begin() + 2, in.begin() + 2 + nl);
        const uint64_t off = get_u64(in.data() + 2 + nl), cnt = get_u64(in.data() + 10 + nl);
        RunHandler hnd;
        bool known;
        {
          std::lock_guard<std::mutex> g(mu_);
          hnd = handler_;
          known = kernels_.count(name) != 0;
        }
        if (!known) { st = AgentStatus::NOT_FOUND; break; }
        ++runs_;
        if (hnd && hnd(name, off, cnt) != 0) st = AgentStatus::ERROR;
        break;
      }
      case AgentCmd::KERNEL_SYNC: break;
      case AgentCmd::STATS: {
        std::string s = "requests=" + std::to_string(requests_.load()) + "\npings=" + std::to_string(pings_.load()) +
                        "\nruns=" + std::to_string(runs_.load()) + "\nerrors=" + std::to_string(errors_.load()) + "\n";
        {
          std::lock_guard<std::mutex> g(mu_);
          s += "regions=" + std::to_string(regions_.size()) + "\nkernels=" + std::to_string(kernels_.size()) + "\n";
        }
        out.assign(s.begin(), s.end());
        break;
      }
      case AgentCmd::SHUTDOWN: shutdown = true; break;
      default: st = AgentStatus::UNKNOWN_COMMAND; break;
    }
    if (st != AgentStatus::OK) ++errors_;
    if (!send_frame(fd, h.cmd, static_cast<uint16_t>(st), out, 2000)) break;
    if (shutdown) {
      running_ = false;
      break;
    }
  }
  ::close(fd);
}

AgentReply agent_request(const std::string& host, int port, AgentCmd cmd, const std::vector<uint8_t>& payload, int timeout_ms) {
  AgentReply r;
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) { r.error = "socket() failed"; return r; }
  timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) { ::close(fd); r.error = "bad address " + host; return r; }
  if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0) {
    r.error = std::string("connect failed: ") + std::strerror(errno);
    ::close(fd);
    return r;
  }
  if (!send_frame(fd, static_cast<uint16_t>(cmd), 0, payload, timeout_ms)) { ::close(fd); r.error = "send failed"; return r; }
  AgentHeader h{};
  if (!io_full(fd, &h, sizeof(h), false, timeout_ms) || h.payload_len > kAgentMaxPayload) { ::close(fd); r.error = "no reply within timeout"; return r; }
  r.payload.resize(h.payload_len);
  if (h.payload_len && !io_full(fd, r.payload.data(), r.payload.size(), false, timeout_ms)) { ::close(fd); r.error = "short reply"; return r; }
  ::close(fd);
  r.ok = true;
  r.status = static_cast<AgentStatus>(h.status);
  return r;
}

}  // namespace mccl
