// Environment-driven configuration.
//
// Parity: the reference reads MCCL_ALLREDUCE_ALGO, MCCL_TREE_BELOW and
// MCCL_WIRE_DTYPE with getenv on every allreduce call so a script can flip
// them between calls (csrc/backend/ProcessGroupMCCL.cpp:117-141), and reads
// MCCL_IFACE_PRIORITY once (csrc/backend/PeerMesh.cpp:23-39).  EnvConfig is
// the once-per-process-group snapshot; the three per-call knobs have their
// own readers below.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace mccl {

enum class Algo : int { AUTO = 0, RING, TREE, BUTTERFLY /* = two-shot */, ONESHOT, NVLS, BUTTERFLY_PUSH /* two-shot, gather half pushed */ };
enum class WireDtype : int { NATIVE = 0, BF16 };

inline const char* algo_name(Algo a) {
  switch (a) {
    case Algo::AUTO: return "auto";
    case Algo::RING: return "ring";
    case Algo::TREE: return "tree";
    case Algo::BUTTERFLY: return "butterfly";
    case Algo::ONESHOT: return "oneshot";
    case Algo::NVLS: return "nvls";
    case Algo::BUTTERFLY_PUSH: return "twoshot_push";
  }
  return "?";
}

namespace env {

inline std::string str(const char* name, const char* dflt = "") {
  const char* v = std::getenv(name);
  return v ? std::string(v) : std::string(dflt);
}
inline int64_t i64(const char* name, int64_t dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  long long x = std::strtoll(v, &end, 10);
  return end == v ? dflt : static_cast<int64_t>(x);
}
inline bool flag(const char* name, bool dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  return !(strcmp(v, "0") == 0 || strcasecmp(v, "false") == 0 || strcasecmp(v, "no") == 0 ||
           strcasecmp(v, "off") == 0);
}
inline std::vector<std::string> csv(const char* name) {
  std::vector<std::string> out;
  std::string s = str(name);
  size_t b = 0;
  while (b <= s.size()) {
    size_t e = s.find(',', b);
    if (e == std::string::npos) e = s.size();
    if (e > b) out.push_back(s.substr(b, e - b));
    b = e + 1;
  }
  return out;
}

}  // namespace env

// Per-call knob: which allreduce algorithm the user asked for.  Any string
// that is not a known name selects TREE, as the reference does
// (ProcessGroupMCCL.cpp:174-176); unset or empty means AUTO.
inline Algo requested_algo() {
  std::string s = env::str("MCCL_ALLREDUCE_ALGO", "auto");
  if (s.empty() || s == "auto") return Algo::AUTO;
  if (s == "ring") return Algo::RING;
  if (s == "tree") return Algo::TREE;
  if (s == "butterfly" || s == "twoshot") return Algo::BUTTERFLY;
  if (s == "oneshot") return Algo::ONESHOT;
  if (s == "nvls") return Algo::NVLS;
  if (s == "twoshot_push" || s == "butterfly_push") return Algo::BUTTERFLY_PUSH;
  return Algo::TREE;
}

// Per-call knob: messages of at most this many bytes take the latency path
// under AUTO (inclusive bound, default 262144 as in ProcessGroupMCCL.cpp:138-141).
inline int64_t tree_below_bytes() { return env::i64("MCCL_TREE_BELOW", 262144); }
// The same bound for CUDA tensors, where it separates the one-shot from the two-shot schedule.  Measured on
// 8 x B200 the one-shot kernel wins up to 1 MiB on the wire (26 us against 37 us at 1 MiB, 41 against 39 at
// 2 MiB), so that is the default when MCCL_TREE_BELOW is not set.
inline int64_t device_oneshot_below_bytes() { return env::i64("MCCL_TREE_BELOW", 1048576); }

// Per-call knob: bf16 on the wire for fp32 tensors.
inline WireDtype requested_wire() {
  return env::str("MCCL_WIRE_DTYPE") == "bf16" ? WireDtype::BF16 : WireDtype::NATIVE;
}

struct EnvConfig {
  std::vector<std::string> iface_priority;  // IPv4 prefixes, empty = accept all
  std::string socket_ifname;                // restrict to one interface name
  int64_t arena_bytes = 0;                  // symmetric staging arena per rank
  int64_t device_timeout_ms = 0;            // bound of every device-side wait; 0 = derive from the group's timeout
  int64_t device_timeout_cap_ms = 0;        // upper bound of the derived value
  int nvls = -1;                            // -1 auto, 0 off, 1 required
  bool blocking_wait = false;               // Work::wait blocks the host
  bool debug_bounds = false;                // kernels check their arena extent; poison fill and canaries (MCCL_DEBUG_BOUNDS)
  int max_queue_depth = 1024;               // bounded progress queue
  std::string symm_mode;                    // "auto" | "vmm" | "ipc"
  std::string fault_inject;                 // host-made faults: "rank=R,skip_signals=N,after=K,delay_ms=M" (MCCL_FAULT_INJECT)
  std::string trace_path;                   // JSON-lines trace file, empty = off
  int max_ctas = 0;                         // cap on CTAs per collective, 0 = default

  static EnvConfig from_env() {
    EnvConfig c;
    c.iface_priority = env::csv("MCCL_IFACE_PRIORITY");
    c.socket_ifname = env::str("MCCL_SOCKET_IFNAME");
    c.arena_bytes = env::i64("MCCL_ARENA_MB", 512) << 20;
    // Unset: the device limit follows the timeout the process group was created with (capped by
    // MCCL_DEVICE_TIMEOUT_CAP_MS, five minutes by default), so ordinary rank skew - a checkpoint or an
    // evaluation on one rank, a data stall - does not end a collective that c10d would still wait for.
    c.device_timeout_ms = env::i64("MCCL_DEVICE_TIMEOUT_MS", 0);
    c.device_timeout_cap_ms = env::i64("MCCL_DEVICE_TIMEOUT_CAP_MS", 300000);
    std::string n = env::str("MCCL_NVLS", "auto");
    c.nvls = (n == "auto" || n.empty()) ? -1 : (env::flag("MCCL_NVLS", true) ? 1 : 0);
    c.blocking_wait = env::flag("MCCL_BLOCKING_WAIT", false);
    c.debug_bounds = env::flag("MCCL_DEBUG_BOUNDS", false);
    c.max_queue_depth = static_cast<int>(
        env::i64("MCCL_MAX_QUEUE_DEPTH", env::i64("DISTRO_MAX_QUEUE_DEPTH", 1024)));
    c.symm_mode = env::str("MCCL_SYMM_MODE", "auto");
    c.fault_inject = env::str("MCCL_FAULT_INJECT");
    c.trace_path = env::str("MCCL_TRACE");
    c.max_ctas = static_cast<int>(env::i64("MCCL_MAX_CTAS", 0));
    return c;
  }
};

}  // namespace mccl
