// Leveled stderr logger.
//
// Parity: the reference has seven levels chosen by DISTRO_LOG_LEVEL (a name
// or a digit), defaults to WARN and serialises lines with a mutex
// (csrc/common/Logging.hpp:22-102).  Here MCCL_LOG_LEVEL is the primary name,
// DISTRO_LOG_LEVEL an alias, and each line carries the process rank.
#pragma once

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <mutex>
#include <sstream>
#include <string>

namespace mccl {

enum class LogLevel : int { TRACE = 0, DEBUG = 1, INFO = 2, WARN = 3, ERROR = 4, FATAL = 5, OFF = 6 };

namespace logdetail {

inline LogLevel parse_level(const char* s, LogLevel dflt) {
  if (!s || !*s) return dflt;
  if (s[0] >= '0' && s[0] <= '6' && s[1] == 0) return static_cast<LogLevel>(s[0] - '0');
  static const char* names[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR", "FATAL", "OFF"};
  for (int i = 0; i < 7; ++i)
    if (strcasecmp(s, names[i]) == 0) return static_cast<LogLevel>(i);
  return dflt;
}

inline std::atomic<int>& level_cell() {
  static std::atomic<int> cell{[] {
    const char* s = std::getenv("MCCL_LOG_LEVEL");
    if (!s) s = std::getenv("DISTRO_LOG_LEVEL");
    return static_cast<int>(parse_level(s, LogLevel::WARN));
  }()};
  return cell;
}

inline std::atomic<int>& rank_cell() {
  static std::atomic<int> cell{-1};
  return cell;
}

inline std::mutex& sink_mutex() {
  static std::mutex m;
  return m;
}

inline void emit(LogLevel lvl, const char* file, int line, const std::string& msg) {
  static const char* tags[] = {"TRC", "DBG", "INF", "WRN", "ERR", "FTL", "OFF"};
  const char* base = file;
  for (const char* p = file; *p; ++p)
    if (*p == '/') base = p + 1;
  auto now = std::chrono::duration_cast<std::chrono::milliseconds>(
                 std::chrono::system_clock::now().time_since_epoch())
                 .count();
  std::lock_guard<std::mutex> g(sink_mutex());
  std::fprintf(stderr, "[MCCL %s r%d %lld %s:%d] %s\n", tags[static_cast<int>(lvl)],
               rank_cell().load(), static_cast<long long>(now), base, line, msg.c_str());
}

}  // namespace logdetail

inline LogLevel log_level() { return static_cast<LogLevel>(logdetail::level_cell().load()); }
inline void set_log_level(LogLevel l) { logdetail::level_cell().store(static_cast<int>(l)); }
inline void set_log_level(const std::string& name) {
  set_log_level(logdetail::parse_level(name.c_str(), log_level()));
}
inline void set_log_rank(int rank) { logdetail::rank_cell().store(rank); }

}  // namespace mccl

#define MCCL_LOG(lvl, streamexpr)                                              \
  do {                                                                         \
    if (static_cast<int>(lvl) >= static_cast<int>(::mccl::log_level())) {      \
      std::ostringstream _mccl_ls;                                             \
      _mccl_ls << streamexpr;                                                  \
      ::mccl::logdetail::emit(lvl, __FILE__, __LINE__, _mccl_ls.str());        \
    }                                                                          \
  } while (0)

#define MCCL_TRACE(x) MCCL_LOG(::mccl::LogLevel::TRACE, x)
#define MCCL_DEBUG(x) MCCL_LOG(::mccl::LogLevel::DEBUG, x)
#define MCCL_INFO(x) MCCL_LOG(::mccl::LogLevel::INFO, x)
#define MCCL_WARN(x) MCCL_LOG(::mccl::LogLevel::WARN, x)
#define MCCL_ERROR(x) MCCL_LOG(::mccl::LogLevel::ERROR, x)
#define MCCL_FATAL(x) MCCL_LOG(::mccl::LogLevel::FATAL, x)
#define MCCL_ABORT(x)        \
  do {                       \
    MCCL_FATAL(x);           \
    std::terminate();        \
  } while (0)
