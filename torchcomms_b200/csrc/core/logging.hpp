// Minimal levelled logger with a bounded in-memory ring that `comm_dump`
// style introspection can read back. Level comes from B200COMMS_LOG_LEVEL
// (error|warn|info|debug); lines go to stderr.
//
// Parity: comms/torchcomms/utils/Logging.hpp:25-62 (rank/name-prefixed log
// macros). The ring replaces the structured sinks of comms/utils/logger.
#pragma once

#include <deque>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace b200c {

enum class LogLevel : int { ERROR = 0, WARN = 1, INFO = 2, DEBUG = 3 };

class Logger {
 public:
  static Logger& get();
  bool enabled(LogLevel lvl) const { return static_cast<int>(lvl) <= level_; }
  void write(LogLevel lvl, const std::string& who, const std::string& msg);
  std::vector<std::string> recent() const;
  void set_level(LogLevel lvl) { level_ = static_cast<int>(lvl); }

 private:
  Logger();
  int level_;
  mutable std::mutex mu_;
  std::deque<std::string> ring_;
  static constexpr size_t kRingCap = 512;
};

} // namespace b200c

#define B200C_LOG(lvl, who, expr)                                         \
  do {                                                                    \
    if (::b200c::Logger::get().enabled(::b200c::LogLevel::lvl)) {         \
      std::ostringstream _b200c_os;                                       \
      _b200c_os << expr;                                                  \
      ::b200c::Logger::get().write(::b200c::LogLevel::lvl, (who), _b200c_os.str()); \
    }                                                                     \
  } while (0)
