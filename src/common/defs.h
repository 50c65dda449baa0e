// Logging, assertions and throw helpers. The log line format and the TP_VERBOSE_LOGGING
// environment variable are those of the reference (tensorpipe/common/defs.h:133-181,257-286) so
// existing users see the same output; TPB_VERBOSE_LOGGING overrides it.
//
// Verbosity levels: 1 context/listener/pipe lifecycle, 2 one line per message, 3 per pipe
// operation, 4 channel lifecycle, 5 per tensor, 6 per channel step, 7 transport lifecycle,
// 8 per transport op, 9 low-level events (polling, library loading).
#pragma once

#include <sys/time.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <iomanip>
#include <iostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <system_error>

namespace tpb {

inline const char* trimFilename(const char* f) {
  const char* s = std::strrchr(f, '/');
  return s ? s + 1 : f;
}

class LogEntry final {
 public:
  explicit LogEntry(char type) {
    timeval tv;
    gettimeofday(&tv, nullptr);
    std::tm tm;
    localtime_r(&tv.tv_sec, &tm);
    oss_ << type << std::setfill('0') << std::setw(2) << 1 + tm.tm_mon << std::setw(2) << tm.tm_mday
         << ' ' << std::setw(2) << tm.tm_hour << ':' << std::setw(2) << tm.tm_min << ':'
         << std::setw(2) << tm.tm_sec << '.' << std::setw(6) << tv.tv_usec << ' ' << getpid() << ' ';
  }
  ~LogEntry() {
    oss_ << '\n';
    std::cerr << oss_.str();
  }
  std::ostream& getStream() { return oss_; }

 private:
  std::ostringstream oss_;
};

inline unsigned long getVerbosityLevel() {
  static unsigned long level = [] {
    const char* s = std::getenv("TPB_VERBOSE_LOGGING");
    if (!s) s = std::getenv("TP_VERBOSE_LOGGING");
    return s ? std::strtoul(s, nullptr, 10) : 0ul;
  }();
  return level;
}

#define TPB_LOG_LOC ::tpb::trimFilename(__FILE__) << ":" << __LINE__ << "] "
#define TPB_LOG_WARNING ::tpb::LogEntry('W').getStream() << TPB_LOG_LOC
#define TPB_LOG_ERROR ::tpb::LogEntry('E').getStream() << TPB_LOG_LOC
#define TPB_LOG_INFO ::tpb::LogEntry('I').getStream() << TPB_LOG_LOC
#define TPB_VLOG(level) \
  if (::tpb::getVerbosityLevel() >= (level)) ::tpb::LogEntry('V').getStream() << TPB_LOG_LOC

[[noreturn]] inline void throwLogic(const char* file, int line, const std::string& what) {
  std::ostringstream ss;
  ss << "In " << trimFilename(file) << ":" << line << " \"" << what << "\"";
  throw std::runtime_error(ss.str());
}
[[noreturn]] inline void throwSystem(const char* file, int line, int err, const std::string& what) {
  std::ostringstream ss;
  ss << "In " << trimFilename(file) << ":" << line << " \"" << what << "\"";
  throw std::system_error(err, std::system_category(), ss.str());
}

// User logic errors throw; they are not delivered through callbacks.
#define TPB_THROW_ASSERT_IF(cond, msg)                                                    \
  do {                                                                                   \
    if (cond) ::tpb::throwLogic(__FILE__, __LINE__, std::string(#cond) + ": " + (msg));  \
  } while (0)
#define TPB_THROW_SYSTEM_IF(cond, err, msg)                                  \
  do {                                                                       \
    if (cond) ::tpb::throwSystem(__FILE__, __LINE__, (err), (msg));          \
  } while (0)
#define TPB_ARG_CHECK(cond, msg) TPB_THROW_ASSERT_IF(!(cond), msg)

#ifdef NDEBUG
#define TPB_DCHECK(cond) \
  do {                   \
  } while (0)
#else
#define TPB_DCHECK(cond)                                                               \
  do {                                                                                 \
    if (!(cond)) {                                                                     \
      TPB_LOG_ERROR << "check failed: " #cond;                                         \
      std::abort();                                                                    \
    }                                                                                  \
  } while (0)
#endif

}  // namespace tpb
