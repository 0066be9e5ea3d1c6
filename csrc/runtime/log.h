// Levelled stream logger, environment flags and check macros of the backend.
//
// Capability parity: the reference's CNLOG (torch_mlu/csrc/aten/util/cnlog.h:46-177,
// cnlog.cpp:41-88) has levels DBG(-1)..FATAL(3), a minimum level read from the
// environment and a prefix with file/line/function/thread/pid; its check macros
// live in torch_mlu/csrc/aten/util/exceptions.h:41-90 and its environment
// switches are listed in the user guide.  This file provides the same
// facilities for the b200 backend with its own variable names.
#pragma once
#include <c10/util/Exception.h>
#include <cstdint>
#include <sstream>
#include <string>

namespace catch_b200 {

enum class LogLevel : int { DBG = -1, INFO = 0, WARNING = 1, ERROR = 2, FATAL = 3 };

int min_log_level();             // CATCH_B200_MIN_LOG_LEVEL, default WARNING
void set_min_log_level(int lvl);  // runtime override (used by tests)

class LogMessage {
 public:
  LogMessage(const char* file, int line, const char* func, LogLevel lvl);
  ~LogMessage() noexcept(false);
  std::ostream& stream() { return os_; }

 private:
  std::ostringstream os_;
  LogLevel lvl_;
};

#define B200LOG(lvl)                                                            \
  if (static_cast<int>(::catch_b200::LogLevel::lvl) < ::catch_b200::min_log_level()) \
    ;                                                                           \
  else                                                                          \
    ::catch_b200::LogMessage(__FILE__, __LINE__, __func__, ::catch_b200::LogLevel::lvl).stream()

// ---- environment flags -------------------------------------------------------
struct Flags {
  bool async_disable;      // CATCH_B200_ASYNC_DISABLE=1  : synchronise after every op / collective
  bool op_trycatch;        // CATCH_B200_OP_TRYCATCH=off  : disable "device kernel failed -> rerun on CPU"
  bool test_cpu_dispatch;  // CATCH_B200_TEST_CPU_DISPATCH=1 : force the CPU implementation of every op
  bool fallback_to_cpu;    // CATCH_B200_FALLBACK_TO_CPU=0 : unregistered ops raise instead of running on CPU
  bool memory_debug;       // CATCH_B200_MEMORY_DEBUG=1   : guard-word debug allocator
  bool blocking_wait;      // CATCH_B200_BLOCKING_WAIT=1  : Work::wait() blocks the host
  int hostsim_devices;     // CATCH_B200_HOSTSIM_DEVICES  : device count of the host-simulated backend
  std::string backend;     // CATCH_B200_BACKEND=auto|cuda|hostsim
};
Flags& flags();            // mutable so tests / Python setters can flip switches
void reload_flags();       // re-read the environment

// ---- checks --------------------------------------------------------------------
const char* device_error_string(int err);

#define B200_CHECK(cond, ...) TORCH_CHECK(cond, ##__VA_ARGS__)

#define B200_DEVICE_CHECK(expr)                                                  \
  do {                                                                           \
    int _b200_err = (expr);                                                      \
    TORCH_CHECK(_b200_err == 0, "b200 runtime error ", _b200_err, " (",          \
                ::catch_b200::device_error_string(_b200_err), ") in `", #expr,   \
                "` at ", __FILE__, ":", __LINE__);                               \
  } while (0)

#define B200_DEVICE_WARN(expr)                                                   \
  do {                                                                           \
    int _b200_err = (expr);                                                      \
    if (_b200_err != 0) {                                                        \
      B200LOG(WARNING) << "b200 runtime error " << _b200_err << " ("             \
                       << ::catch_b200::device_error_string(_b200_err)           \
                       << ") in `" #expr "`";                                    \
    }                                                                            \
  } while (0)

}  // namespace catch_b200
