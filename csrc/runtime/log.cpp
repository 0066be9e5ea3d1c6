#include "log.h"

#include <unistd.h>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <mutex>
#include <thread>

#include "../device/device_api.h"

namespace catch_b200 {

namespace {
std::atomic<int> g_min_level{-100};

int parse_level_env() {
  const char* s = std::getenv("CATCH_B200_MIN_LOG_LEVEL");
  if (!s || !*s) return static_cast<int>(LogLevel::WARNING);
  char* end = nullptr;
  long v = std::strtol(s, &end, 10);
  if (end == s) {
    if (!strcasecmp(s, "DEBUG") || !strcasecmp(s, "DBG")) return -1;
    if (!strcasecmp(s, "INFO")) return 0;
    if (!strcasecmp(s, "WARNING")) return 1;
    if (!strcasecmp(s, "ERROR")) return 2;
    if (!strcasecmp(s, "FATAL")) return 3;
    return 1;
  }
  if (v < -1) v = -1;
  if (v > 3) v = 3;
  return static_cast<int>(v);
}

const char* level_name(LogLevel l) {
  switch (l) {
    case LogLevel::DBG: return "DEBUG";
    case LogLevel::INFO: return "INFO";
    case LogLevel::WARNING: return "WARNING";
    case LogLevel::ERROR: return "ERROR";
    case LogLevel::FATAL: return "FATAL";
  }
  return "?";
}

bool env_true(const char* name, bool dflt) {
  const char* s = std::getenv(name);
  if (!s || !*s) return dflt;
  if (!strcasecmp(s, "1") || !strcasecmp(s, "on") || !strcasecmp(s, "true") || !strcasecmp(s, "yes")) return true;
  if (!strcasecmp(s, "0") || !strcasecmp(s, "off") || !strcasecmp(s, "false") || !strcasecmp(s, "no")) return false;
  return dflt;
}
}  // namespace

int min_log_level() {
  int v = g_min_level.load(std::memory_order_relaxed);
  if (v == -100) {
    v = parse_level_env();
    g_min_level.store(v, std::memory_order_relaxed);
  }
  return v;
}

void set_min_log_level(int lvl) { g_min_level.store(lvl, std::memory_order_relaxed); }

LogMessage::LogMessage(const char* file, int line, const char* func, LogLevel lvl) : lvl_(lvl) {
  const char* base = std::strrchr(file, '/');
  os_ << "[" << level_name(lvl) << "][" << (base ? base + 1 : file) << "][line:" << line << "][" << func
      << "][thread:" << std::this_thread::get_id() << "][process:" << getpid() << "]: ";
}

LogMessage::~LogMessage() noexcept(false) {
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    std::cerr << os_.str() << std::endl;
  }
  if (lvl_ == LogLevel::FATAL) std::abort();
}

namespace {
Flags* flags_storage() {
  static Flags f{};
  return &f;
}
}  // namespace

void reload_flags() {
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  Flags x;
  x.async_disable = env_true("CATCH_B200_ASYNC_DISABLE", false);
  x.op_trycatch = env_true("CATCH_B200_OP_TRYCATCH", true);
  x.test_cpu_dispatch = env_true("CATCH_B200_TEST_CPU_DISPATCH", false);
  x.fallback_to_cpu = env_true("CATCH_B200_FALLBACK_TO_CPU", true);
  x.memory_debug = env_true("CATCH_B200_MEMORY_DEBUG", false);
  x.blocking_wait = env_true("CATCH_B200_BLOCKING_WAIT", false);
  const char* n = std::getenv("CATCH_B200_HOSTSIM_DEVICES");
  x.hostsim_devices = (n && *n) ? std::max(1, std::atoi(n)) : 2;
  const char* b = std::getenv("CATCH_B200_BACKEND");
  x.backend = (b && *b) ? b : "auto";
  *flags_storage() = x;
}

Flags& flags() {
  static std::once_flag once;
  std::call_once(once, [] { reload_flags(); });
  return *flags_storage();
}

const char* device_error_string(int err) { return b200_error_string(err); }

}  // namespace catch_b200
