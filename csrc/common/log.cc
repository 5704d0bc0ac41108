#include "log.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include <atomic>

namespace mccs {

static std::atomic<int> g_level{-1};

static int parse_level(const char* s) {
  if (!s) return kLogWarn;
  if (!strcasecmp(s, "error")) return kLogError;
  if (!strcasecmp(s, "warn")) return kLogWarn;
  if (!strcasecmp(s, "info")) return kLogInfo;
  if (!strcasecmp(s, "debug")) return kLogDebug;
  if (!strcasecmp(s, "trace")) return kLogTrace;
  return kLogWarn;
}

int log_level() {
  int l = g_level.load(std::memory_order_relaxed);
  if (l < 0) {
    l = parse_level(getenv("MCCS_LOG"));
    g_level.store(l, std::memory_order_relaxed);
  }
  return l;
}

void set_log_level(int level) { g_level.store(level, std::memory_order_relaxed); }

void log_write(int level, const char* file, int line, const char* fmt, ...) {
  static const char* names[] = {"ERROR", "WARN", "INFO", "DEBUG", "TRACE"};
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  struct tm tmv;
  localtime_r(&tv.tv_sec, &tmv);
  char msg[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof msg, fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  char out[1200];
  int n = snprintf(out, sizeof out, "[%04d-%02d-%02d %02d:%02d:%02d.%06ld %s %s:%d pid=%d] %s\n",
                   tmv.tm_year + 1900, tmv.tm_mon + 1, tmv.tm_mday, tmv.tm_hour, tmv.tm_min,
                   tmv.tm_sec, (long)tv.tv_usec, names[level < 0 ? 0 : (level > 4 ? 4 : level)], base,
                   line, (int)getpid(), msg);
  if (n > 0) fwrite(out, 1, (size_t)(n < (int)sizeof out ? n : (int)sizeof out - 1), stderr);
}

}  // namespace mccs
