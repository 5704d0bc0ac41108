// Leveled logging with the reference daemon's timestamped line format
// (src/mccs/src/main.rs:38-64). The level comes from MCCS_LOG
// (error|warn|info|debug|trace; default warn).
#pragma once
#include <stdarg.h>

namespace mccs {

enum LogLevel { kLogError = 0, kLogWarn = 1, kLogInfo = 2, kLogDebug = 3, kLogTrace = 4 };

int log_level();
void set_log_level(int level);
void log_write(int level, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 4, 5)));

}  // namespace mccs

#define MCCS_LOG(level, ...)                                                      \
  do {                                                                            \
    if ((level) <= ::mccs::log_level()) ::mccs::log_write((level), __FILE__, __LINE__, __VA_ARGS__); \
  } while (0)
#define LOG_ERROR(...) MCCS_LOG(::mccs::kLogError, __VA_ARGS__)
#define LOG_WARN(...) MCCS_LOG(::mccs::kLogWarn, __VA_ARGS__)
#define LOG_INFO(...) MCCS_LOG(::mccs::kLogInfo, __VA_ARGS__)
#define LOG_DEBUG(...) MCCS_LOG(::mccs::kLogDebug, __VA_ARGS__)
#define LOG_TRACE(...) MCCS_LOG(::mccs::kLogTrace, __VA_ARGS__)
