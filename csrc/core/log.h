// Process-wide logger of the native code: text or JSON lines on stderr.
// Environment (same knobs as the reference's logging-lib, rust/logging-lib/src/lib.rs:8-66):
//   PPLX_LOG_FORMAT = text | json         (default text)
//   PPLX_LOG_COLOR  = auto | always | never
//   PPLX_LOG / RUST_LOG = error | warn | info | debug | trace   (default info)
#pragma once

#include <cstdarg>
#include <string>

namespace pplx {

enum class LogLevel : int { kError = 0, kWarn = 1, kInfo = 2, kDebug = 3, kTrace = 4 };
enum class LogFormat : int { kText = 0, kJson = 1 };

void log_init_from_env();
void log_set_level(LogLevel level);
void log_set_format(LogFormat format);
LogLevel log_level();
bool log_enabled(LogLevel level);
void log_message(LogLevel level, const char* target, const char* fmt, ...)
    __attribute__((format(printf, 3, 4)));
// Renders one record the way log_message would (used by tests).
std::string log_render(LogLevel level, const char* target, const std::string& msg,
                       LogFormat format, bool color, double unix_time);

#define PPLX_LOG(level, ...)                                         \
  do {                                                               \
    if (::pplx::log_enabled(level)) {                                \
      ::pplx::log_message(level, PPLX_LOG_TARGET, __VA_ARGS__);      \
    }                                                                \
  } while (0)
#define PPLX_ERROR(...) PPLX_LOG(::pplx::LogLevel::kError, __VA_ARGS__)
#define PPLX_WARN(...) PPLX_LOG(::pplx::LogLevel::kWarn, __VA_ARGS__)
#define PPLX_INFO(...) PPLX_LOG(::pplx::LogLevel::kInfo, __VA_ARGS__)
#define PPLX_DEBUG(...) PPLX_LOG(::pplx::LogLevel::kDebug, __VA_ARGS__)

#ifndef PPLX_LOG_TARGET
#define PPLX_LOG_TARGET "pplx_garden"
#endif

}  // namespace pplx
