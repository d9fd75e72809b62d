#include "log.h"

#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>
#include <vector>

namespace pplx {
namespace {

std::atomic<int> g_level{static_cast<int>(LogLevel::kInfo)};
std::atomic<int> g_format{static_cast<int>(LogFormat::kText)};
std::atomic<bool> g_color{false};
std::mutex g_mutex;

const char* level_name(LogLevel l) {
  switch (l) {
    case LogLevel::kError: return "ERROR";
    case LogLevel::kWarn: return "WARN";
    case LogLevel::kInfo: return "INFO";
    case LogLevel::kDebug: return "DEBUG";
    default: return "TRACE";
  }
}

const char* level_color(LogLevel l) {
  switch (l) {
    case LogLevel::kError: return "\x1b[31m";
    case LogLevel::kWarn: return "\x1b[33m";
    case LogLevel::kInfo: return "\x1b[32m";
    case LogLevel::kDebug: return "\x1b[34m";
    default: return "\x1b[35m";
  }
}

bool parse_level(const char* s, LogLevel* out) {
  if (s == nullptr) return false;
  std::string v;
  for (const char* p = s; *p; ++p) v.push_back(static_cast<char>(std::tolower(*p)));
  // accept "target=level,..." filters by taking the last bare level word
  const size_t eq = v.rfind('=');
  if (eq != std::string::npos) v = v.substr(eq + 1);
  if (v == "error") *out = LogLevel::kError;
  else if (v == "warn" || v == "warning") *out = LogLevel::kWarn;
  else if (v == "info") *out = LogLevel::kInfo;
  else if (v == "debug") *out = LogLevel::kDebug;
  else if (v == "trace") *out = LogLevel::kTrace;
  else return false;
  return true;
}

void json_escape(const std::string& in, std::string* out) {
  for (unsigned char c : in) {
    switch (c) {
      case '"': *out += "\\\""; break;
      case '\\': *out += "\\\\"; break;
      case '\n': *out += "\\n"; break;
      case '\r': *out += "\\r"; break;
      case '\t': *out += "\\t"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\u%04x", c);
          *out += buf;
        } else {
          out->push_back(static_cast<char>(c));
        }
    }
  }
}

std::string iso_time(double unix_time) {
  const time_t secs = static_cast<time_t>(unix_time);
  const int micros = static_cast<int>((unix_time - static_cast<double>(secs)) * 1e6);
  struct tm tmv;
  gmtime_r(&secs, &tmv);
  char buf[64];
  std::snprintf(buf, sizeof(buf), "%04d-%02d-%02dT%02d:%02d:%02d.%06dZ", tmv.tm_year + 1900,
                tmv.tm_mon + 1, tmv.tm_mday, tmv.tm_hour, tmv.tm_min, tmv.tm_sec, micros);
  return buf;
}

}  // namespace

void log_init_from_env() {
  LogLevel lvl;
  if (parse_level(std::getenv("PPLX_LOG"), &lvl) || parse_level(std::getenv("RUST_LOG"), &lvl)) {
    g_level = static_cast<int>(lvl);
  }
  const char* fmt = std::getenv("PPLX_LOG_FORMAT");
  if (fmt != nullptr && std::strcmp(fmt, "json") == 0) {
    g_format = static_cast<int>(LogFormat::kJson);
  } else {
    g_format = static_cast<int>(LogFormat::kText);
  }
  const char* color = std::getenv("PPLX_LOG_COLOR");
  if (color != nullptr && std::strcmp(color, "always") == 0) {
    g_color = true;
  } else if (color != nullptr && std::strcmp(color, "never") == 0) {
    g_color = false;
  } else {
    g_color = isatty(fileno(stderr)) != 0;
  }
}

void log_set_level(LogLevel level) { g_level = static_cast<int>(level); }
void log_set_format(LogFormat format) { g_format = static_cast<int>(format); }
LogLevel log_level() { return static_cast<LogLevel>(g_level.load()); }
bool log_enabled(LogLevel level) { return static_cast<int>(level) <= g_level.load(); }

std::string log_render(LogLevel level, const char* target, const std::string& msg,
                       LogFormat format, bool color, double unix_time) {
  std::string out;
  if (format == LogFormat::kJson) {
    out += "{\"timestamp\":\"" + iso_time(unix_time) + "\",\"level\":\"" + level_name(level) +
           "\",\"target\":\"";
    json_escape(target, &out);
    out += "\",\"fields\":{\"message\":\"";
    json_escape(msg, &out);
    out += "\"}}";
  } else {
    out += iso_time(unix_time);
    out += ' ';
    if (color) out += level_color(level);
    char lv[8];
    std::snprintf(lv, sizeof(lv), "%5s", level_name(level));
    out += lv;
    if (color) out += "\x1b[0m";
    out += ' ';
    out += target;
    out += ": ";
    out += msg;
  }
  return out;
}

void log_message(LogLevel level, const char* target, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  va_list ap2;
  va_copy(ap2, ap);
  const int n = std::vsnprintf(nullptr, 0, fmt, ap);
  va_end(ap);
  std::vector<char> buf(static_cast<size_t>(n > 0 ? n : 0) + 1);
  std::vsnprintf(buf.data(), buf.size(), fmt, ap2);
  va_end(ap2);
  const double now = std::chrono::duration<double>(
                         std::chrono::system_clock::now().time_since_epoch())
                         .count();
  const std::string line =
      log_render(level, target, std::string(buf.data()),
                 static_cast<LogFormat>(g_format.load()), g_color.load(), now);
  std::lock_guard<std::mutex> lock(g_mutex);
  std::fprintf(stderr, "%s\n", line.c_str());
}

}  // namespace pplx
