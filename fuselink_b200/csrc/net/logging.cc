#include "logging.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

namespace flnet {
namespace {
ncclDebugLogger_t g_logger = nullptr;
int stderr_level() {
  static int lvl = -1;
  if (lvl < 0) {
    const char* s = getenv("FUSELINK_DEBUG");
    lvl = NCCL_LOG_WARN;
    if (s) {
      if (!strcasecmp(s, "INFO")) lvl = NCCL_LOG_INFO;
      else if (!strcasecmp(s, "TRACE")) lvl = NCCL_LOG_TRACE;
      else if (!strcasecmp(s, "NONE")) lvl = NCCL_LOG_NONE;
    }
  }
  return lvl;
}
}  // namespace

void log_set(ncclDebugLogger_t fn) { g_logger = fn; }

void log_msg(ncclDebugLogLevel lvl, const char* file, int line, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (g_logger) {
    g_logger(lvl, ~0ul /* all subsystems */, file, line, "NET/FuseLink : %s", buf);
    return;
  }
  const int order = lvl == NCCL_LOG_WARN ? 1 : lvl == NCCL_LOG_INFO ? 2 : 3;
  const int cfg = stderr_level();
  const int cfg_order = cfg == NCCL_LOG_NONE ? 0 : cfg == NCCL_LOG_WARN ? 1 : cfg == NCCL_LOG_INFO ? 2 : 3;
  if (order <= cfg_order) fprintf(stderr, "[fuselink %s] %s\n", lvl == NCCL_LOG_WARN ? "WARN" : lvl == NCCL_LOG_INFO ? "INFO" : "TRACE", buf);
}

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

void Timers::print(const char* who) const {
  static const char* names[T_COUNT] = {"isend", "irecv", "post_desc", "progress", "flush", "select"};
  for (int i = 0; i < T_COUNT; ++i)
    if (calls[i]) fprintf(stderr, "[fuselink timer] %s %-9s calls %llu total %.3f ms avg %.2f us\n", who, names[i],
                          (unsigned long long)calls[i], total_ns[i] / 1e6, total_ns[i] / 1e3 / calls[i]);
}
}  // namespace flnet
