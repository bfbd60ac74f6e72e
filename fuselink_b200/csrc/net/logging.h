// Logging through NCCL's logger when the plugin runs inside NCCL, to stderr otherwise; plus the
// phase timers the reference compiles out behind ENABLE_TIMER (src/extern/timer.h:33-59,
// src/plugin.cc:23) — here they are a run-time switch (FUSELINK_TIMERS=1) and use the monotonic clock.
#pragma once
#include <stdint.h>
#include "nccl_net_abi.h"

namespace flnet {
void log_set(ncclDebugLogger_t fn);
void log_msg(ncclDebugLogLevel lvl, const char* file, int line, const char* fmt, ...) __attribute__((format(printf, 4, 5)));
uint64_t now_ns();

enum TimerId { T_ISEND = 0, T_IRECV = 1, T_POST_DESC = 2, T_PROGRESS = 3, T_FLUSH = 4, T_SELECT = 5, T_COUNT = 6 };
struct Timers {
  uint64_t total_ns[T_COUNT] = {0};
  uint64_t calls[T_COUNT] = {0};
  void add(int id, uint64_t ns) { total_ns[id] += ns; calls[id]++; }
  void print(const char* who) const;
};
struct ScopedTimer {
  Timers* t; int id; uint64_t t0; bool on;
  ScopedTimer(Timers* t_, int id_, bool on_) : t(t_), id(id_), t0(on_ ? now_ns() : 0), on(on_) {}
  ~ScopedTimer() { if (on) t->add(id, now_ns() - t0); }
};
}  // namespace flnet

#define FL_WARN(...) ::flnet::log_msg(NCCL_LOG_WARN, __FILE__, __LINE__, __VA_ARGS__)
#define FL_INFO(...) ::flnet::log_msg(NCCL_LOG_INFO, __FILE__, __LINE__, __VA_ARGS__)
#define FL_TRACE(...) ::flnet::log_msg(NCCL_LOG_TRACE, __FILE__, __LINE__, __VA_ARGS__)
