// fuselink-monitor: stand-alone idleness monitor daemon.
//
// Creates the shared table (POSIX shm) and runs the sweeper until SIGINT/SIGTERM or for --seconds.  The
// reference's daemon (src/monitor_main.cpp:5-13) starts its thread without initialising the shared segment
// first; here the table is created and validated before the sweeper starts.
//
//   fuselink-monitor [--shm /fuselink_monitor] [--groups 8|auto] [--paths-per-group 1] [--timeout-us 160]
//                    [--period-us 40] [--seconds N] [--print-every-ms M]
//
// --groups auto sizes the table from the machine the way the reference's detectRdmaNics does
// (src/monitor.cpp:88-100): the RDMA devices under /sys/class/infiniband, else the GPUs the NVIDIA driver lists, else 8.
#include <dirent.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <string>

#include "monitor.h"

static int count_entries(const char* dir) {
  DIR* d = opendir(dir);
  if (!d) return 0;
  int n = 0;
  while (dirent* e = readdir(d))
    if (e->d_name[0] != '.') ++n;
  closedir(d);
  return n;
}
static int detect_paths() {
  int n = count_entries("/sys/class/infiniband");
  if (n <= 0) n = count_entries("/proc/driver/nvidia/gpus");
  if (n <= 0) n = 8;
  return n > 64 ? 64 : n;
}

static volatile sig_atomic_t g_stop = 0;
static void on_sig(int) { g_stop = 1; }

int main(int argc, char** argv) {
  std::string shm = "/fuselink_monitor";
  int groups = 8, ppg = 1, timeout_us = FL_MON_DEFAULT_TIMEOUT_US, period_us = 40, print_ms = 0;
  double seconds = 0;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() { return i + 1 < argc ? argv[++i] : (char*)"0"; };
    if (a == "--shm") shm = next();
    else if (a == "--groups") { const char* v = next(); groups = !strcmp(v, "auto") ? detect_paths() : atoi(v); }
    else if (a == "--paths-per-group") ppg = atoi(next());
    else if (a == "--timeout-us") timeout_us = atoi(next());
    else if (a == "--period-us") period_us = atoi(next());
    else if (a == "--seconds") seconds = atof(next());
    else if (a == "--print-every-ms") print_ms = atoi(next());
    else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
  }
  FlMonitor* m = fl_monitor_open(shm.c_str(), 1, groups, ppg, timeout_us);
  if (!m) { fprintf(stderr, "fuselink-monitor: %s\n", fl_monitor_last_error()); return 1; }
  signal(SIGINT, on_sig);
  signal(SIGTERM, on_sig);
  fl_monitor_start(m, period_us);
  printf("fuselink-monitor: table %s, %d paths, lease %d us\n", shm.c_str(), fl_monitor_num_paths(m), timeout_us);
  fflush(stdout);
  const uint64_t t0 = fl_monitor_now_ns();
  uint64_t last_print = t0;
  while (!g_stop) {
    usleep(1000);
    const uint64_t now = fl_monitor_now_ns();
    if (seconds > 0 && (now - t0) > (uint64_t)(seconds * 1e9)) break;
    if (print_ms > 0 && now - last_print > (uint64_t)print_ms * 1000000ull) {
      last_print = now;
      printf("tx idle mask %016llx  rx idle mask %016llx  decisions %llu\n", (unsigned long long)fl_monitor_idle_mask(m, FL_DIR_TX),
             (unsigned long long)fl_monitor_idle_mask(m, FL_DIR_RX), (unsigned long long)fl_monitor_decisions(m));
      fflush(stdout);
    }
  }
  fl_monitor_close(m, 1);
  return 0;
}
