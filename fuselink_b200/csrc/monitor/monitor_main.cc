// fuselink-monitor: stand-alone idleness monitor daemon.
//
// Creates the shared table (POSIX shm) and runs the sweeper until SIGINT/SIGTERM or for --seconds.  The
// reference's daemon (src/monitor_main.cpp:5-13) starts its thread without initialising the shared segment
// first; here the table is created and validated before the sweeper starts.
//
//   fuselink-monitor [--shm /fuselink_monitor] [--groups 8|auto] [--paths-per-group 1] [--timeout-us 160]
//                    [--period-us 40] [--seconds N] [--print-every-ms M]
//   fuselink-monitor --bench ITERATIONS [--threads T] [--groups 8]
//
// --bench times what a sender pays per transfer, on a private table with the sweeper running and T threads at once:
// one selector decision (fl_select_paths, degree 2, with the release of the borrowed path), one borrow + release,
// one activity stamp, one posted + completed byte count; prints one JSON line with the nanoseconds per call.
//
// --groups auto sizes the table from the machine the way the reference's detectRdmaNics does
// (src/monitor.cpp:88-100): the RDMA devices under /sys/class/infiniband, else the GPUs the NVIDIA driver lists, else 8.
#include <dirent.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

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

// ns per call of `op`, run `iters` times by each of `threads` threads at once (the slowest thread's average)
template <class Op>
static double time_calls(int threads, long iters, Op op) {
  std::vector<double> ns(threads, 0.0);
  std::atomic<int> ready{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < threads; ++t)
    ts.emplace_back([&, t] {
      ready.fetch_add(1);
      while (ready.load() < threads) {}
      const uint64_t t0 = fl_monitor_now_ns();
      for (long i = 0; i < iters; ++i) op(t, i);
      ns[t] = double(fl_monitor_now_ns() - t0) / double(iters);
    });
  double worst = 0;
  for (int t = 0; t < threads; ++t) {
    ts[t].join();
    if (ns[t] > worst) worst = ns[t];
  }
  return worst;
}

static int run_bench(long iters, int threads, int groups) {
  FlMonitor* m = fl_monitor_open("", 1, groups, 1, FL_MON_DEFAULT_TIMEOUT_US);
  if (!m) { fprintf(stderr, "fuselink-monitor: %s\n", fl_monitor_last_error()); return 1; }
  fl_monitor_start(m, 40);
  FlSelectorCfg cfg;
  cfg.degree = 2; cfg.step = 1; cfg.min_stripe_bytes = 1 << 20; cfg.align = 1 << 19; cfg.allow_relay = 1;
  const double select_ns = time_calls(threads, iters, [&](int t, long i) {
    FlStripe st[4];
    const int src = t % groups, dst = (t + 1) % groups;
    const int n = fl_select_paths(m, &cfg, src, dst, 64ull << 20, (unsigned long long)i, st, 4, fl_monitor_now_ns());
    for (int k = 1; k < n; ++k) fl_monitor_release(m, FL_DIR_TX, st[k].path);
  });
  const double borrow_ns = time_calls(threads, iters, [&](int t, long) {
    const int p = fl_monitor_borrow_idle(m, FL_DIR_TX, t % groups, t % groups, ~0ull, fl_monitor_now_ns());
    if (p >= 0) fl_monitor_release(m, FL_DIR_TX, p);
  });
  const double stamp_ns = time_calls(threads, iters, [&](int t, long) { fl_monitor_mark_active(m, FL_DIR_TX, t % groups, fl_monitor_now_ns()); });
  const double bytes_ns = time_calls(threads, iters, [&](int t, long) {
    const uint64_t now = fl_monitor_now_ns();
    fl_monitor_post_bytes(m, FL_DIR_TX, t % groups, 4096, now);
    fl_monitor_complete_bytes(m, FL_DIR_TX, t % groups, 4096, now);
  });
  const double clock_ns = time_calls(threads, iters, [&](int, long) { (void)fl_monitor_now_ns(); });
  printf("{\"bench\": \"monitor\", \"threads\": %d, \"paths\": %d, \"iterations\": %ld, \"select_paths_ns\": %.1f, "
         "\"borrow_release_ns\": %.1f, \"mark_active_ns\": %.1f, \"post_complete_bytes_ns\": %.1f, \"clock_read_ns\": %.1f, "
         "\"decisions\": %llu}\n",
         threads, fl_monitor_num_paths(m), iters, select_ns, borrow_ns, stamp_ns, bytes_ns, clock_ns,
         (unsigned long long)fl_monitor_decisions(m));
  fl_monitor_stop(m);
  fl_monitor_close(m, 0);
  return 0;
}

static volatile sig_atomic_t g_stop = 0;
static void on_sig(int) { g_stop = 1; }

int main(int argc, char** argv) {
  std::string shm = "/fuselink_monitor";
  int groups = 8, ppg = 1, timeout_us = FL_MON_DEFAULT_TIMEOUT_US, period_us = 40, print_ms = 0;
  double seconds = 0;
  long bench_iters = 0;
  int bench_threads = 1;
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
    else if (a == "--bench") bench_iters = atol(next());
    else if (a == "--threads") bench_threads = atoi(next());
    else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
  }
  if (bench_iters > 0) return run_bench(bench_iters, bench_threads < 1 ? 1 : bench_threads, groups);
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
