// Stress driver of the lock-free monitor for the sanitizer tier (built with -fsanitize=thread or address,undefined):
// several borrower threads, an activity-stamping thread and the sweeper thread hammer one table.  Exit code 0 means the
// exclusivity invariant held (a BORROWED path has exactly one holder) and, under a sanitizer, that no report was raised.
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <thread>
#include <vector>

#include "monitor.h"

int main(int argc, char** argv) {
  const int iters = argc > 1 ? atoi(argv[1]) : 20000;
  const int npaths = 16;
  FlMonitor* m = fl_monitor_open("", 1, npaths, 1, 1000000 /* long lease: only explicit releases free a path */);
  if (!m) { fprintf(stderr, "open failed: %s\n", fl_monitor_last_error()); return 2; }
  fl_monitor_start(m, 20);
  std::atomic<int> holders[npaths];
  for (auto& h : holders) h.store(0);
  std::atomic<long> violations{0}, grants{0};
  std::vector<std::thread> ths;
  for (int g = 0; g < 4; ++g) {
    ths.emplace_back([&, g]() {
      for (int i = 0; i < iters; ++i) {
        const int p = fl_monitor_borrow_idle(m, FL_DIR_TX, g, g + i, 0xffff, fl_monitor_now_ns());
        if (p < 0) continue;
        grants.fetch_add(1);
        if (holders[p].fetch_add(1) != 0) violations.fetch_add(1);
        fl_monitor_post_bytes(m, FL_DIR_TX, p, 4096, fl_monitor_now_ns());
        fl_monitor_complete_bytes(m, FL_DIR_TX, p, 4096, fl_monitor_now_ns());
        holders[p].fetch_sub(1);
        fl_monitor_release(m, FL_DIR_TX, p);
      }
    });
  }
  // claimers: each wants "its own" path for itself; a claim that succeeds for two different owners at once is a violation
  for (int o = 0; o < 3; ++o) {
    ths.emplace_back([&, o]() {
      const int owner = 1000 + o;
      for (int i = 0; i < iters; ++i) {
        const int p = (i + o) % npaths;
        if (!fl_monitor_claim(m, FL_DIR_TX, p, owner, fl_monitor_now_ns())) continue;
        grants.fetch_add(1);
        if (holders[p].fetch_add(1) != 0) violations.fetch_add(1);
        holders[p].fetch_sub(1);
        fl_monitor_release(m, FL_DIR_TX, p);
      }
    });
  }
  ths.emplace_back([&]() {
    for (int i = 0; i < iters; ++i) {
      fl_monitor_mark_active(m, FL_DIR_RX, i % npaths, fl_monitor_now_ns());
      (void)fl_monitor_idle_mask(m, FL_DIR_RX);
      (void)fl_monitor_bandwidth_gbs(m, FL_DIR_TX, i % npaths);
    }
  });
  for (auto& t : ths) t.join();
  fl_monitor_stop(m);
  const long v = violations.load();
  printf("grants %ld violations %ld decisions %llu\n", grants.load(), v, (unsigned long long)fl_monitor_decisions(m));
  fl_monitor_close(m, 0);
  return v == 0 ? 0 : 1;
}
