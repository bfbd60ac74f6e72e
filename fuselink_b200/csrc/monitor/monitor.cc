// Lock-free idleness monitor + path selector (see monitor.h).
#include "monitor.h"

#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <new>
#include <string>
#include <thread>

namespace {

thread_local char g_err[256] = "";

constexpr uint32_t kMagic = 0x464c4d4eu;  // "FLMN"

struct alignas(64) Slot {
  std::atomic<uint32_t> status;
  std::atomic<int32_t> borrower;        // group that holds the lease, -1 if none
  std::atomic<uint64_t> last_active_ns;
  std::atomic<uint64_t> posted;
  std::atomic<uint64_t> completed;
  std::atomic<uint64_t> ext_seen;       // last value folded in from an attached external counter
  std::atomic<uint64_t> bw_bytes_mark;  // completed bytes at the last bandwidth sample
  std::atomic<uint64_t> bw_time_mark;
  std::atomic<uint64_t> bw_milli_gbs;   // EWMA bandwidth in 1e-3 GB/s
};
static_assert(sizeof(Slot) == 64 || sizeof(Slot) == 128, "slot must be cache-line sized");

struct Table {
  std::atomic<uint32_t> magic;
  uint32_t n_groups;
  uint32_t paths_per_group;
  uint32_t timeout_us;
  std::atomic<uint32_t> running;
  std::atomic<uint64_t> decisions;
  std::atomic<uint64_t> sweeps;
  Slot slots[2][FL_MON_MAX_PATHS];
};

}  // namespace

struct FlMonitor {
  Table* t = nullptr;
  bool shared = false;
  std::string shm_name;
  std::thread thr;
  std::atomic<bool> stop{false};
  const volatile uint64_t* ext[2] = {nullptr, nullptr};
};

extern "C" {

const char* fl_monitor_last_error(void) { return g_err; }

uint64_t fl_monitor_now_ns(void) {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

FlMonitor* fl_monitor_open(const char* shm_name, int owner, int n_groups, int paths_per_group, int timeout_us) {
  if (n_groups < 1 || paths_per_group < 1 || n_groups * paths_per_group > FL_MON_MAX_PATHS) {
    snprintf(g_err, sizeof g_err, "n_groups*paths_per_group must be in [1, %d]", FL_MON_MAX_PATHS);
    return nullptr;
  }
  FlMonitor* m = new FlMonitor();
  if (shm_name && shm_name[0]) {
    m->shared = true;
    m->shm_name = shm_name;
    int fd = shm_open(shm_name, owner ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
    if (fd < 0) {
      snprintf(g_err, sizeof g_err, "shm_open(%s) failed: is the monitor running?", shm_name);
      delete m;
      return nullptr;
    }
    if (owner && ftruncate(fd, sizeof(Table)) != 0) {
      snprintf(g_err, sizeof g_err, "ftruncate(%s) failed", shm_name);
      close(fd);
      delete m;
      return nullptr;
    }
    void* p = mmap(nullptr, sizeof(Table), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) {
      snprintf(g_err, sizeof g_err, "mmap(%s) failed", shm_name);
      delete m;
      return nullptr;
    }
    m->t = reinterpret_cast<Table*>(p);
  } else {
    owner = 1;
    void* p = mmap(nullptr, sizeof(Table), PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (p == MAP_FAILED) {
      snprintf(g_err, sizeof g_err, "anonymous mmap failed");
      delete m;
      return nullptr;
    }
    m->t = reinterpret_cast<Table*>(p);
  }
  if (owner) {
    memset((void*)m->t, 0, sizeof(Table));
    m->t->n_groups = (uint32_t)n_groups;
    m->t->paths_per_group = (uint32_t)paths_per_group;
    m->t->timeout_us = (uint32_t)(timeout_us > 0 ? timeout_us : FL_MON_DEFAULT_TIMEOUT_US);
    for (int d = 0; d < 2; ++d)
      for (int p = 0; p < FL_MON_MAX_PATHS; ++p) m->t->slots[d][p].borrower.store(-1, std::memory_order_relaxed);
    m->t->magic.store(kMagic, std::memory_order_release);
  } else if (m->t->magic.load(std::memory_order_acquire) != kMagic) {
    snprintf(g_err, sizeof g_err, "segment %s is not an initialised monitor table", shm_name);
    munmap(m->t, sizeof(Table));
    delete m;
    return nullptr;
  }
  return m;
}

void fl_monitor_close(FlMonitor* m, int unlink_shm) {
  if (!m) return;
  fl_monitor_stop(m);
  if (m->t) munmap(m->t, sizeof(Table));
  if (m->shared && unlink_shm) shm_unlink(m->shm_name.c_str());
  delete m;
}

int fl_monitor_num_paths(const FlMonitor* m) { return (int)(m->t->n_groups * m->t->paths_per_group); }
int fl_monitor_timeout_us(const FlMonitor* m) { return (int)m->t->timeout_us; }

void fl_monitor_sweep(FlMonitor* m, uint64_t now_ns) {
  Table* t = m->t;
  const int n = fl_monitor_num_paths(m);
  const uint64_t timeout_ns = (uint64_t)t->timeout_us * 1000ull;
  for (int d = 0; d < 2; ++d) {
    for (int p = 0; p < n; ++p) {
      Slot& s = t->slots[d][p];
      // fold in externally incremented completion counters (GPU-written)
      if (m->ext[d]) {
        const uint64_t v = m->ext[d][p];
        const uint64_t seen = s.ext_seen.load(std::memory_order_relaxed);
        if (v != seen) {
          s.ext_seen.store(v, std::memory_order_relaxed);
          s.completed.fetch_add(v - seen, std::memory_order_relaxed);
          s.last_active_ns.store(now_ns, std::memory_order_relaxed);
          uint32_t st = s.status.load(std::memory_order_relaxed);
          if (st == FL_PATH_IDLE) s.status.compare_exchange_strong(st, FL_PATH_BUSY, std::memory_order_acq_rel);
        }
      }
      // bandwidth estimate: EWMA over >= 50 us windows
      const uint64_t tm = s.bw_time_mark.load(std::memory_order_relaxed);
      if (tm == 0) {
        s.bw_time_mark.store(now_ns, std::memory_order_relaxed);
        s.bw_bytes_mark.store(s.completed.load(std::memory_order_relaxed), std::memory_order_relaxed);
      } else if (now_ns - tm >= 50000) {
        const uint64_t c = s.completed.load(std::memory_order_relaxed);
        const uint64_t db = c - s.bw_bytes_mark.load(std::memory_order_relaxed);
        const double gbs = (double)db / (double)(now_ns - tm);  // bytes per ns == GB/s
        const double prev = (double)s.bw_milli_gbs.load(std::memory_order_relaxed) / 1000.0;
        const double next = 0.75 * prev + 0.25 * gbs;
        s.bw_milli_gbs.store((uint64_t)(next * 1000.0), std::memory_order_relaxed);
        s.bw_time_mark.store(now_ns, std::memory_order_relaxed);
        s.bw_bytes_mark.store(c, std::memory_order_relaxed);
      }
      // lease / activity expiry: nothing outstanding and no stamp inside the window -> IDLE
      uint32_t st = s.status.load(std::memory_order_acquire);
      if (st == FL_PATH_BUSY || st == FL_PATH_BORROWED) {
        const uint64_t la = s.last_active_ns.load(std::memory_order_relaxed);
        const uint64_t outstanding = s.posted.load(std::memory_order_relaxed) - s.completed.load(std::memory_order_relaxed);
        if ((int64_t)outstanding <= 0 && la + timeout_ns <= now_ns) {
          if (s.status.compare_exchange_strong(st, FL_PATH_IDLE, std::memory_order_acq_rel))
            s.borrower.store(-1, std::memory_order_relaxed);
        }
      }
    }
  }
  t->sweeps.fetch_add(1, std::memory_order_relaxed);
}

int fl_monitor_start(FlMonitor* m, int period_us) {
  if (m->thr.joinable()) return 0;
  if (period_us <= 0) period_us = 40;
  m->stop.store(false);
  m->t->running.store(1, std::memory_order_release);
  m->thr = std::thread([m, period_us]() {
    timespec req;
    req.tv_sec = 0;
    req.tv_nsec = (long)period_us * 1000L;
    while (!m->stop.load(std::memory_order_acquire)) {
      fl_monitor_sweep(m, fl_monitor_now_ns());
      nanosleep(&req, nullptr);
    }
  });
  return 0;
}

void fl_monitor_stop(FlMonitor* m) {
  if (!m || !m->thr.joinable()) return;
  m->stop.store(true, std::memory_order_release);
  m->thr.join();
  m->t->running.store(0, std::memory_order_release);
}

static inline Slot* slot_of(FlMonitor* m, int dir, int path) {
  if (!m || dir < 0 || dir > 1 || path < 0 || path >= fl_monitor_num_paths(m)) return nullptr;
  return &m->t->slots[dir][path];
}

void fl_monitor_mark_active(FlMonitor* m, int dir, int path, uint64_t now_ns) {
  Slot* s = slot_of(m, dir, path);
  if (!s) return;
  s->last_active_ns.store(now_ns, std::memory_order_relaxed);
  uint32_t st = s->status.load(std::memory_order_relaxed);
  // a borrowed path stays BORROWED (its holder is the one stamping); DEAD stays DEAD
  if (st == FL_PATH_IDLE) s->status.compare_exchange_strong(st, FL_PATH_BUSY, std::memory_order_acq_rel);
}

void fl_monitor_post_bytes(FlMonitor* m, int dir, int path, uint64_t bytes, uint64_t now_ns) {
  Slot* s = slot_of(m, dir, path);
  if (!s) return;
  s->posted.fetch_add(bytes, std::memory_order_relaxed);
  fl_monitor_mark_active(m, dir, path, now_ns);
}

void fl_monitor_complete_bytes(FlMonitor* m, int dir, int path, uint64_t bytes, uint64_t now_ns) {
  Slot* s = slot_of(m, dir, path);
  if (!s) return;
  s->completed.fetch_add(bytes, std::memory_order_relaxed);
  s->last_active_ns.store(now_ns, std::memory_order_relaxed);
}

void fl_monitor_attach_counters(FlMonitor* m, int dir, const volatile uint64_t* counters) {
  if (m && dir >= 0 && dir < 2) m->ext[dir] = counters;
}

int fl_monitor_borrow_idle(FlMonitor* m, int dir, int group, int primary, uint64_t mask, uint64_t now_ns) {
  if (!m || dir < 0 || dir > 1) return -1;
  const int n = fl_monitor_num_paths(m);
  const int ppg = (int)m->t->paths_per_group;
  for (int k = 1; k <= n; ++k) {
    const int p = ((primary < 0 ? 0 : primary) + k) % n;
    if (p / ppg == group) continue;          // only other groups' paths can be borrowed
    if (!((mask >> p) & 1ull)) continue;
    Slot& s = m->t->slots[dir][p];
    uint32_t expect = FL_PATH_IDLE;
    if (s.status.compare_exchange_strong(expect, FL_PATH_BORROWED, std::memory_order_acq_rel)) {
      s.borrower.store(group, std::memory_order_relaxed);
      s.last_active_ns.store(now_ns, std::memory_order_relaxed);
      m->t->decisions.fetch_add(1, std::memory_order_relaxed);
      return p;
    }
  }
  return -1;
}

int fl_monitor_claim(FlMonitor* m, int dir, int path, int owner, uint64_t now_ns) {
  Slot* s = slot_of(m, dir, path);
  if (!s) return 0;
  uint32_t expect = FL_PATH_IDLE;
  if (s->status.compare_exchange_strong(expect, FL_PATH_BORROWED, std::memory_order_acq_rel)) {
    s->borrower.store(owner, std::memory_order_relaxed);
    s->last_active_ns.store(now_ns, std::memory_order_relaxed);
    return 1;
  }
  if (expect == FL_PATH_BORROWED && s->borrower.load(std::memory_order_relaxed) == owner) {
    s->last_active_ns.store(now_ns, std::memory_order_relaxed);
    return 1;
  }
  return 0;
}

void fl_monitor_release(FlMonitor* m, int dir, int path) {
  Slot* s = slot_of(m, dir, path);
  if (!s) return;
  uint32_t expect = FL_PATH_BORROWED;
  if (s->status.compare_exchange_strong(expect, FL_PATH_IDLE, std::memory_order_acq_rel))
    s->borrower.store(-1, std::memory_order_relaxed);
}

void fl_monitor_mark_dead(FlMonitor* m, int dir, int path, int dead) {
  Slot* s = slot_of(m, dir, path);
  if (!s) return;
  s->status.store(dead ? FL_PATH_DEAD : FL_PATH_IDLE, std::memory_order_release);
  s->borrower.store(-1, std::memory_order_relaxed);
}

int fl_monitor_status(const FlMonitor* m, int dir, int path) {
  Slot* s = slot_of(const_cast<FlMonitor*>(m), dir, path);
  return s ? (int)s->status.load(std::memory_order_acquire) : -1;
}

uint64_t fl_monitor_outstanding(const FlMonitor* m, int dir, int path) {
  Slot* s = slot_of(const_cast<FlMonitor*>(m), dir, path);
  if (!s) return 0;
  const int64_t o = (int64_t)(s->posted.load(std::memory_order_relaxed) - s->completed.load(std::memory_order_relaxed));
  return o > 0 ? (uint64_t)o : 0;
}

double fl_monitor_bandwidth_gbs(const FlMonitor* m, int dir, int path) {
  Slot* s = slot_of(const_cast<FlMonitor*>(m), dir, path);
  return s ? (double)s->bw_milli_gbs.load(std::memory_order_relaxed) / 1000.0 : 0.0;
}

uint64_t fl_monitor_idle_mask(const FlMonitor* m, int dir) {
  uint64_t mask = 0;
  const int n = fl_monitor_num_paths(m);
  for (int p = 0; p < n; ++p)
    if (m->t->slots[dir][p].status.load(std::memory_order_acquire) == FL_PATH_IDLE) mask |= 1ull << p;
  return mask;
}

uint64_t fl_monitor_decisions(const FlMonitor* m) { return m->t->decisions.load(std::memory_order_relaxed); }

int fl_select_paths(FlMonitor* m, const FlSelectorCfg* cfg, int src, int dst, unsigned long long bytes,
                    unsigned long long transfer_index, FlStripe* out, int max_out, uint64_t now_ns) {
  if (max_out < 1) return 0;
  out[0].path = dst;
  out[0].offset = 0;
  out[0].bytes = bytes;
  if (!m || !cfg || !cfg->allow_relay || cfg->degree <= 1 || bytes == 0) return 1;
  const unsigned long long align = cfg->align ? cfg->align : 1;
  const unsigned long long min_stripe = cfg->min_stripe_bytes ? cfg->min_stripe_bytes : align;
  int want = cfg->degree < max_out ? cfg->degree : max_out;
  // never cut stripes smaller than min_stripe
  while (want > 1 && bytes / (unsigned long long)want < min_stripe) --want;
  if (want <= 1) return 1;
  const int n = fl_monitor_num_paths(m);
  const int ppg = (int)m->t->paths_per_group;
  const uint64_t all = n >= 64 ? ~0ull : ((1ull << n) - 1ull);
  uint64_t mask = all & ~(1ull << src) & ~(1ull << dst);
  int relays[FL_MON_MAX_PATHS];
  int nrel = 0;
  // rotate the starting point so consecutive transfers spread over different relays
  int primary = (int)((src + (transfer_index * (unsigned long long)(cfg->step > 0 ? cfg->step : 1))) % (unsigned long long)n);
  for (int i = 0; i < want - 1; ++i) {
    const int p = fl_monitor_borrow_idle(m, FL_DIR_TX, src / ppg, primary, mask, now_ns);
    if (p < 0) break;
    relays[nrel++] = p;
    mask &= ~(1ull << p);
    primary = p;
  }
  if (nrel == 0) return 1;  // nothing idle: the answer is "direct"
  const int parts = nrel + 1;
  unsigned long long per = bytes / (unsigned long long)parts;
  per = per / align * align;
  if (per < min_stripe) {
    for (int i = 0; i < nrel; ++i) fl_monitor_release(m, FL_DIR_TX, relays[i]);
    return 1;
  }
  // relay stripes sit at aligned offsets [i*per, (i+1)*per); the direct stripe takes the tail remainder
  for (int i = 0; i < nrel; ++i) {
    out[i + 1].path = relays[i];
    out[i + 1].offset = per * (unsigned long long)i;
    out[i + 1].bytes = per;
  }
  out[0].offset = per * (unsigned long long)nrel;
  out[0].bytes = bytes - out[0].offset;
  return parts;
}

}  // extern "C"
