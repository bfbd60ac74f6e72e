#include "nic_rate.h"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <string>

#include "logging.h"
#include "params.h"
#include "tcp_transport.h"

namespace flnet {
namespace {
struct NicBucket {
  std::atomic<uint32_t> lock;     // spin lock (the buckets may live in memory shared between processes)
  uint32_t pad;
  double tokens;                  // bytes that may be sent now
  uint64_t last_ns;
};
NicBucket g_local_nic[kMaxDev];
NicBucket* g_nic = nullptr;

NicBucket* nic_buckets() {
  static std::once_flag once;
  std::call_once(once, [] {
    g_nic = g_local_nic;
    const std::string name = params().nic_shm;
    if (name.empty()) return;
    // one set of buckets for every process that names the segment: several jobs then really share the "NICs"
    int fd = shm_open(name.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, sizeof(NicBucket) * kMaxDev) != 0) {
      FL_WARN("FUSELINK_TCP_NIC_SHM=%s cannot be opened (%s): line rates are per process", name.c_str(), strerror(errno));
      if (fd >= 0) close(fd);
      return;
    }
    void* p = mmap(nullptr, sizeof(NicBucket) * kMaxDev, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);   // fresh segments are zero
    close(fd);
    if (p != MAP_FAILED) g_nic = reinterpret_cast<NicBucket*>(p);
  });
  return g_nic;
}

}  // namespace

size_t nic_allowance(int dev, size_t want) {
  const int64_t mbps = params().nic_mbps;
  if (mbps <= 0) return want;
  NicBucket& b = nic_buckets()[dev];
  uint32_t expect = 0;
  int spins = 0;
  while (!b.lock.compare_exchange_weak(expect, 1, std::memory_order_acquire)) {
    expect = 0;
    if (++spins > 100000) return 0;                            // a holder died: give up for now, never hang
  }
  const uint64_t now = now_ns();
  const double rate = (double)mbps * 1e6;                      // bytes per second
  if (b.last_ns == 0 || now < b.last_ns) b.last_ns = now;
  b.tokens += rate * (double)(now - b.last_ns) * 1e-9;
  b.last_ns = now;
  const double burst = rate * 2e-3;                            // at most 2 ms worth of line rate in one go
  if (b.tokens > burst) b.tokens = burst;
  const size_t ok = b.tokens < 1.0 ? 0 : (size_t)b.tokens < want ? (size_t)b.tokens : want;
  b.tokens -= (double)ok;
  b.lock.store(0, std::memory_order_release);
  return ok;
}

}  // namespace flnet
