#include "conn_manager.h"
#include <unistd.h>

#include "logging.h"
#include "params.h"

namespace flnet {

ConnManager::ConnManager(int ndev, int priority_dev, bool use_monitor, const char* shm_name, int timeout_us)
    : ndev_(ndev), priority_dev_(priority_dev) {
  for (auto& dir : own_out_)
    for (auto& v : dir) v.store(0, std::memory_order_relaxed);
  prefer_own_ = param_i64("FUSELINK_PREFER_OWN", 1) != 0;
  owner_id_ = 0x40000000 | (int)(getpid() & 0x3fffffff);    // never equal to a group index
  if (use_monitor && ndev > 0) {
    const bool shared = shm_name && shm_name[0];
    if (shared) mon_ = fl_monitor_open(shm_name, 0, ndev, 1, timeout_us);      // a daemon owns the table
    if (!mon_) {
      mon_ = fl_monitor_open(shared ? shm_name : "", 1, ndev, 1, timeout_us);  // own it ourselves
      if (mon_) fl_monitor_start(mon_, timeout_us / 4 > 0 ? timeout_us / 4 : 40);
    }
    if (!mon_) FL_WARN("monitor unavailable (%s); falling back to channel-modulo path selection", fl_monitor_last_error());
  }
}

ConnManager::~ConnManager() {
  if (mon_) fl_monitor_close(mon_, 0);
}

int ConnManager::refresh_rx(int channel, int own_dev, int current, uint64_t tx_mask, bool quiescent) {
  if (ndev_ <= 1) return own_dev;
  if (!quiescent && current >= 0) return current;
  if (!mon_) {
    decisions_++;
    return channel % ndev_;   // the reference's shipped rule ("packet spraying", src/fuselink.h:230-237)
  }
  const uint64_t now = fl_monitor_now_ns();
  if (current >= 0 && current != own_dev) fl_monitor_release(mon_, FL_DIR_RX, current);
  if (prefer_own_ && own_dev >= 0 && own_dev < 64 && fl_monitor_claim(mon_, FL_DIR_RX, own_dev, owner_id_, now)) {
    decisions_++;
    return own_dev;             // nobody else is on the affine device: it is now held by this process (one atomic claim,
  }                             // so two jobs that start together cannot both conclude that it is free)
  const int p = fl_monitor_borrow_idle(mon_, FL_DIR_RX, own_dev, own_dev + channel, tx_mask, now);
  decisions_++;
  if (p < 0) {
    fallbacks_++;
    return own_dev;           // nothing idle: stay on the own device
  }
  return p;
}

int ConnManager::bid_tx(int channel, int own_dev, int proposed) {
  (void)channel;
  if (proposed < 0 || proposed >= ndev_) return own_dev;
  if (proposed == own_dev || !mon_) return proposed;
  const int st = fl_monitor_status(mon_, FL_DIR_TX, proposed);
  if (st == FL_PATH_DEAD) {
    fallbacks_++;
    return own_dev;
  }
  return proposed;
}

int ConnManager::borrow_tx(int own_dev, uint64_t used_mask, int after) {
  if (!mon_ || ndev_ <= 1) return -1;
  const int p = fl_monitor_borrow_idle(mon_, FL_DIR_TX, own_dev, after, ~used_mask, fl_monitor_now_ns());
  if (p >= 0) decisions_++;
  return p >= ndev_ ? -1 : p;
}

void ConnManager::release_tx(int dev) {
  if (mon_ && dev >= 0) fl_monitor_release(mon_, FL_DIR_TX, dev);
}

void ConnManager::mark_tx(int dev, uint64_t bytes) {
  if (!mon_) return;
  if (dev >= 0 && dev < 64) own_out_[FL_DIR_TX][dev].fetch_add((int64_t)bytes, std::memory_order_relaxed);
  fl_monitor_post_bytes(mon_, FL_DIR_TX, dev, bytes, fl_monitor_now_ns());
}
void ConnManager::done_tx(int dev, uint64_t bytes) {
  if (!mon_) return;
  if (dev >= 0 && dev < 64) own_out_[FL_DIR_TX][dev].fetch_sub((int64_t)bytes, std::memory_order_relaxed);
  fl_monitor_complete_bytes(mon_, FL_DIR_TX, dev, bytes, fl_monitor_now_ns());
}
void ConnManager::touch_rx(int dev) {
  if (mon_) fl_monitor_mark_active(mon_, FL_DIR_RX, dev, fl_monitor_now_ns());
}
void ConnManager::mark_rx(int dev, uint64_t bytes) {
  if (!mon_) return;
  if (dev >= 0 && dev < 64) own_out_[FL_DIR_RX][dev].fetch_add((int64_t)bytes, std::memory_order_relaxed);
  fl_monitor_post_bytes(mon_, FL_DIR_RX, dev, bytes, fl_monitor_now_ns());
}
void ConnManager::done_rx(int dev, uint64_t bytes) {
  if (!mon_) return;
  if (dev >= 0 && dev < 64) own_out_[FL_DIR_RX][dev].fetch_sub((int64_t)bytes, std::memory_order_relaxed);
  fl_monitor_complete_bytes(mon_, FL_DIR_RX, dev, bytes, fl_monitor_now_ns());
}

uint64_t ConnManager::tx_mask(int own_dev) {
  if (!mon_) return ~0ull;    // the reference's placeholder value (src/fuselink.h:261-267)
  uint64_t m = fl_monitor_idle_mask(mon_, FL_DIR_TX);
  if (own_dev >= 0 && own_dev < 64) m |= 1ull << own_dev;
  for (int d = 0; d < ndev_ && d < 64; ++d)
    if (fl_monitor_status(mon_, FL_DIR_TX, d) == FL_PATH_DEAD) m &= ~(1ull << d);
  return m;
}

void ConnManager::set_dead(int dev, bool dead) {
  if (mon_) {
    fl_monitor_mark_dead(mon_, FL_DIR_TX, dev, dead);
    fl_monitor_mark_dead(mon_, FL_DIR_RX, dev, dead);
  }
}

}  // namespace flnet
