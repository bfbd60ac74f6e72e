// Path / NIC selection for the plugin: which device carries the next message of a channel.
//
// Reference: class FuseLinkConnManager (src/fuselink.h:68-314).  Intended behaviour there (most of it is
// stubbed in the shipped code): the receiver periodically asks the idleness monitor for an idle NIC of
// another group (refreshRxComm, :190-244), tells the sender through the receive descriptor, and the
// sender "bids" for that NIC, falling back to its own when the bid fails (bidTxChannel, :153-161,
// src/plugin.cc:1538-1547); the sender's availability mask travels back with the data
// (src/plugin.cc:1441-1451).  The only rule live in the shipped code is dev = channelId % nNics.
// This class implements the intended rules on top of the lock-free monitor, and keeps the channel-modulo
// rule as the fallback when the monitor is off.
#pragma once
#include <stdint.h>

#include <atomic>

#include "../monitor/monitor.h"

namespace flnet {

class ConnManager {
 public:
  ConnManager(int ndev, int priority_dev, bool use_monitor, const char* shm_name, int timeout_us);
  ~ConnManager();
  int ndev() const { return ndev_; }
  int priority_dev() const { return priority_dev_; }
  FlMonitor* monitor() { return mon_; }

  // Receiver side: device that should carry the next message of `channel`.  The own (affine) device is kept while the
  // shared table shows no load on it besides this process's own; otherwise an idle device of another group is borrowed
  // (the reference's intended getIdleNicRx, src/fuselink.h:239-243).  FUSELINK_PREFER_OWN=0 always tries to borrow first.  `current` is the device in
  // use (or -1); `tx_mask` is the sender's last advertised availability mask.  A new device is looked for
  // only when `quiescent` (nothing posted is still incomplete), as the reference does every 8 completions
  // when received == done (src/plugin.cc:1700-1716).
  int refresh_rx(int channel, int own_dev, int current, uint64_t tx_mask, bool quiescent);
  // Sender side: accept the receiver's proposal if that device is usable for tx, else fall back to own_dev.
  int bid_tx(int channel, int own_dev, int proposed);
  // Sender side, stripes after the first: an idle device (tx direction) outside `used_mask`, borrowed from the monitor;
  // -1 when the monitor is off or nothing is idle (the caller then walks on by NCCL_FUSELINK_STEP).  `release_tx` gives it back.
  int borrow_tx(int own_dev, uint64_t used_mask, int after);
  void release_tx(int dev);
  // Activity stamps (the "todo: update nic activities" of src/plugin.cc:1812).
  void mark_tx(int dev, uint64_t bytes_posted);
  void done_tx(int dev, uint64_t bytes);
  void mark_rx(int dev, uint64_t bytes_posted);
  void touch_rx(int dev);                    // a receive was posted with this device proposed: activity stamp only
  void done_rx(int dev, uint64_t bytes);
  // 64-bit mask of devices this process considers available for tx (bit set = idle or own)
  uint64_t tx_mask(int own_dev);
  void set_dead(int dev, bool dead);
  uint64_t decisions() const { return decisions_.load(std::memory_order_relaxed); }
  uint64_t fallbacks() const { return fallbacks_.load(std::memory_order_relaxed); }

 private:
  int ndev_, priority_dev_;
  FlMonitor* mon_ = nullptr;
  std::atomic<uint64_t> decisions_{0}, fallbacks_{0};   // entered from every proxy thread
  std::atomic<int64_t> own_out_[2][64];                // bytes this process has posted and not completed, per direction and device
  int owner_id_ = 0;                                    // identifies this process in the shared table
  bool prefer_own_ = true;                              // FUSELINK_PREFER_OWN (1): stay on the own device while nobody else loads it
};

}  // namespace flnet
