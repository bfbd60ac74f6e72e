// Environment knobs of the plugin.  Same names and defaults as the reference's NCCL_PARAM uses
// (src/plugin.cc:87-117,584,887,1410; src/extern/param.h:19-28): NCCL_<NAME>, read once and cached.
// FUSELINK_* names are additions of this project.
#pragma once
#include <stdint.h>
#include <string>

namespace flnet {

int64_t param_i64(const char* env, int64_t dflt);     // cached per name
std::string param_str(const char* env, const char* dflt);
void params_reset_cache();                             // tests change the environment between cases

struct Params {
  int64_t priority_dev;        // NCCL_FUSELINK_PRIORITY_DEV (0)
  int64_t degree;              // NCCL_FUSELINK_DEGREE (1): paths one message may be striped over
  int64_t step;                // NCCL_FUSELINK_STEP (1): rotation between consecutive selections
  int64_t ib_disable;          // NCCL_IB_DISABLE (0)
  int64_t ib_gid_index, ib_timeout, ib_retry_cnt, ib_pkey, ib_use_inline, ib_sl, ib_tc;
  int64_t ib_ar_threshold;     // NCCL_IB_AR_THRESHOLD (8192)
  int64_t ib_pci_relaxed_ordering, ib_adaptive_routing, ib_merge_vfs, ib_qps_per_conn, ib_split_data_on_qps;
  int64_t gdr_flush_disable;   // NCCL_GDR_FLUSH_DISABLE (1, as the reference sets it)
  int64_t buffsize;            // NCCL_BUFFSIZE
  int64_t chunk_size;          // NCCL_P2P_NET_CHUNKSIZE (524288)
  std::string ib_hca;          // NCCL_IB_HCA
  std::string socket_ifname;   // NCCL_SOCKET_IFNAME
  std::string socket_family;   // NCCL_SOCKET_FAMILY
  // additions
  int64_t tcp_ndev;            // FUSELINK_TCP_NDEV (4): virtual NICs the TCP transport exposes
  int64_t monitor_enable;      // FUSELINK_MONITOR (1)
  std::string monitor_shm;     // FUSELINK_MONITOR_SHM ("" = private table)
  int64_t monitor_timeout_us;  // FUSELINK_MONITOR_TIMEOUT_US (160)
  int64_t min_stripe_bytes;    // FUSELINK_MIN_STRIPE_BYTES (65536)
  int64_t net_timeout_ms;      // FUSELINK_NET_TIMEOUT_MS (30000): a request with no progress for this long fails
  int64_t timers;              // FUSELINK_TIMERS (0): print per-phase timers at close
  int64_t cuda_ptrs;           // FUSELINK_CUDA_PTRS (0): accept NCCL_PTR_CUDA registrations (cuMem adopt + relay remap + staging)
  int64_t vmm_fake;            // FUSELINK_VMM_FAKE (0): memfd-backed stand-in for the CUDA driver (CPU tests)
  int64_t nvl;                 // FUSELINK_NVL (1): same-host direct path, receive buffers exported as cuMem handles
  int64_t remap;               // FUSELINK_REMAP (1): re-home a registered CUDA buffer onto the relay GPU
  int64_t nic_mbps;            // FUSELINK_TCP_NIC_MBPS (0 = unlimited): line rate of every virtual NIC in MB/s, per process (experiments)
  std::string nic_shm;         // FUSELINK_TCP_NIC_SHM (""): POSIX shm name; with it the line-rate buckets are shared by every process that names it
  int64_t connect_retries;     // FUSELINK_CONNECT_RETRIES (20000): refused connects are retried this many times, 1 ms apart (the reference's budget, src/extern/socket.h:15-17)
  int64_t failover;            // FUSELINK_FAILOVER (1): a broken data socket's stripes are re-sent on another device instead of failing the connection
  int64_t fault_bad_rkey_after; // FUSELINK_FAULT_BAD_RKEY_AFTER (0): test hook, the Nth RDMA message carries a wrong remote key
  int64_t fault_drop_after;    // FUSELINK_FAULT_CLOSE_AFTER_BYTES (0): test hook, sender closes a data socket mid-stream
};
const Params& params();
void params_reload();

}  // namespace flnet
