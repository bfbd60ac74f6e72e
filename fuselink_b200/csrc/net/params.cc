#include "params.h"

#include <stdlib.h>

#include <map>
#include <mutex>

namespace flnet {
namespace {
std::mutex g_mu;
std::map<std::string, int64_t> g_cache;
Params g_params;
bool g_loaded = false;
}  // namespace

int64_t param_i64(const char* env, int64_t dflt) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_cache.find(env);
  if (it != g_cache.end()) return it->second;
  int64_t v = dflt;
  const char* s = getenv(env);
  if (s && *s) {
    char* end = nullptr;
    long long p = strtoll(s, &end, 0);
    if (end != s) v = p;
  }
  g_cache[env] = v;
  return v;
}

std::string param_str(const char* env, const char* dflt) {
  const char* s = getenv(env);
  return s ? std::string(s) : std::string(dflt);
}

void params_reset_cache() {
  std::lock_guard<std::mutex> l(g_mu);
  g_cache.clear();
  g_loaded = false;
}

void params_reload() {
  params_reset_cache();
  (void)params();
}

const Params& params() {
  if (g_loaded) return g_params;
  Params p;
  p.priority_dev = param_i64("NCCL_FUSELINK_PRIORITY_DEV", 0);
  p.degree = param_i64("NCCL_FUSELINK_DEGREE", 1);
  p.step = param_i64("NCCL_FUSELINK_STEP", 1);
  p.ib_disable = param_i64("NCCL_IB_DISABLE", 0);
  p.ib_gid_index = param_i64("NCCL_IB_GID_INDEX", 0);
  p.ib_timeout = param_i64("NCCL_IB_TIMEOUT", 18);
  p.ib_retry_cnt = param_i64("NCCL_IB_RETRY_CNT", 7);
  p.ib_pkey = param_i64("NCCL_IB_PKEY", 0);
  p.ib_use_inline = param_i64("NCCL_IB_USE_INLINE", 0);
  p.ib_sl = param_i64("NCCL_IB_SL", 0);
  p.ib_tc = param_i64("NCCL_IB_TC", 0);
  p.ib_ar_threshold = param_i64("NCCL_IB_AR_THRESHOLD", 8192);
  p.ib_pci_relaxed_ordering = param_i64("NCCL_IB_PCI_RELAXED_ORDERING", 2);
  p.ib_adaptive_routing = param_i64("NCCL_IB_ADAPTIVE_ROUTING", -2);
  p.ib_merge_vfs = param_i64("NCCL_IB_MERGE_VFS", 1);
  p.ib_qps_per_conn = param_i64("NCCL_IB_QPS_PER_CONNECTION", 1);
  p.ib_split_data_on_qps = param_i64("NCCL_IB_SPLIT_DATA_ON_QPS", 1);
  p.gdr_flush_disable = param_i64("NCCL_GDR_FLUSH_DISABLE", 1);
  p.buffsize = param_i64("NCCL_BUFFSIZE", -2);
  p.chunk_size = param_i64("NCCL_P2P_NET_CHUNKSIZE", 524288);
  p.ib_hca = param_str("NCCL_IB_HCA", "");
  p.socket_ifname = param_str("NCCL_SOCKET_IFNAME", "");
  p.socket_family = param_str("NCCL_SOCKET_FAMILY", "");
  p.tcp_ndev = param_i64("FUSELINK_TCP_NDEV", 4);
  p.monitor_enable = param_i64("FUSELINK_MONITOR", 1);
  p.monitor_shm = param_str("FUSELINK_MONITOR_SHM", "");
  p.monitor_timeout_us = param_i64("FUSELINK_MONITOR_TIMEOUT_US", 160);
  p.min_stripe_bytes = param_i64("FUSELINK_MIN_STRIPE_BYTES", 65536);
  p.net_timeout_ms = param_i64("FUSELINK_NET_TIMEOUT_MS", 30000);
  p.timers = param_i64("FUSELINK_TIMERS", 0);
  p.cuda_ptrs = param_i64("FUSELINK_CUDA_PTRS", 0);
  p.vmm_fake = param_i64("FUSELINK_VMM_FAKE", 0);
  p.nvl = param_i64("FUSELINK_NVL", 1);
  p.remap = param_i64("FUSELINK_REMAP", 1);
  p.nic_mbps = param_i64("FUSELINK_TCP_NIC_MBPS", 0);
  p.nic_shm = param_str("FUSELINK_TCP_NIC_SHM", "");
  p.connect_retries = param_i64("FUSELINK_CONNECT_RETRIES", 20000);
  p.failover = param_i64("FUSELINK_FAILOVER", 1);
  p.fault_bad_rkey_after = param_i64("FUSELINK_FAULT_BAD_RKEY_AFTER", 0);
  p.fault_drop_after = param_i64("FUSELINK_FAULT_CLOSE_AFTER_BYTES", 0);
  if (p.tcp_ndev < 1) p.tcp_ndev = 1;
  if (p.tcp_ndev > 16) p.tcp_ndev = 16;
  if (p.degree < 1) p.degree = 1;
  g_params = p;
  g_loaded = true;
  return g_params;
}

}  // namespace flnet
