// NCCL_IB_HCA filter of the verbs path, with the syntax of the reference (src/plugin.cc:194-230): a comma list of
// device-name prefixes, a leading '^' excludes, a leading '=' matches exactly, "name:port" selects one port, and bare
// numbers continue the previous prefix ("=mlx5_0,3,4" names mlx5_0, mlx5_3 and mlx5_4, as the reference's bandwidth
// script writes it).  Device discovery itself and the queue-pair data path are in verbs_provider.cc and
// rdma_transport.cc; the filter is separate so that it can be tested without a NIC.
#pragma once
#include <stdint.h>
#include <string>
#include <vector>

namespace flnet {

struct HcaFilter {
  bool exclude = false, exact = false;
  std::vector<std::pair<std::string, int>> entries;   // (name prefix, port or -1)
};
HcaFilter parse_hca_filter(const std::string& spec);
bool hca_allowed(const HcaFilter& f, const std::string& name, int port);

}  // namespace flnet

extern "C" int fuselink_hca_allowed(const char* spec, const char* name, int port);
