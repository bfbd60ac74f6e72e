// Optional verbs (RDMA) side of the plugin.  libibverbs is opened at run time (the reference does the same
// through NCCL's ibvsymbols, src/extern/ibvwrap.h:30-90, src/plugin.cc:177) so the plugin loads on machines
// without RDMA.  What is here: device discovery with the NCCL_IB_HCA filter syntax of the reference
// (src/plugin.cc:194-230: leading '^' excludes, leading '=' matches exactly, "name:port" selects a port)
// and the per-device record the connection manager needs.  A queue-pair data path needs RDMA hardware to
// be exercised; on a box without NICs discovery returns 0 devices and the TCP transport carries the data.
#pragma once
#include <stdint.h>
#include <string>
#include <vector>

namespace flnet {

struct IbDevice {
  std::string name;
  int port;
  uint64_t guid;
  std::string pci_path;
};

// Number of usable verbs devices (0 when libibverbs or devices are missing).
int ib_discover();
const std::vector<IbDevice>& ib_devices();

// Filter evaluation, separated from discovery so it can be tested anywhere.
struct HcaFilter {
  bool exclude = false, exact = false;
  std::vector<std::pair<std::string, int>> entries;   // (name prefix, port or -1)
};
HcaFilter parse_hca_filter(const std::string& spec);
bool hca_allowed(const HcaFilter& f, const std::string& name, int port);

}  // namespace flnet

extern "C" int fuselink_hca_allowed(const char* spec, const char* name, int port);
