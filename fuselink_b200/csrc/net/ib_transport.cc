#include "ib_transport.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "logging.h"
#include "params.h"

namespace flnet {
namespace {
std::vector<IbDevice> g_devs;

// The two verbs structures whose leading fields are read here.  Layout prefix of rdma-core's public
// `struct ibv_device` (ops table of two pointers, two enums, then the fixed-size name arrays).
struct ibv_device_prefix {
  void* ops[2];
  int node_type;
  int transport_type;
  char name[64];
  char dev_name[64];
  char dev_path[256];
  char ibdev_path[256];
};
}  // namespace

HcaFilter parse_hca_filter(const std::string& spec_in) {
  HcaFilter f;
  std::string spec = spec_in;
  if (!spec.empty() && spec[0] == '^') { f.exclude = true; spec = spec.substr(1); }
  if (!spec.empty() && spec[0] == '=') { f.exact = true; spec = spec.substr(1); }
  size_t pos = 0;
  std::string last_prefix;
  while (pos < spec.size()) {
    size_t c = spec.find(',', pos);
    if (c == std::string::npos) c = spec.size();
    std::string item = spec.substr(pos, c - pos);
    pos = c + 1;
    if (item.empty()) continue;
    int port = -1;
    size_t colon = item.find(':');
    if (colon != std::string::npos) {
      port = atoi(item.c_str() + colon + 1);
      item = item.substr(0, colon);
    }
    // "mlx5_0,3,4" style lists (as in the reference's bandwidth script) mean mlx5_0, mlx5_3, mlx5_4
    bool digits = !item.empty();
    for (char ch : item) if (ch < '0' || ch > '9') digits = false;
    if (digits && !last_prefix.empty()) item = last_prefix + item;
    else {
      size_t us = item.rfind('_');
      if (us != std::string::npos) last_prefix = item.substr(0, us + 1);
    }
    f.entries.emplace_back(item, port);
  }
  return f;
}

bool hca_allowed(const HcaFilter& f, const std::string& name, int port) {
  if (f.entries.empty()) return true;
  bool match = false;
  for (auto& e : f.entries) {
    const bool name_ok = f.exact ? (name == e.first) : (name.compare(0, e.first.size(), e.first) == 0);
    if (name_ok && (e.second < 0 || e.second == port)) match = true;
  }
  return f.exclude ? !match : match;
}

const std::vector<IbDevice>& ib_devices() { return g_devs; }

int ib_discover() {
  g_devs.clear();
  void* lib = dlopen("libibverbs.so.1", RTLD_NOW);
  if (!lib) lib = dlopen("libibverbs.so", RTLD_NOW);
  if (!lib) {
    FL_INFO("libibverbs not found: verbs path disabled");
    return 0;
  }
  using get_list_t = void** (*)(int*);
  using free_list_t = void (*)(void**);
  auto get_list = reinterpret_cast<get_list_t>(dlsym(lib, "ibv_get_device_list"));
  auto free_list = reinterpret_cast<free_list_t>(dlsym(lib, "ibv_free_device_list"));
  if (!get_list || !free_list) return 0;
  int n = 0;
  void** list = get_list(&n);
  if (!list) return 0;
  const HcaFilter f = parse_hca_filter(params().ib_hca);
  for (int i = 0; i < n; ++i) {
    const ibv_device_prefix* d = reinterpret_cast<const ibv_device_prefix*>(list[i]);
    std::string name(d->name, strnlen(d->name, sizeof d->name));
    if (!hca_allowed(f, name, 1)) continue;
    IbDevice dev;
    dev.name = name;
    dev.port = 1;
    dev.guid = 0;
    dev.pci_path = std::string(d->ibdev_path, strnlen(d->ibdev_path, sizeof d->ibdev_path));
    g_devs.push_back(dev);
  }
  free_list(list);
  FL_INFO("verbs: %d device(s) after NCCL_IB_HCA filter", (int)g_devs.size());
  return (int)g_devs.size();
}

}  // namespace flnet

extern "C" __attribute__((visibility("default"))) int fuselink_hca_allowed(const char* spec, const char* name, int port) {
  return flnet::hca_allowed(flnet::parse_hca_filter(spec ? spec : ""), name ? name : "", port) ? 1 : 0;
}
