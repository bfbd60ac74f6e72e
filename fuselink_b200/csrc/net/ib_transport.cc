#include "ib_transport.h"

#include <stdlib.h>
#include <string.h>

#include "logging.h"
#include "params.h"

namespace flnet {
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

}  // namespace flnet

extern "C" __attribute__((visibility("default"))) int fuselink_hca_allowed(const char* spec, const char* name, int port) {
  return flnet::hca_allowed(flnet::parse_hca_filter(spec ? spec : ""), name ? name : "", port) ? 1 : 0;
}
