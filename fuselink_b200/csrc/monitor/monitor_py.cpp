// pybind11 surface of the monitor / selector (kept apart from monitor.cc so the ncclNet plugin can link
// the monitor without Python).
#include <torch/extension.h>
#include "monitor.h"

namespace py = pybind11;

static FlMonitor* M(int64_t h) { return reinterpret_cast<FlMonitor*>(h); }

void fl_monitor_bind(py::module& m) {
  m.def("monitor_open", [](const std::string& name, bool owner, int64_t groups, int64_t ppg, int64_t timeout_us) {
    FlMonitor* h = fl_monitor_open(name.c_str(), owner, (int)groups, (int)ppg, (int)timeout_us);
    if (!h) throw std::runtime_error(std::string("fl_monitor_open: ") + fl_monitor_last_error());
    return reinterpret_cast<int64_t>(h);
  });
  m.def("monitor_close", [](int64_t h, bool unlink_shm) { fl_monitor_close(M(h), unlink_shm); });
  m.def("monitor_num_paths", [](int64_t h) { return fl_monitor_num_paths(M(h)); });
  m.def("monitor_timeout_us", [](int64_t h) { return fl_monitor_timeout_us(M(h)); });
  m.def("monitor_start", [](int64_t h, int64_t period_us) { return fl_monitor_start(M(h), (int)period_us); });
  m.def("monitor_stop", [](int64_t h) { fl_monitor_stop(M(h)); });
  m.def("monitor_sweep", [](int64_t h, uint64_t now) { fl_monitor_sweep(M(h), now); });
  m.def("monitor_now_ns", []() { return fl_monitor_now_ns(); });
  m.def("monitor_mark_active", [](int64_t h, int64_t d, int64_t p, uint64_t now) { fl_monitor_mark_active(M(h), (int)d, (int)p, now); });
  m.def("monitor_post_bytes", [](int64_t h, int64_t d, int64_t p, uint64_t b, uint64_t now) { fl_monitor_post_bytes(M(h), (int)d, (int)p, b, now); });
  m.def("monitor_complete_bytes", [](int64_t h, int64_t d, int64_t p, uint64_t b, uint64_t now) { fl_monitor_complete_bytes(M(h), (int)d, (int)p, b, now); });
  m.def("monitor_attach_counters", [](int64_t h, int64_t d, int64_t ptr) {
    fl_monitor_attach_counters(M(h), (int)d, reinterpret_cast<const volatile uint64_t*>(ptr));
  });
  m.def("monitor_borrow_idle", [](int64_t h, int64_t d, int64_t group, int64_t primary, uint64_t mask, uint64_t now) {
    return fl_monitor_borrow_idle(M(h), (int)d, (int)group, (int)primary, mask, now);
  });
  m.def("monitor_claim", [](int64_t h, int64_t d, int64_t p, int64_t owner, uint64_t now) { return fl_monitor_claim(M(h), (int)d, (int)p, (int)owner, now); });
  m.def("monitor_release", [](int64_t h, int64_t d, int64_t p) { fl_monitor_release(M(h), (int)d, (int)p); });
  m.def("monitor_mark_dead", [](int64_t h, int64_t d, int64_t p, bool dead) { fl_monitor_mark_dead(M(h), (int)d, (int)p, dead); });
  m.def("monitor_status", [](int64_t h, int64_t d, int64_t p) { return fl_monitor_status(M(h), (int)d, (int)p); });
  m.def("monitor_outstanding", [](int64_t h, int64_t d, int64_t p) { return fl_monitor_outstanding(M(h), (int)d, (int)p); });
  m.def("monitor_bandwidth_gbs", [](int64_t h, int64_t d, int64_t p) { return fl_monitor_bandwidth_gbs(M(h), (int)d, (int)p); });
  m.def("monitor_idle_mask", [](int64_t h, int64_t d) { return fl_monitor_idle_mask(M(h), (int)d); });
  m.def("monitor_decisions", [](int64_t h) { return fl_monitor_decisions(M(h)); });
  m.def("select_paths", [](int64_t h, int64_t degree, int64_t step, uint64_t min_stripe, uint64_t align, bool allow_relay,
                           int64_t src, int64_t dst, uint64_t bytes, uint64_t index, uint64_t now) {
    FlSelectorCfg cfg;
    cfg.degree = (int)degree; cfg.step = (int)step; cfg.min_stripe_bytes = min_stripe; cfg.align = align;
    cfg.allow_relay = allow_relay;
    FlStripe out[FL_MON_MAX_PATHS];
    int n = fl_select_paths(M(h), &cfg, (int)src, (int)dst, bytes, index, out, FL_MON_MAX_PATHS, now);
    std::vector<std::tuple<int, uint64_t, uint64_t>> res;
    for (int i = 0; i < n; ++i) res.emplace_back(out[i].path, (uint64_t)out[i].offset, (uint64_t)out[i].bytes);
    return res;
  });
}
