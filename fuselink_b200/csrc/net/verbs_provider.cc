// The NIC interface over libibverbs, opened at run time.  Discovery follows the reference's init
// (src/plugin.cc:174-310): every active IB / RoCE port that passes the NCCL_IB_HCA filter becomes a device, with
// its speed from the width and rate tables, its PCI path (virtual functions and ports of one adapter merged when
// NCCL_IB_MERGE_VFS is set), and a protection domain allocated up front.  Queue pairs are reliable-connected and
// walk INIT -> RTR -> RTS with the NCCL_IB_* attributes (src/plugin.cc:626-688).
//
// No machine this project is tested on has RDMA hardware: this file is compiled and loaded everywhere, and
// reports zero devices there.  The transport above it is exercised through the software NIC.
#include <dlfcn.h>
#include <errno.h>
#include <limits.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <mutex>
#include <vector>

#include "ib_transport.h"
#include "logging.h"
#include "params.h"
#include "rdma_provider.h"
#include "verbs_abi.h"

namespace flnet {
namespace rdma {
namespace {
using namespace verbs_abi;

struct Lib {
  void* handle = nullptr;
  void** (*get_device_list)(int*) = nullptr;
  void (*free_device_list)(void**) = nullptr;
  const char* (*get_device_name)(void*) = nullptr;
  uint64_t (*get_device_guid)(void*) = nullptr;
  ibv_context* (*open_device)(void*) = nullptr;
  int (*close_device)(ibv_context*) = nullptr;
  int (*query_device)(ibv_context*, ibv_device_attr*) = nullptr;
  int (*query_port)(ibv_context*, uint8_t, ibv_port_attr*) = nullptr;
  int (*query_gid)(ibv_context*, uint8_t, int, ibv_gid*) = nullptr;
  ibv_pd* (*alloc_pd)(ibv_context*) = nullptr;
  int (*dealloc_pd)(ibv_pd*) = nullptr;
  ibv_mr* (*reg_mr)(ibv_pd*, void*, size_t, int) = nullptr;
  ibv_mr* (*reg_mr_iova2)(ibv_pd*, void*, size_t, uint64_t, unsigned int) = nullptr;   // newer libraries only
  ibv_mr* (*reg_dmabuf_mr)(ibv_pd*, uint64_t, size_t, uint64_t, int, int) = nullptr;    // offset, length, iova, fd, access
  int (*dereg_mr)(ibv_mr*) = nullptr;
  ibv_cq* (*create_cq)(ibv_context*, int, void*, void*, int) = nullptr;
  int (*destroy_cq)(ibv_cq*) = nullptr;
  ibv_qp* (*create_qp)(ibv_pd*, ibv_qp_init_attr*) = nullptr;
  int (*modify_qp)(ibv_qp*, ibv_qp_attr*, int) = nullptr;
  int (*destroy_qp)(ibv_qp*) = nullptr;
  int (*query_ece)(ibv_qp*, ibv_ece*) = nullptr;      // newer libraries only
  int (*set_ece)(ibv_qp*, ibv_ece*) = nullptr;
  int (*get_async_event)(ibv_context*, ibv_async_event*) = nullptr;
  void (*ack_async_event)(ibv_async_event*) = nullptr;
  const char* (*event_type_str)(int) = nullptr;
};

template <class F>
bool sym(void* h, const char* name, F* out, bool required = true) {
  *out = reinterpret_cast<F>(dlsym(h, name));
  return *out != nullptr || !required;
}

// Mb/s of one lane for the verbs "active_speed" code, and lanes for the "active_width" code.
int lane_mbps(int code) {
  switch (code) {
    case 1: return 2500;     // SDR
    case 2: return 5000;     // DDR
    case 4: return 10000;    // QDR
    case 8: return 10000;    // FDR10
    case 16: return 14000;   // FDR
    case 32: return 25000;   // EDR
    case 64: return 50000;   // HDR
    case 128: return 100000; // NDR
    default: return 2500;
  }
}
int lanes(int code) {
  switch (code) {
    case 1: return 1;
    case 2: return 4;
    case 4: return 8;
    case 8: return 12;
    case 16: return 2;
    default: return 1;
  }
}

struct Port {
  DeviceInfo info;
  ibv_context* ctx = nullptr;
  int active_mtu = 3;
  uint16_t lid = 0;
};

struct VPd { int dev; ibv_pd* pd; };
struct VCq { int dev; ibv_cq* cq; };
struct VQp { int dev; ibv_qp* qp; };

class VerbsProvider : public Provider {
 public:
  VerbsProvider() { discover(); }
  const char* name() const override { return "verbs"; }
  int device_count() override { return (int)ports_.size(); }
  DeviceInfo device(int dev) override { return ports_[dev].info; }

  Pd* alloc_pd(int dev) override {
    ibv_pd* pd = lib_.alloc_pd(ports_[dev].ctx);
    return pd ? reinterpret_cast<Pd*>(new VPd{dev, pd}) : nullptr;
  }
  void dealloc_pd(Pd* h) override {
    VPd* p = reinterpret_cast<VPd*>(h);
    if (!p) return;
    lib_.dealloc_pd(p->pd);
    delete p;
  }
  Mr* reg_mr(Pd* h, void* addr, size_t len, int access) override {
    VPd* p = reinterpret_cast<VPd*>(h);
    int flags = 0;
    if (access & kAccessLocalWrite) flags |= IBV_ACCESS_LOCAL_WRITE;
    if (access & kAccessRemoteWrite) flags |= IBV_ACCESS_REMOTE_WRITE;
    if (access & kAccessRemoteRead) flags |= IBV_ACCESS_REMOTE_READ;
    ibv_mr* mr = nullptr;
    if ((access & kAccessRelaxedOrdering) && lib_.reg_mr_iova2)
      mr = lib_.reg_mr_iova2(p->pd, addr, len, (uint64_t)(uintptr_t)addr, (unsigned)(flags | IBV_ACCESS_RELAXED_ORDERING));
    else
      mr = lib_.reg_mr(p->pd, addr, len, flags);
    if (!mr) return nullptr;
    Mr* m = new Mr();
    m->lkey = mr->lkey;
    m->rkey = mr->rkey;
    m->addr = addr;
    m->len = len;
    m->impl = mr;
    return m;
  }
  Mr* reg_dmabuf_mr(Pd* h, int fd, uint64_t offset, size_t len, uint64_t iova, int access) override {
    VPd* p = reinterpret_cast<VPd*>(h);
    if (!lib_.reg_dmabuf_mr) return nullptr;
    int flags = 0;
    if (access & kAccessLocalWrite) flags |= IBV_ACCESS_LOCAL_WRITE;
    if (access & kAccessRemoteWrite) flags |= IBV_ACCESS_REMOTE_WRITE;
    if (access & kAccessRemoteRead) flags |= IBV_ACCESS_REMOTE_READ;
    if (access & kAccessRelaxedOrdering) flags |= IBV_ACCESS_RELAXED_ORDERING;
    ibv_mr* mr = lib_.reg_dmabuf_mr(p->pd, offset, len, iova, fd, flags);
    if (!mr) return nullptr;
    Mr* m = new Mr();
    m->lkey = mr->lkey;
    m->rkey = mr->rkey;
    m->addr = reinterpret_cast<void*>(iova);
    m->len = len;
    m->impl = mr;
    return m;
  }
  // The kernel side is probed with a registration that cannot succeed (no descriptor): a kernel or device without
  // dma-buf support answers "not supported", one with it answers "bad descriptor" (src/plugin.cc:337-356).
  bool dmabuf_supported(int dev) override {
    if (!lib_.reg_dmabuf_mr || dev < 0 || dev >= (int)ports_.size()) return false;
    std::lock_guard<std::mutex> l(probe_mu_);
    if (dmabuf_probe_.size() < ports_.size()) dmabuf_probe_.resize(ports_.size(), -1);
    if (dmabuf_probe_[dev] < 0) {
      ibv_pd* pd = lib_.alloc_pd(ports_[dev].ctx);
      int ok = 0;
      if (pd) {
        errno = 0;
        ibv_mr* mr = lib_.reg_dmabuf_mr(pd, 0, 0, 0, -1, 0);
        if (mr) lib_.dereg_mr(mr);
        ok = errno != EOPNOTSUPP && errno != EPROTONOSUPPORT;
        lib_.dealloc_pd(pd);
      }
      dmabuf_probe_[dev] = ok;
    }
    return dmabuf_probe_[dev] == 1;
  }
  // A peer-memory module lets ibv_reg_mr take a device pointer (src/plugin.cc:321-331).  FUSELINK_PEERMEM=0|1 overrides.
  bool peer_memory_supported() override {
    const int64_t forced = param_i64("FUSELINK_PEERMEM", -1);
    if (forced >= 0) return forced != 0;
    static const char* const kFiles[] = {"/sys/kernel/mm/memory_peers/nv_mem/version", "/sys/kernel/mm/memory_peers/nv_mem_nc/version",
                                         "/sys/module/nvidia_peermem/version"};
    for (const char* f : kFiles)
      if (access(f, F_OK) == 0) return true;
    return false;
  }
  void dereg_mr(Mr* m) override {
    if (!m) return;
    lib_.dereg_mr(reinterpret_cast<ibv_mr*>(m->impl));
    delete m;
  }
  Cq* create_cq(int dev, int depth) override {
    ibv_cq* cq = lib_.create_cq(ports_[dev].ctx, depth, nullptr, nullptr, 0);
    return cq ? reinterpret_cast<Cq*>(new VCq{dev, cq}) : nullptr;
  }
  void destroy_cq(Cq* h) override {
    VCq* c = reinterpret_cast<VCq*>(h);
    if (!c) return;
    lib_.destroy_cq(c->cq);
    delete c;
  }
  Qp* create_qp(Pd* ph, Cq* ch, const QpCaps& caps) override {
    VPd* p = reinterpret_cast<VPd*>(ph);
    VCq* c = reinterpret_cast<VCq*>(ch);
    ibv_qp_init_attr a;
    memset(&a, 0, sizeof a);
    a.send_cq = c->cq;
    a.recv_cq = c->cq;
    a.qp_type = IBV_QPT_RC;
    a.cap.max_send_wr = (uint32_t)caps.max_send_wr;
    a.cap.max_recv_wr = (uint32_t)caps.max_recv_wr;
    a.cap.max_send_sge = 1;
    a.cap.max_recv_sge = 1;
    a.cap.max_inline_data = (uint32_t)caps.max_inline;
    ibv_qp* qp = lib_.create_qp(p->pd, &a);
    return qp ? reinterpret_cast<Qp*>(new VQp{p->dev, qp}) : nullptr;
  }
  void destroy_qp(Qp* h) override {
    VQp* q = reinterpret_cast<VQp*>(h);
    if (!q) return;
    lib_.destroy_qp(q->qp);
    delete q;
  }
  int query_qp_info(Qp* h, int gid_index, QpInfo* out) override {
    VQp* q = reinterpret_cast<VQp*>(h);
    const Port& pt = ports_[q->dev];
    memset(out, 0, sizeof *out);
    out->qpn = q->qp->qp_num;
    out->lid = pt.lid;
    out->link = (uint8_t)pt.info.link;
    out->port = (uint8_t)pt.info.port;
    out->mtu = (uint8_t)pt.active_mtu;
    if (pt.info.link == kLinkEthernet) {
      ibv_gid g;
      if (lib_.query_gid(pt.ctx, (uint8_t)pt.info.port, gid_index, &g)) return -1;
      memcpy(out->gid, g.raw, 16);
    }
    return 0;
  }
  bool query_ece(Qp* h, Ece* out) override {
    if (!lib_.query_ece || !lib_.set_ece) return false;
    ibv_ece e;
    memset(&e, 0, sizeof e);
    if (lib_.query_ece(reinterpret_cast<VQp*>(h)->qp, &e)) return false;      // EOPNOTSUPP on devices without it
    out->vendor_id = e.vendor_id; out->options = e.options; out->comp_mask = e.comp_mask;
    return true;
  }
  bool set_ece(Qp* h, const Ece& in) override {
    if (!lib_.set_ece) return false;
    ibv_ece e;
    e.vendor_id = in.vendor_id; e.options = in.options; e.comp_mask = in.comp_mask;
    return lib_.set_ece(reinterpret_cast<VQp*>(h)->qp, &e) == 0;
  }
  int connect_qp(Qp* h, const QpInfo& remote, const QpConnectParams& p) override {
    VQp* q = reinterpret_cast<VQp*>(h);
    const Port& pt = ports_[q->dev];
    ibv_qp_attr a;
    memset(&a, 0, sizeof a);
    a.qp_state = IBV_QPS_INIT;
    a.pkey_index = (uint16_t)p.pkey;
    a.port_num = (uint8_t)pt.info.port;
    a.qp_access_flags = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ;
    if (lib_.modify_qp(q->qp, &a, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS)) return -1;
    memset(&a, 0, sizeof a);
    a.qp_state = IBV_QPS_RTR;
    a.path_mtu = remote.mtu < pt.active_mtu ? remote.mtu : pt.active_mtu;
    a.dest_qp_num = remote.qpn;
    a.rq_psn = 0;
    a.max_dest_rd_atomic = 1;
    a.min_rnr_timer = 12;
    if (remote.link == kLinkEthernet) {
      a.ah_attr.is_global = 1;
      memcpy(a.ah_attr.grh.dgid.raw, remote.gid, 16);
      a.ah_attr.grh.flow_label = 0;
      a.ah_attr.grh.sgid_index = (uint8_t)p.gid_index;
      a.ah_attr.grh.hop_limit = 255;
      a.ah_attr.grh.traffic_class = (uint8_t)p.tc;
    } else {
      a.ah_attr.is_global = 0;
      a.ah_attr.dlid = remote.lid;
    }
    a.ah_attr.sl = (uint8_t)p.sl;
    a.ah_attr.src_path_bits = 0;
    a.ah_attr.port_num = (uint8_t)pt.info.port;
    if (lib_.modify_qp(q->qp, &a, IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC |
                                      IBV_QP_MIN_RNR_TIMER))
      return -1;
    memset(&a, 0, sizeof a);
    a.qp_state = IBV_QPS_RTS;
    a.timeout = (uint8_t)p.timeout;
    a.retry_cnt = (uint8_t)p.retry_cnt;
    a.rnr_retry = 7;
    a.sq_psn = 0;
    a.max_rd_atomic = 1;
    if (lib_.modify_qp(q->qp, &a, IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC))
      return -1;
    return 0;
  }
  int post_send(Qp* h, const SendWr* wrs, int n) override {
    VQp* q = reinterpret_cast<VQp*>(h);
    if (n < 1 || n > 8) return -1;
    ibv_send_wr w[8];
    ibv_sge sge[8];
    memset(w, 0, sizeof w);
    for (int i = 0; i < n; ++i) {
      sge[i].addr = (uint64_t)(uintptr_t)wrs[i].laddr;
      sge[i].length = wrs[i].len;
      sge[i].lkey = wrs[i].lkey;
      w[i].wr_id = wrs[i].wr_id;
      w[i].next = i + 1 < n ? &w[i + 1] : nullptr;
      w[i].sg_list = wrs[i].len ? &sge[i] : nullptr;
      w[i].num_sge = wrs[i].len ? 1 : 0;
      w[i].opcode = wrs[i].op == kWriteImm ? IBV_WR_RDMA_WRITE_WITH_IMM : wrs[i].op == kRead ? IBV_WR_RDMA_READ : IBV_WR_RDMA_WRITE;
      w[i].send_flags = (wrs[i].signaled ? IBV_SEND_SIGNALED : 0) | (wrs[i].inline_data ? IBV_SEND_INLINE : 0);
      w[i].imm_data = wrs[i].imm;
      w[i].wr.rdma.remote_addr = wrs[i].raddr;
      w[i].wr.rdma.rkey = wrs[i].rkey;
    }
    ibv_send_wr* bad = nullptr;
    auto fn = reinterpret_cast<post_send_fn>(q->qp->context->ops[kOpPostSend]);
    return fn(q->qp, w, &bad);
  }
  int post_recv(Qp* h, uint64_t wr_id) override {
    VQp* q = reinterpret_cast<VQp*>(h);
    ibv_recv_wr w;
    memset(&w, 0, sizeof w);
    w.wr_id = wr_id;
    ibv_recv_wr* bad = nullptr;
    auto fn = reinterpret_cast<post_recv_fn>(q->qp->context->ops[kOpPostRecv]);
    return fn(q->qp, &w, &bad);
  }
  int poll_cq(Cq* h, int max, Completion* out) override {
    VCq* c = reinterpret_cast<VCq*>(h);
    ibv_wc wc[16];
    if (max > 16) max = 16;
    auto fn = reinterpret_cast<poll_cq_fn>(c->cq->context->ops[kOpPollCq]);
    const int n = fn(c->cq, max, wc);
    for (int i = 0; i < n; ++i) {
      out[i] = Completion();
      out[i].wr_id = wc[i].wr_id;
      out[i].status = wc[i].status;
      out[i].is_recv = wc[i].opcode == IBV_WC_RECV_RDMA_WITH_IMM;
      out[i].imm = wc[i].imm_data;
      out[i].byte_len = wc[i].byte_len;
      out[i].qpn = wc[i].qp_num;
    }
    return n;
  }
  int wait_async_event(int dev, int timeout_ms, std::string* what) override {
    (void)timeout_ms;                                   // the library call blocks until an event arrives
    ibv_async_event ev;
    if (!lib_.get_async_event || lib_.get_async_event(ports_[dev].ctx, &ev)) return -1;
    *what = lib_.event_type_str ? lib_.event_type_str(ev.event_type) : "event";
    lib_.ack_async_event(&ev);
    return 1;
  }

 private:
  std::mutex probe_mu_;
  std::vector<int> dmabuf_probe_;      // per device: -1 not probed yet, 0 no, 1 yes
  void discover() {
    if (params().ib_disable) return;
    void* h = dlopen("libibverbs.so.1", RTLD_NOW);
    if (!h) h = dlopen("libibverbs.so", RTLD_NOW);
    if (!h) {
      FL_INFO("libibverbs not found: no verbs devices");
      return;
    }
    lib_.handle = h;
    bool ok = sym(h, "ibv_get_device_list", &lib_.get_device_list) && sym(h, "ibv_free_device_list", &lib_.free_device_list) &&
              sym(h, "ibv_get_device_name", &lib_.get_device_name) && sym(h, "ibv_get_device_guid", &lib_.get_device_guid) &&
              sym(h, "ibv_open_device", &lib_.open_device) && sym(h, "ibv_close_device", &lib_.close_device) &&
              sym(h, "ibv_query_device", &lib_.query_device) && sym(h, "ibv_query_port", &lib_.query_port) &&
              sym(h, "ibv_query_gid", &lib_.query_gid) && sym(h, "ibv_alloc_pd", &lib_.alloc_pd) && sym(h, "ibv_dealloc_pd", &lib_.dealloc_pd) &&
              sym(h, "ibv_reg_mr", &lib_.reg_mr) && sym(h, "ibv_dereg_mr", &lib_.dereg_mr) && sym(h, "ibv_create_cq", &lib_.create_cq) &&
              sym(h, "ibv_destroy_cq", &lib_.destroy_cq) && sym(h, "ibv_create_qp", &lib_.create_qp) && sym(h, "ibv_modify_qp", &lib_.modify_qp) &&
              sym(h, "ibv_destroy_qp", &lib_.destroy_qp);
    sym(h, "ibv_reg_mr_iova2", &lib_.reg_mr_iova2, false);
    sym(h, "ibv_reg_dmabuf_mr", &lib_.reg_dmabuf_mr, false);
    sym(h, "ibv_query_ece", &lib_.query_ece, false);
    sym(h, "ibv_set_ece", &lib_.set_ece, false);
    sym(h, "ibv_get_async_event", &lib_.get_async_event, false);
    sym(h, "ibv_ack_async_event", &lib_.ack_async_event, false);
    sym(h, "ibv_event_type_str", &lib_.event_type_str, false);
    if (!ok) {
      FL_WARN("libibverbs lacks a required symbol: verbs path disabled");
      return;
    }
    int n = 0;
    void** list = lib_.get_device_list(&n);
    if (!list) return;
    const HcaFilter filter = parse_hca_filter(params().ib_hca);
    for (int i = 0; i < n && ports_.size() < 32; ++i) {
      ibv_context* ctx = lib_.open_device(list[i]);
      if (!ctx) continue;
      ibv_device_attr da;
      memset(&da, 0, sizeof da);
      if (lib_.query_device(ctx, &da)) { lib_.close_device(ctx); continue; }
      const std::string name = lib_.get_device_name(list[i]);
      bool used = false;
      for (int port = 1; port <= da.phys_port_cnt; ++port) {
        ibv_port_attr pa;
        memset(&pa, 0, sizeof pa);
        if (lib_.query_port(ctx, (uint8_t)port, &pa)) continue;
        if (pa.state != IBV_PORT_ACTIVE) continue;
        if (pa.link_layer != IBV_LINK_LAYER_INFINIBAND && pa.link_layer != IBV_LINK_LAYER_ETHERNET) continue;
        if (!hca_allowed(filter, name, port)) continue;
        Port p;
        p.ctx = ctx;
        p.info.name = name;
        p.info.port = port;
        p.info.guid = lib_.get_device_guid(list[i]);
        p.info.max_qp = da.max_qp;
        p.info.link = pa.link_layer == IBV_LINK_LAYER_ETHERNET ? kLinkEthernet : kLinkIB;
        p.info.speed_mbps = lane_mbps(pa.active_speed) * lanes(pa.active_width);
        p.info.relaxed_ordering = lib_.reg_mr_iova2 != nullptr;
        p.info.pci_path = pci_path(name);
        p.active_mtu = pa.active_mtu;
        p.lid = pa.lid;
        ports_.push_back(p);
        used = true;
      }
      if (!used) lib_.close_device(ctx);
    }
    lib_.free_device_list(list);
  }

  // Resolved sysfs path of the adapter.  The trailing PCI function digit is cleared so that the ports of one
  // adapter share a path, and with NCCL_IB_MERGE_VFS the device digits too, so that virtual functions fold into
  // their physical function (what the reference does at src/plugin.cc:119-138).
  static std::string pci_path(const std::string& name) {
    char link[PATH_MAX], real[PATH_MAX];
    snprintf(link, sizeof link, "/sys/class/infiniband/%s/device", name.c_str());
    if (!realpath(link, real)) return std::string();
    size_t n = strlen(real);
    if (n >= 1) real[n - 1] = '0';
    if (params().ib_merge_vfs && n >= 4) real[n - 3] = real[n - 4] = '0';
    return real;
  }

  Lib lib_;
  std::vector<Port> ports_;
};

}  // namespace

Provider* make_verbs_provider() {
  static VerbsProvider* p = new VerbsProvider();
  return p;
}

Provider* get_provider() {
  static Provider* chosen = [] () -> Provider* {
    const std::string which = param_str("FUSELINK_RDMA_PROVIDER", "verbs");
    if (which == "soft") return make_soft_provider();
    if (which == "none") return nullptr;
    return make_verbs_provider();
  }();
  return chosen;
}

}  // namespace rdma
}  // namespace flnet
