// A stand-in for libibverbs.so.1 used by the tests of the verbs provider: the exported ibv_* functions and the
// function table inside ibv_context, laid out as the real library lays them out, on top of the software NIC.  It lets
// the provider's discovery (ports, link layer, speed codes, NCCL_IB_HCA), its queue-pair state machine and its
// translation of work requests and completions run end to end through the plugin on a machine without RDMA hardware.
// The transitions check the attribute masks the real library requires, so a missing attribute fails here too.
#include <errno.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "../../fuselink_b200/csrc/net/rdma_provider.h"
#include "../../fuselink_b200/csrc/net/verbs_abi.h"

using namespace flnet::verbs_abi;
namespace rd = flnet::rdma;

namespace {
rd::Provider* nic() { return rd::make_soft_provider(); }

struct FakeDevice { char name[64]; int index; };
struct FakeContext { ibv_context ctx; int dev; };
struct FakePd { ibv_pd pd; rd::Pd* impl; int dev; };
struct FakeMr { ibv_mr mr; rd::Mr* impl; };
struct FakeCq { ibv_cq cq; rd::Cq* impl; };
struct FakeQp { ibv_qp qp; rd::Qp* impl; int dev; int state; uint32_t dest_qpn; uint64_t dest_cookie; uint32_t ece_options; int ece_set; };

FakeDevice g_devs[8];
int g_ndevs = 0;

// FUSELINK_FAKE_IB_LOG=<file>: one line per call whose arguments a test wants to see (queue-pair attributes, access flags).
void record(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
void record(const char* fmt, ...) {
  const char* path = getenv("FUSELINK_FAKE_IB_LOG");
  if (!path || !*path) return;
  char line[512];
  va_list ap;
  va_start(ap, fmt);
  int n = vsnprintf(line, sizeof line - 1, fmt, ap);
  va_end(ap);
  if (n < 0) return;
  if (n > (int)sizeof line - 2) n = (int)sizeof line - 2;
  line[n++] = '\n';
  FILE* f = fopen(path, "a");                   // O_APPEND: whole lines from both processes of a test
  if (!f) return;
  fwrite(line, 1, (size_t)n, f);
  fclose(f);
}

int ndevs() {
  const char* e = getenv("FUSELINK_FAKE_IB_NDEV");
  int n = e ? atoi(e) : 2;
  return n < 1 ? 1 : n > 8 ? 8 : n;
}

int fake_poll_cq(ibv_cq* cq, int n, ibv_wc* wc) {
  rd::Completion c[16];
  if (n > 16) n = 16;
  const int got = nic()->poll_cq(reinterpret_cast<FakeCq*>(cq)->impl, n, c);
  for (int i = 0; i < got; ++i) {
    memset(&wc[i], 0, sizeof wc[i]);
    wc[i].wr_id = c[i].wr_id;
    wc[i].status = c[i].status;
    wc[i].opcode = c[i].is_recv ? IBV_WC_RECV_RDMA_WITH_IMM : 1 /* IBV_WC_RDMA_WRITE */;
    wc[i].byte_len = c[i].byte_len;
    wc[i].imm_data = c[i].imm;
    wc[i].qp_num = c[i].qpn;
    wc[i].wc_flags = c[i].is_recv ? 2 /* IBV_WC_WITH_IMM */ : 0;
  }
  return got;
}

int fake_post_send(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) {
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  if (q->state != IBV_QPS_RTS) { *bad = wr; return EINVAL; }
  rd::SendWr out[8];
  int n = 0;
  for (ibv_send_wr* w = wr; w; w = w->next) {
    if (n == 8 || w->num_sge > 1) { *bad = w; return EINVAL; }
    rd::SendWr& o = out[n++];
    o = rd::SendWr();
    o.wr_id = w->wr_id;
    o.op = w->opcode == IBV_WR_RDMA_WRITE_WITH_IMM ? rd::kWriteImm : w->opcode == IBV_WR_RDMA_READ ? rd::kRead : rd::kWrite;
    if (w->opcode != IBV_WR_RDMA_WRITE && w->opcode != IBV_WR_RDMA_WRITE_WITH_IMM && w->opcode != IBV_WR_RDMA_READ) { *bad = w; return EINVAL; }
    if (w->num_sge == 1) {
      o.laddr = reinterpret_cast<const void*>(w->sg_list[0].addr);
      o.len = w->sg_list[0].length;
      o.lkey = w->sg_list[0].lkey;
    }
    o.raddr = w->wr.rdma.remote_addr;
    o.rkey = w->wr.rdma.rkey;
    o.imm = w->imm_data;
    o.signaled = (w->send_flags & IBV_SEND_SIGNALED) != 0;
    o.inline_data = (w->send_flags & IBV_SEND_INLINE) != 0;
  }
  const int rc = nic()->post_send(q->impl, out, n);
  if (rc) *bad = wr;
  return rc ? ENOMEM : 0;
}

int fake_post_recv(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad) {
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  if (q->state < IBV_QPS_INIT) { *bad = wr; return EINVAL; }      // receives may be posted from INIT on
  for (ibv_recv_wr* w = wr; w; w = w->next)
    if (nic()->post_recv(q->impl, w->wr_id)) { *bad = w; return ENOMEM; }
  return 0;
}
}  // namespace

extern "C" {

void** ibv_get_device_list(int* num) {
  g_ndevs = ndevs() < nic()->device_count() ? ndevs() : nic()->device_count();
  void** list = static_cast<void**>(calloc(g_ndevs + 1, sizeof(void*)));
  for (int i = 0; i < g_ndevs; ++i) {
    snprintf(g_devs[i].name, sizeof g_devs[i].name, "mlx5_%d", i);
    g_devs[i].index = i;
    list[i] = &g_devs[i];
  }
  if (num) *num = g_ndevs;
  return list;
}
void ibv_free_device_list(void** list) { free(list); }
const char* ibv_get_device_name(void* dev) { return static_cast<FakeDevice*>(dev)->name; }
uint64_t ibv_get_device_guid(void* dev) { return 0xfa4e000000000000ull + (uint64_t)static_cast<FakeDevice*>(dev)->index; }

ibv_context* ibv_open_device(void* dev) {
  FakeContext* c = static_cast<FakeContext*>(calloc(1, sizeof(FakeContext)));
  c->dev = static_cast<FakeDevice*>(dev)->index;
  c->ctx.device = dev;
  c->ctx.ops[kOpPollCq] = reinterpret_cast<void*>(&fake_poll_cq);
  c->ctx.ops[kOpPostSend] = reinterpret_cast<void*>(&fake_post_send);
  c->ctx.ops[kOpPostRecv] = reinterpret_cast<void*>(&fake_post_recv);
  return &c->ctx;
}
int ibv_close_device(ibv_context* ctx) { free(ctx); return 0; }

int ibv_query_device(ibv_context* ctx, ibv_device_attr* a) {
  memset(a, 0, sizeof(ibv_device_attr) - sizeof a->reserve);
  snprintf(a->fw_ver, sizeof a->fw_ver, "fake-1.0");
  a->node_guid = 0xfa4e000000000000ull + (uint64_t)reinterpret_cast<FakeContext*>(ctx)->dev;
  a->max_qp = 4096;
  a->max_qp_wr = 8192;
  a->max_cq = 4096;
  a->max_cqe = 1 << 20;
  a->max_mr = 1 << 20;
  a->phys_port_cnt = 2;           // port 2 exists and is down: discovery has to skip it
  return 0;
}
int ibv_query_port(ibv_context*, uint8_t port, ibv_port_attr* a) {
  memset(a, 0, sizeof(ibv_port_attr) - sizeof a->reserve);
  a->state = port == 1 ? IBV_PORT_ACTIVE : 1 /* IBV_PORT_DOWN */;
  a->max_mtu = 5;
  a->active_mtu = 5;
  a->gid_tbl_len = 4;
  a->lid = 0;
  a->active_width = 2;            // 4x
  a->active_speed = 32;           // EDR, 25 Gb/s per lane -> 100 Gb/s
  a->link_layer = IBV_LINK_LAYER_ETHERNET;
  return 0;
}
int ibv_query_gid(ibv_context* ctx, uint8_t, int, ibv_gid* gid) {
  memset(gid, 0, sizeof *gid);
  const uint64_t pid = (uint64_t)getpid();
  memcpy(gid->raw, &pid, 8);      // the "address" of a software NIC is its process
  gid->raw[8] = (uint8_t)reinterpret_cast<FakeContext*>(ctx)->dev;
  gid->raw[15] = 1;
  return 0;
}

ibv_pd* ibv_alloc_pd(ibv_context* ctx) {
  FakePd* p = static_cast<FakePd*>(calloc(1, sizeof(FakePd)));
  p->pd.context = ctx;
  p->dev = reinterpret_cast<FakeContext*>(ctx)->dev;
  p->impl = nic()->alloc_pd(p->dev);
  return &p->pd;
}
int ibv_dealloc_pd(ibv_pd* pd) {
  FakePd* p = reinterpret_cast<FakePd*>(pd);
  nic()->dealloc_pd(p->impl);
  free(p);
  return 0;
}
ibv_mr* ibv_reg_mr(ibv_pd* pd, void* addr, size_t len, int access) {
  int a = 0;
  if (access & IBV_ACCESS_LOCAL_WRITE) a |= rd::kAccessLocalWrite;
  if (access & IBV_ACCESS_REMOTE_WRITE) a |= rd::kAccessRemoteWrite;
  if (access & IBV_ACCESS_REMOTE_READ) a |= rd::kAccessRemoteRead;
  if ((access & IBV_ACCESS_REMOTE_WRITE) && !(access & IBV_ACCESS_LOCAL_WRITE)) { errno = EINVAL; return nullptr; }   // verbs rule
  record("reg_mr len=%zu access=0x%x", len, (unsigned)access);
  FakeMr* m = static_cast<FakeMr*>(calloc(1, sizeof(FakeMr)));
  m->impl = nic()->reg_mr(reinterpret_cast<FakePd*>(pd)->impl, addr, len, a);
  m->mr.context = pd->context;
  m->mr.pd = pd;
  m->mr.addr = addr;
  m->mr.length = len;
  m->mr.lkey = m->impl->lkey;
  m->mr.rkey = m->impl->rkey;
  return &m->mr;
}
// The entry point newer libraries add; relaxed ordering can only be asked for through it.
ibv_mr* ibv_reg_mr_iova2(ibv_pd* pd, void* addr, size_t len, uint64_t iova, unsigned int access) {
  if (iova != (uint64_t)(uintptr_t)addr) { errno = EINVAL; return nullptr; }
  return ibv_reg_mr(pd, addr, len, (int)access);
}
// FUSELINK_FAKE_IB_DMABUF=0: a kernel without dma-buf support.
ibv_mr* ibv_reg_dmabuf_mr(ibv_pd* pd, uint64_t offset, size_t len, uint64_t iova, int fd, int access) {
  const char* e = getenv("FUSELINK_FAKE_IB_DMABUF");
  if (e && e[0] == '0') { errno = EOPNOTSUPP; return nullptr; }
  if (fd < 0) { errno = EBADF; return nullptr; }
  int a = 0;
  if (access & IBV_ACCESS_LOCAL_WRITE) a |= rd::kAccessLocalWrite;
  if (access & IBV_ACCESS_REMOTE_WRITE) a |= rd::kAccessRemoteWrite;
  if (access & IBV_ACCESS_REMOTE_READ) a |= rd::kAccessRemoteRead;
  record("reg_dmabuf_mr len=%zu offset=%llu access=0x%x", len, (unsigned long long)offset, (unsigned)access);
  rd::Mr* impl = nic()->reg_dmabuf_mr(reinterpret_cast<FakePd*>(pd)->impl, fd, offset, len, iova, a);
  if (!impl) return nullptr;
  FakeMr* m = static_cast<FakeMr*>(calloc(1, sizeof(FakeMr)));
  m->impl = impl;
  m->mr.context = pd->context;
  m->mr.pd = pd;
  m->mr.addr = reinterpret_cast<void*>(iova);
  m->mr.length = len;
  m->mr.lkey = impl->lkey;
  m->mr.rkey = impl->rkey;
  return &m->mr;
}
int ibv_dereg_mr(ibv_mr* mr) {
  FakeMr* m = reinterpret_cast<FakeMr*>(mr);
  nic()->dereg_mr(m->impl);
  free(m);
  return 0;
}
ibv_cq* ibv_create_cq(ibv_context* ctx, int cqe, void*, void*, int) {
  FakeCq* c = static_cast<FakeCq*>(calloc(1, sizeof(FakeCq)));
  c->cq.context = ctx;
  c->impl = nic()->create_cq(reinterpret_cast<FakeContext*>(ctx)->dev, cqe);
  return &c->cq;
}
int ibv_destroy_cq(ibv_cq* cq) {
  FakeCq* c = reinterpret_cast<FakeCq*>(cq);
  nic()->destroy_cq(c->impl);
  free(c);
  return 0;
}
ibv_qp* ibv_create_qp(ibv_pd* pd, ibv_qp_init_attr* ia) {
  if (ia->qp_type != IBV_QPT_RC || !ia->send_cq || ia->send_cq != ia->recv_cq) { errno = EINVAL; return nullptr; }
  FakeQp* q = static_cast<FakeQp*>(calloc(1, sizeof(FakeQp)));
  rd::QpCaps caps;
  caps.max_send_wr = (int)ia->cap.max_send_wr;
  caps.max_recv_wr = (int)ia->cap.max_recv_wr;
  caps.max_inline = (int)ia->cap.max_inline_data;
  q->dev = reinterpret_cast<FakePd*>(pd)->dev;
  q->impl = nic()->create_qp(reinterpret_cast<FakePd*>(pd)->impl, reinterpret_cast<FakeCq*>(ia->send_cq)->impl, caps);
  rd::QpInfo info;
  nic()->query_qp_info(q->impl, 0, &info);
  q->qp.context = pd->context;
  q->qp.pd = pd;
  q->qp.send_cq = ia->send_cq;
  q->qp.recv_cq = ia->recv_cq;
  q->qp.qp_num = info.qpn;
  q->state = IBV_QPS_RESET;
  record("create_qp dev=%d max_send_wr=%u max_recv_wr=%u max_inline=%u", q->dev, ia->cap.max_send_wr, ia->cap.max_recv_wr, ia->cap.max_inline_data);
  return &q->qp;
}
int ibv_modify_qp(ibv_qp* qp, ibv_qp_attr* a, int mask) {
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  if (!(mask & IBV_QP_STATE)) return EINVAL;
  if (a->qp_state == IBV_QPS_INIT) {
    const int need = IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS;
    if (q->state != IBV_QPS_RESET || (mask & need) != need || a->port_num != 1) return EINVAL;
    record("init dev=%d pkey=%u access=0x%x", q->dev, (unsigned)a->pkey_index, a->qp_access_flags);
  } else if (a->qp_state == IBV_QPS_RTR) {
    const int need = IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER;
    if (q->state != IBV_QPS_INIT || (mask & need) != need || !a->ah_attr.is_global || a->path_mtu < 1 || a->path_mtu > 5) return EINVAL;
    q->dest_qpn = a->dest_qp_num;
    record("rtr dev=%d mtu=%d sgid_index=%u tc=%u sl=%u hop_limit=%u", q->dev, (int)a->path_mtu, (unsigned)a->ah_attr.grh.sgid_index,
           (unsigned)a->ah_attr.grh.traffic_class, (unsigned)a->ah_attr.sl, (unsigned)a->ah_attr.grh.hop_limit);
    memcpy(&q->dest_cookie, a->ah_attr.grh.dgid.raw, 8);
  } else if (a->qp_state == IBV_QPS_RTS) {
    const int need = IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC;
    if (q->state != IBV_QPS_RTR || (mask & need) != need) return EINVAL;
    record("rts dev=%d timeout=%u retry_cnt=%u rnr_retry=%u", q->dev, (unsigned)a->timeout, (unsigned)a->retry_cnt, (unsigned)a->rnr_retry);
    rd::QpInfo remote;
    memset(&remote, 0, sizeof remote);
    remote.qpn = q->dest_qpn;
    remote.cookie = q->dest_cookie;
    rd::QpConnectParams p;
    if (nic()->connect_qp(q->impl, remote, p)) return ENETUNREACH;
  } else {
    return EINVAL;
  }
  q->state = a->qp_state;
  return 0;
}
// FUSELINK_FAKE_IB_ECE=<options>: the device offers these enhanced-connection options (vendor 0x15b3); unset: the calls
// answer "not supported".  Options may only be set while the queue pair has not been connected, and what a later query
// returns is what both ends have in common.
int ibv_query_ece(ibv_qp* qp, ibv_ece* ece) {
  const char* e = getenv("FUSELINK_FAKE_IB_ECE");
  if (!e) return EOPNOTSUPP;
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  ece->vendor_id = 0x15b3;
  ece->options = q->ece_set ? q->ece_options : (uint32_t)strtoul(e, nullptr, 0);
  ece->comp_mask = 0;
  return 0;
}
int ibv_set_ece(ibv_qp* qp, ibv_ece* ece) {
  const char* e = getenv("FUSELINK_FAKE_IB_ECE");
  if (!e) return EOPNOTSUPP;
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  if (q->state != IBV_QPS_RESET && q->state != IBV_QPS_INIT) return EINVAL;
  if (ece->vendor_id != 0x15b3) return EINVAL;
  q->ece_options = ece->options & (uint32_t)strtoul(e, nullptr, 0);
  q->ece_set = 1;
  record("set_ece dev=%d given=0x%x kept=0x%x", q->dev, ece->options, q->ece_options);
  return 0;
}
int ibv_destroy_qp(ibv_qp* qp) {
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  nic()->destroy_qp(q->impl);
  free(q);
  return 0;
}
int ibv_get_async_event(ibv_context* ctx, ibv_async_event* ev) {
  // FUSELINK_FAKE_IB_EVENT_MS=<ms>: device 0 reports "port error" once, that long after the first wait; otherwise nothing
  // ever happens to a fake port
  static int fired = 0;
  const char* e = getenv("FUSELINK_FAKE_IB_EVENT_MS");
  if (e && reinterpret_cast<FakeContext*>(ctx)->dev == 0 && !__atomic_exchange_n(&fired, 1, __ATOMIC_ACQ_REL)) {
    usleep((useconds_t)atoi(e) * 1000);
    memset(ev, 0, sizeof *ev);
    ev->element.port_num = 1;
    ev->event_type = 10;         // IBV_EVENT_PORT_ERR
    return 0;
  }
  for (;;) sleep(3600);
  return -1;
}
void ibv_ack_async_event(ibv_async_event* ev) { record("ack_async_event type=%d", ev->event_type); }
const char* ibv_event_type_str(int t) { return t == 10 ? "port error" : "fake event"; }

}  // extern "C"
