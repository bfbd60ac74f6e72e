// RDMA transport: bootstrap, registration, posting and completion handling (protocol in rdma_transport.h).
#include "rdma_transport.h"

#include <errno.h>
#include <poll.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <thread>
#include <vector>

#include "logging.h"
#include "params.h"

namespace flnet {
namespace {

constexpr uint64_t kHelloMagic = 0x464c4e4b48454c4full;   // same hello as the TCP transport, kind 2
constexpr uint32_t kInfoMagic = 0x464c5244u;              // "FLRD"
constexpr uint64_t kWrFifo = 1ull << 62;                   // wr_id of a signalled descriptor write
constexpr uint64_t kWrRecv = 1ull << 61;                   // wr_id of the anonymous zero-length receives
constexpr uint64_t kWrFlush = 1ull << 60;                  // wr_id of a flush read (low bits: request slot)
constexpr uint64_t kWrRecord = 1ull << 59;                 // wr_id of the unsignalled per-slot record write (a piece's own id may be 0)

rdma::Provider* g_prov = nullptr;
rdma::Pd* g_pd[kMaxDev];
int g_ndev = 0;
std::atomic<uint64_t> g_uid{1};
std::atomic<uint64_t> g_pieces{0}, g_work_requests{0}, g_messages{0}, g_failovers{0};

int access_flags() {
  int f = rdma::kAccessLocalWrite | rdma::kAccessRemoteWrite | rdma::kAccessRemoteRead;
  const int64_t ro = params().ib_pci_relaxed_ordering;      // 0 off, 1 on, 2 when the library supports it
  if (ro == 1 || (ro == 2 && g_ndev > 0 && g_prov->device(0).relaxed_ordering)) f |= rdma::kAccessRelaxedOrdering;
  return f;
}

void fail(RdmaComm* c, ncclResult_t why, const char* what) {
  if (!c->error) {
    c->error = why;
    FL_WARN("rdma %s comm (channel %d, dev %d): %s", c->is_send ? "send" : "recv", c->channel_id, c->own_dev, what);
  }
}

void* alloc_zeroed(size_t bytes) {
  void* p = nullptr;
  if (posix_memalign(&p, 4096, bytes) != 0) return nullptr;
  memset(p, 0, bytes);
  return p;
}

// One completion queue and nqps queue pairs on every device, receives pre-posted on the receiving side.
bool make_endpoints(RdmaComm* c) {
  rdma::QpCaps caps;
  caps.max_send_wr = 4 * kMaxRequests;
  caps.max_recv_wr = 2 * kMaxRequests;
  caps.max_inline = params().ib_use_inline ? (int)sizeof(RdmaDesc) : 0;
  memset(&c->mine, 0, sizeof c->mine);
  c->mine.magic = kInfoMagic;
  c->mine.ndev = c->ndev;
  c->mine.nqps = c->nqps;
  c->mine.own_dev = c->own_dev;
  for (int d = 0; d < c->ndev; ++d) {
    c->dev[d].cq = g_prov->create_cq(d, 8 * kMaxRequests);
    if (!c->dev[d].cq) return false;
    for (int q = 0; q < c->nqps; ++q) {
      c->dev[d].qp[q] = g_prov->create_qp(g_pd[d], c->dev[d].cq, caps);
      if (!c->dev[d].qp[q]) return false;
      rdma::QpInfo& mine = c->mine.qp[d][q];
      if (g_prov->query_qp_info(c->dev[d].qp[q], (int)params().ib_gid_index, &mine)) return false;
      // Enhanced connection establishment.  The connecting side offers its options; the accepting side (which knows
      // the offer by now) takes them and answers with what is left; the connecting side applies the answer in
      // connect_endpoints.  All of it before the queue pair leaves INIT.
      rdma::Ece ece;
      mine.ece_supported = 0;
      if (c->is_send) {
        if (g_prov->query_ece(c->dev[d].qp[q], &ece)) mine.ece_supported = 1;
      } else if (c->theirs.qp[d][q].ece_supported) {
        const rdma::QpInfo& t = c->theirs.qp[d][q];
        rdma::Ece offer;
        offer.vendor_id = t.ece_vendor_id; offer.options = t.ece_options; offer.comp_mask = t.ece_comp_mask;
        if (g_prov->set_ece(c->dev[d].qp[q], offer) && g_prov->query_ece(c->dev[d].qp[q], &ece)) mine.ece_supported = 1;
      }
      if (mine.ece_supported) {
        mine.ece_vendor_id = ece.vendor_id; mine.ece_options = ece.options; mine.ece_comp_mask = ece.comp_mask;
        FL_INFO("rdma dev %d qp %d: ece %s vendor 0x%x options 0x%x", d, q, c->is_send ? "offered" : "agreed", ece.vendor_id, ece.options);
      }
    }
  }
  return true;
}

bool connect_endpoints(RdmaComm* c) {
  rdma::QpConnectParams p;
  const Params& e = params();
  p.gid_index = (int)e.ib_gid_index; p.timeout = (int)e.ib_timeout; p.retry_cnt = (int)e.ib_retry_cnt;
  p.pkey = (int)e.ib_pkey; p.sl = (int)e.ib_sl; p.tc = (int)e.ib_tc;
  for (int d = 0; d < c->ndev; ++d)
    for (int q = 0; q < c->nqps; ++q) {
      const rdma::QpInfo& t = c->theirs.qp[d][q];
      if (c->is_send && t.ece_supported && c->mine.qp[d][q].ece_supported) {
        rdma::Ece agreed;
        agreed.vendor_id = t.ece_vendor_id; agreed.options = t.ece_options; agreed.comp_mask = t.ece_comp_mask;
        if (!g_prov->set_ece(c->dev[d].qp[q], agreed)) FL_WARN("rdma dev %d qp %d: the agreed ece options were refused", d, q);
      }
      if (g_prov->connect_qp(c->dev[d].qp[q], t, p)) return false;
    }
  return true;
}

// returns 1 when all `total` bytes moved, 0 to come back later, -1 on error
int io_step(int fd, void* buf, size_t total, size_t* done, bool sending) {
  while (*done < total) {
    ssize_t r = sending ? send(fd, (uint8_t*)buf + *done, total - *done, MSG_DONTWAIT | MSG_NOSIGNAL)
                        : recv(fd, (uint8_t*)buf + *done, total - *done, MSG_DONTWAIT);
    if (r > 0) { *done += (size_t)r; continue; }
    if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return 0;
    return -1;
  }
  return 1;
}

RdmaRequest* get_request(RdmaComm* c) {
  static thread_local int hint = 0;
  for (int i = 0; i < kMaxRequests; ++i) {
    const int s = (hint + i) % kMaxRequests;
    if (!c->reqs[s].used) {
      hint = s + 1;
      RdmaRequest& r = c->reqs[s];
      r = RdmaRequest();
      r.used = true;
      r.comm = c;
      r.slot = (uint32_t)s;
      r.last_progress_ns = now_ns();
      return &r;
    }
  }
  return nullptr;
}

int rdma_next_alive(const RdmaComm* c, int from) {
  for (int i = 0; i < c->ndev; ++i) {
    const int d = ((from % c->ndev) + c->ndev + i) % c->ndev;
    if (!c->dead[d]) return d;
  }
  return -1;
}

// Posts piece `pi` of send request `r` on the device / queue pair recorded in the piece.
bool post_piece(RdmaComm* c, RdmaRequest* r, int pi) {
  const Params& p = params();
  RdmaPiece& pc = r->pieces[pi];
  const RdmaDesc& d = r->desc;
  const int dev = pc.dev;
  const int npieces = (int)r->pieces.size();
  const uint32_t imm = (d.slot & 0xffu) | ((uint32_t)npieces << 8) | ((uint32_t)pi << 16);
  rdma::SendWr wr[3];
  int n = 0;
  if (pi == 0) {                            // the record for the slot travels ahead of the first immediate
    wr[n].wr_id = kWrRecord;
    wr[n].op = rdma::kWrite;
    wr[n].laddr = &c->done_src[d.slot % kMaxRequests];
    wr[n].len = sizeof(RdmaDoneRec);
    wr[n].lkey = c->done_src_mr->mr[dev]->lkey;
    wr[n].raddr = c->remote_done_addr + sizeof(RdmaDoneRec) * (d.slot % kMaxRequests);
    wr[n].rkey = c->remote_done_rkey[dev];
    wr[n].inline_data = p.ib_use_inline != 0;
    ++n;
  }
  const uint64_t wr_id = (uint64_t)r->slot | ((uint64_t)pi << 16) | ((uint64_t)pc.gen << 32);
  // With adaptive routing packets of one write may overtake each other, so a large payload goes as a plain write and
  // the immediate follows in an empty write of its own; NCCL_IB_ADAPTIVE_ROUTING = -2 means "on for InfiniBand, off for
  // RoCE" (src/plugin.cc:96,253-254,1454-1462).  Without it one write-with-immediate carries the payload.
  const int64_t ar_knob = p.ib_adaptive_routing;
  const bool ar = ar_knob == -2 ? g_prov->device(dev).link == rdma::kLinkIB : ar_knob != 0;
  const bool split = ar && pc.len > (uint64_t)p.ib_ar_threshold;
  if (split) {
    wr[n].wr_id = wr_id;
    wr[n].op = rdma::kWrite;
    wr[n].laddr = r->data + pc.off;
    wr[n].len = (uint32_t)pc.len;
    wr[n].lkey = r->mr->mr[dev]->lkey;
    wr[n].raddr = d.addr + pc.off;
    wr[n].rkey = d.rkey[dev];
    ++n;
  }
  wr[n].wr_id = wr_id;
  wr[n].op = rdma::kWriteImm;
  wr[n].laddr = split || pc.len == 0 ? nullptr : r->data + pc.off;
  wr[n].len = split ? 0 : (uint32_t)pc.len;
  wr[n].lkey = r->mr->mr[dev]->lkey;
  wr[n].raddr = d.addr + pc.off;
  wr[n].rkey = d.rkey[dev];
  wr[n].imm = imm;
  wr[n].signaled = true;
  ++n;
  if (r->bad_key)                            // test hook: wrong key on the payload
    for (int k = pi == 0 ? 1 : 0; k < n; ++k) wr[k].rkey ^= 0x5a5a5a5au;
  g_pieces.fetch_add(1, std::memory_order_relaxed);
  g_work_requests.fetch_add((uint64_t)n, std::memory_order_relaxed);
  return g_prov->post_send(c->dev[dev].qp[pc.q], wr, n) == 0;
}

bool post_descriptor(RdmaComm* c, uint64_t idx) {
  RdmaDesc* d = &c->fifo_src[idx % kMaxRequests];
  rdma::SendWr wr;
  wr.wr_id = kWrFifo;
  wr.op = rdma::kWrite;
  wr.laddr = d;
  wr.len = sizeof *d;
  wr.lkey = c->fifo_src_mr->mr[c->ctrl_dev]->lkey;
  wr.raddr = c->remote_fifo_addr + sizeof(RdmaDesc) * (idx % kMaxRequests);
  wr.rkey = c->remote_fifo_rkey[c->ctrl_dev];
  wr.signaled = (idx % kFifoSignalEvery) == kFifoSignalEvery - 1;
  wr.inline_data = params().ib_use_inline != 0;
  return g_prov->post_send(c->dev[c->ctrl_dev].qp[0], &wr, 1) == 0;
}

// A completion came back in error on device d.  Returns false when the connection cannot go on.
bool device_failed(RdmaComm* c, ConnManager* cm, int d, const rdma::Completion& wc) {
  if (wc.status == rdma::kWcRemoteAccess || !params().failover) return false;
  if (wc.wr_id & kWrFlush) return false;
  const bool first = !c->dead[d];
  c->dead[d] = true;
  if (cm) cm->set_dead(d, true);
  const int to = rdma_next_alive(c, d + 1);
  if (to < 0) return false;
  if (first)
    FL_WARN("rdma %s comm (channel %d): device %d gave completion status %d and is given up; traffic moves to device %d",
            c->is_send ? "send" : "recv", c->channel_id, d, wc.status, to);
  if (!c->is_send) {
    // receiver: the descriptor writes went through this device.  Move them and write the descriptors of every
    // unfinished receive again (entries the sender has consumed already are behind its head and are ignored).
    if (!first) return true;
    if (d == c->ctrl_dev) c->ctrl_dev = to;
    uint64_t lo = UINT64_MAX;
    for (auto& r : c->reqs)
      if (r.used && !r.is_send && !r.is_flush && (r.pieces_total < 0 || r.pieces_done < r.pieces_total) && r.fifo_idx < lo) lo = r.fifo_idx;
    for (uint64_t idx = lo; lo != UINT64_MAX && idx < c->fifo_tail; ++idx) {
      if (!post_descriptor(c, idx)) return false;
      g_failovers.fetch_add(1, std::memory_order_relaxed);
    }
    return true;
  }
  if (wc.wr_id & (kWrFifo | kWrRecord)) return true;        // the unsignalled record write: its piece reports separately
  const uint32_t slot = (uint32_t)(wc.wr_id & 0xffffu), pi = (uint32_t)((wc.wr_id >> 16) & 0xffffu), gen = (uint32_t)((wc.wr_id >> 32) & 0xffu);
  RdmaRequest& r = c->reqs[slot % kMaxRequests];
  if (!r.used || !r.is_send || pi >= r.pieces.size()) return true;
  RdmaPiece& pc = r.pieces[pi];
  if (pc.done || pc.gen != gen) return true;               // an older posting of a piece that has moved on
  pc.gen++;
  pc.dev = to;
  g_failovers.fetch_add(1, std::memory_order_relaxed);
  return post_piece(c, &r, (int)pi);
}

void poll_all(RdmaComm* c, ConnManager* cm) {
  ScopedTimer tm(&c->timers, T_PROGRESS, params().timers != 0);
  g_prov->progress();
  rdma::Completion wc[16];
  for (int d = 0; d < c->ndev; ++d) {
    if (!c->dev[d].cq) continue;
    for (;;) {
      const int n = g_prov->poll_cq(c->dev[d].cq, 16, wc);
      if (n <= 0) break;
      for (int i = 0; i < n; ++i) {
        if (wc[i].status != rdma::kWcOk) {
          if (!wc[i].is_recv && device_failed(c, cm, d, wc[i])) continue;
          if (cm && wc[i].status == rdma::kWcRetryExceeded) cm->set_dead(d, true);
          char msg[192];
          snprintf(msg, sizeof msg, "completion with status %d on device %d (%s), queue pair %u, %s, wr_id 0x%llx, %u bytes, peer device %d",
                   wc[i].status, d, g_prov->device(d).name.c_str(), wc[i].qpn, wc[i].is_recv ? "receive" : "send side",
                   (unsigned long long)wc[i].wr_id, wc[i].byte_len, c->peer_dev);
          fail(c, wc[i].status == rdma::kWcRemoteAccess ? ncclInvalidUsage : ncclRemoteError, msg);
          continue;
        }
        if (wc[i].is_recv) {
          // keep the pool of zero-length receives full on the queue pair that consumed one
          for (int q = 0; q < c->nqps; ++q)
            if (c->dev[d].qp[q] && c->mine.qp[d][q].qpn == wc[i].qpn) g_prov->post_recv(c->dev[d].qp[q], kWrRecv);
          const uint32_t slot = wc[i].imm & 0xffu;
          const int npieces = (int)((wc[i].imm >> 8) & 0xffu);
          const int pi = (int)((wc[i].imm >> 16) & 0xffu);
          RdmaRequest& r = c->reqs[slot];
          if (!r.used || r.is_send || npieces < 1 || npieces > 64 || pi >= npieces) { fail(c, ncclInternalError, "immediate for a slot that is not posted"); continue; }
          r.pieces_total = npieces;
          if (!((r.piece_mask >> pi) & 1ull)) {
            r.piece_mask |= 1ull << pi;
            r.pieces_done++;
          }
          r.last_progress_ns = now_ns();
        } else if (wc[i].wr_id & kWrFifo) {
          // a signalled descriptor write: nothing to do but to have reaped the send queue
        } else if (wc[i].wr_id & kWrFlush) {
          RdmaRequest& r = c->reqs[wc[i].wr_id & 0xffffu];
          if (r.used && r.is_flush) r.pieces_done = r.pieces_total = 1;
        } else {
          const uint32_t slot = (uint32_t)(wc[i].wr_id & 0xffffu);
          const uint32_t piece = (uint32_t)((wc[i].wr_id >> 16) & 0xffffu);
          const uint32_t gen = (uint32_t)((wc[i].wr_id >> 32) & 0xffu);
          RdmaRequest& r = c->reqs[slot % kMaxRequests];
          if (!r.used || !r.is_send || piece >= r.pieces.size()) { fail(c, ncclInternalError, "send completion for an unknown piece"); continue; }
          if (r.pieces[piece].done || r.pieces[piece].gen != gen) continue;     // an earlier posting of a piece that was sent again
          r.pieces[piece].done = true;
          r.pieces_done++;
          r.last_progress_ns = now_ns();
          if (cm) cm->done_tx(r.pieces[piece].dev, r.pieces[piece].len);
        }
      }
    }
  }
}

void async_thread(int dev) {
  // one watcher per device, as the reference starts one per port (src/plugin.cc:100-113): events are logged
  for (;;) {
    std::string what;
    const int rc = g_prov->wait_async_event(dev, 500, &what);
    if (rc < 0) return;
    if (rc > 0) FL_WARN("rdma device %d (%s): asynchronous event: %s", dev, g_prov->device(dev).name.c_str(), what.c_str());
  }
}

}  // namespace

// -----------------------------------------------------------------------------------------------------
int rdma_init(ConnManager* cm) {
  (void)cm;
  if (g_ndev > 0) return g_ndev;
  g_prov = rdma::get_provider();
  if (!g_prov) return 0;
  int n = g_prov->device_count();
  if (n > kMaxDev) n = kMaxDev;
  for (int d = 0; d < n; ++d) {
    g_pd[d] = g_prov->alloc_pd(d);                         // up front, shared by every connection
    if (!g_pd[d]) {
      FL_WARN("rdma: no protection domain on device %d", d);
      return 0;
    }
  }
  g_ndev = n;
  for (int d = 0; d < n; ++d) std::thread(async_thread, d).detach();
  if (n) FL_INFO("rdma transport: %d device(s) through the %s provider", n, g_prov->name());
  return n;
}

rdma::DeviceInfo rdma_device(int dev) { return g_prov->device(dev); }

// Registration cache, one per device, as NCCL's verbs transport keeps one (the reference fills it in
// src/plugin.cc:1265-1305): NCCL registers the same buffer once per channel and connection, and a registration pins
// pages through the kernel, so a range that is registered already is shared and counted.  Ordinary registrations are
// widened to whole pages, which lets neighbouring sub-buffers of one allocation share an entry too; a dma-buf
// registration is keyed by its exact range.
namespace {
struct MrSlot {
  uintptr_t addr;
  size_t len;
  bool dmabuf;
  int refs;
  rdma::Mr* mr;
};
std::mutex g_mr_mu;
std::vector<MrSlot> g_mr_cache[kMaxDev];
std::atomic<uint64_t> g_mr_regs{0}, g_mr_hits{0}, g_mr_dmabuf{0};

void release_mr_locked(int dev, rdma::Mr* mr) {
  std::vector<MrSlot>& cache = g_mr_cache[dev];
  for (size_t i = 0; i < cache.size(); ++i) {
    if (cache[i].mr != mr) continue;
    if (--cache[i].refs == 0) {
      g_prov->dereg_mr(mr);
      cache[i] = cache.back();
      cache.pop_back();
    }
    return;
  }
  g_prov->dereg_mr(mr);          // not cached (cannot happen through rdma_reg)
}
}  // namespace

RdmaMrSet* rdma_reg(void* data, size_t size, int dmabuf_fd, uint64_t dmabuf_offset) {
  RdmaMrSet* m = new RdmaMrSet();
  memset(m, 0, sizeof *m);
  m->data = data;
  m->size = size;
  const int flags = access_flags();
  const bool dmabuf = dmabuf_fd >= 0;
  uintptr_t addr = (uintptr_t)data;
  size_t len = size ? size : 1;
  if (!dmabuf) {
    const uintptr_t page = (uintptr_t)sysconf(_SC_PAGESIZE);
    addr = (uintptr_t)data / page * page;
    len = ((uintptr_t)data + len - addr + page - 1) / page * page;
  }
  std::lock_guard<std::mutex> l(g_mr_mu);
  for (int d = 0; d < g_ndev; ++d) {
    // every device gets its own registration so that any of them can carry a stripe (the reference registers
    // every per-GPU alias on every NIC, src/plugin.cc:1250-1320)
    for (MrSlot& s : g_mr_cache[d]) {
      if (s.addr == addr && s.len == len && s.dmabuf == dmabuf) {
        ++s.refs;
        m->mr[d] = s.mr;
        g_mr_hits.fetch_add(1, std::memory_order_relaxed);
        break;
      }
    }
    if (m->mr[d]) continue;
    rdma::Mr* mr = dmabuf ? g_prov->reg_dmabuf_mr(g_pd[d], dmabuf_fd, dmabuf_offset, len, (uint64_t)addr, flags)
                          : g_prov->reg_mr(g_pd[d], reinterpret_cast<void*>(addr), len, flags);
    if (!mr) {
      FL_WARN("rdma: registration of %zu bytes at %p failed on device %d%s", size, data, d, dmabuf ? " (dma-buf)" : "");
      for (int k = 0; k < d; ++k) release_mr_locked(k, m->mr[k]);
      delete m;
      return nullptr;
    }
    g_mr_regs.fetch_add(1, std::memory_order_relaxed);
    if (dmabuf) g_mr_dmabuf.fetch_add(1, std::memory_order_relaxed);
    g_mr_cache[d].push_back(MrSlot{addr, len, dmabuf, 1, mr});
    m->mr[d] = mr;
  }
  return m;
}

void rdma_dereg(RdmaMrSet* m) {
  if (!m) return;
  std::lock_guard<std::mutex> l(g_mr_mu);
  for (int d = 0; d < kMaxDev; ++d)
    if (m->mr[d]) release_mr_locked(d, m->mr[d]);
  delete m;
}

bool rdma_dmabuf_supported() {
  if (!g_prov || g_ndev <= 0) return false;
  for (int d = 0; d < g_ndev; ++d)
    if (!g_prov->dmabuf_supported(d)) return false;      // a stripe may take any device: all of them or none
  return true;
}
bool rdma_peer_memory_supported() { return g_prov && g_ndev > 0 && g_prov->peer_memory_supported(); }

void rdma_mr_counters(unsigned long long* registrations, unsigned long long* cache_hits, unsigned long long* dmabuf) {
  *registrations = g_mr_regs.load();
  *cache_hits = g_mr_hits.load();
  *dmabuf = g_mr_dmabuf.load();
}

ncclResult_t rdma_listen(int dev, int channel_id, Handle* h, RdmaListenComm** out) {
  memset(h, 0, NCCL_NET_HANDLE_MAXSIZE);
  sockaddr_in6 addr;
  pick_listen_addr(&addr);
  addr.sin6_port = 0;
  int fd = socket(AF_INET6, SOCK_STREAM, 0);
  if (fd < 0) return ncclSystemError;
  int zero = 0, one = 1;
  setsockopt(fd, IPPROTO_IPV6, IPV6_V6ONLY, &zero, sizeof zero);
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  if (bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || listen(fd, 256) != 0) {
    close(fd);
    return ncclSystemError;
  }
  socklen_t len = sizeof addr;
  getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  set_nonblock_nodelay(fd);
  RdmaListenComm* lc = new RdmaListenComm();
  lc->fd = fd;
  lc->dev = dev;
  lc->channel_id = channel_id;
  h->magic = kHandleMagic;
  h->addr = addr;
  h->channel_id = channel_id;
  h->ndev = g_ndev;
  h->listen_dev = dev;
  *out = lc;
  return ncclSuccess;
}

static int clamp_qps() {
  int64_t n = params().ib_qps_per_conn;
  if (n < 1) n = 1;
  if (n > kRdmaMaxQps) n = kRdmaMaxQps;
  return (int)n;
}

// Sender: stage 0 TCP connect, 1 hello + own info, 2 peer info + queue pairs to RTS + "ready".
ncclResult_t rdma_connect(int dev, Handle* h, RdmaComm** out) {
  *out = nullptr;
  if (h->magic != kHandleMagic) return ncclInvalidArgument;
  RdmaComm* c = reinterpret_cast<RdmaComm*>(h->connect_state);
  auto abandon = [&](ncclResult_t rc, const char* why) {
    FL_WARN("rdma connect: %s", why);
    h->connect_state = nullptr;
    rdma_close(c);
    return rc;
  };
  if (!c) {
    c = new RdmaComm();
    c->is_send = true;
    c->own_dev = dev;
    c->peer_dev = h->listen_dev;
    c->ndev = h->ndev < g_ndev ? h->ndev : g_ndev;
    c->nqps = clamp_qps();
    c->channel_id = h->channel_id;
    c->ctrl_fd = socket(AF_INET6, SOCK_STREAM, 0);
    h->connect_state = c;
    if (c->ctrl_fd < 0) return abandon(ncclSystemError, "no socket");
    set_nonblock_nodelay(c->ctrl_fd);
    if (connect(c->ctrl_fd, reinterpret_cast<sockaddr*>(&h->addr), sizeof h->addr) != 0 && errno != EINPROGRESS)
      return abandon(ncclSystemError, strerror(errno));
    c->stage = 0;
  }
  if (c->stage == 0) {
    pollfd pfd{c->ctrl_fd, POLLOUT, 0};
    if (poll(&pfd, 1, 0) <= 0 || !(pfd.revents & (POLLOUT | POLLERR | POLLHUP))) return ncclSuccess;
    int err = 0;
    socklen_t el = sizeof err;
    getsockopt(c->ctrl_fd, SOL_SOCKET, SO_ERROR, &err, &el);
    if (err) return abandon(ncclSystemError, strerror(err));
    Hello hello;
    memset(&hello, 0, sizeof hello);
    hello.magic = kHelloMagic;
    hello.comm_uid = g_uid.fetch_add(1);
    hello.kind = 2;
    hello.dev = -1;
    hello.sender_dev = c->own_dev;
    hello.ndev = c->ndev;
    if (send(c->ctrl_fd, &hello, sizeof hello, MSG_NOSIGNAL) != (ssize_t)sizeof hello) return abandon(ncclSystemError, "hello not sent");
    if (!make_endpoints(c)) return abandon(ncclSystemError, "cannot create queue pairs");
    c->fifo = reinterpret_cast<RdmaDesc*>(alloc_zeroed(sizeof(RdmaDesc) * kMaxRequests));
    c->done_src = reinterpret_cast<RdmaDoneRec*>(alloc_zeroed(sizeof(RdmaDoneRec) * kMaxRequests));
    if (!c->fifo || !c->done_src) return abandon(ncclSystemError, "out of memory");
    c->fifo_mr = rdma_reg(c->fifo, sizeof(RdmaDesc) * kMaxRequests);
    c->done_src_mr = rdma_reg(c->done_src, sizeof(RdmaDoneRec) * kMaxRequests);
    if (!c->fifo_mr || !c->done_src_mr) return abandon(ncclSystemError, "cannot register the FIFO");
    c->mine.fifo_addr = (uint64_t)(uintptr_t)c->fifo;
    for (int d = 0; d < c->ndev; ++d) c->mine.fifo_rkey[d] = c->fifo_mr->mr[d]->rkey;
    c->io_done = 0;
    c->stage = 1;
  }
  if (c->stage == 1) {
    const int rc = io_step(c->ctrl_fd, &c->mine, sizeof c->mine, &c->io_done, true);
    if (rc < 0) return abandon(ncclSystemError, "bootstrap socket closed");
    if (rc == 0) return ncclSuccess;
    c->io_done = 0;
    c->stage = 2;
  }
  if (c->stage == 2) {
    const int rc = io_step(c->ctrl_fd, &c->theirs, sizeof c->theirs, &c->io_done, false);
    if (rc < 0) return abandon(ncclSystemError, "bootstrap socket closed");
    if (rc == 0) return ncclSuccess;
    if (c->theirs.magic != kInfoMagic || c->theirs.ndev != c->ndev || c->theirs.nqps != c->nqps)
      return abandon(ncclInternalError, "peer disagrees on devices / queue pairs per connection");
    if (!connect_endpoints(c)) return abandon(ncclSystemError, "cannot connect queue pairs");
    c->remote_done_addr = c->theirs.done_addr;
    memcpy(c->remote_done_rkey, c->theirs.done_rkey, sizeof c->remote_done_rkey);
    const uint8_t ready = 1;
    if (send(c->ctrl_fd, &ready, 1, MSG_NOSIGNAL) != 1) return abandon(ncclSystemError, "ready not sent");
    c->stage = 3;
    h->connect_state = nullptr;
    *out = c;
  }
  return ncclSuccess;
}

// Receiver: per pending connection, stage 0 hello, 1 peer info, then endpoints + receives + own info, 2 "ready".
ncclResult_t rdma_accept(RdmaListenComm* lc, RdmaComm** out) {
  *out = nullptr;
  for (;;) {
    int fd = accept(lc->fd, nullptr, nullptr);
    if (fd < 0) break;
    set_nonblock_nodelay(fd);
    RdmaComm* c = new RdmaComm();
    c->is_send = false;
    c->own_dev = lc->dev;
    c->channel_id = lc->channel_id;
    c->ctrl_fd = fd;
    c->stage = 0;
    c->io_done = 0;
    c->since_ns = now_ns();
    lc->pending.push_back(c);
  }
  for (size_t i = 0; i < lc->pending.size();) {
    RdmaComm* c = lc->pending[i];
    auto drop = [&](const char* why) {
      FL_WARN("rdma accept: dropping a connection: %s", why);
      rdma_close(c);
      lc->pending.erase(lc->pending.begin() + i);
    };
    const uint64_t age = now_ns() - c->since_ns;
    if ((c->stage == 0 && age > kHelloTimeoutNs) || age > kPartialTimeoutNs) {
      drop("bootstrap stalled");
      continue;
    }
    if (c->stage == 0) {
      static_assert(sizeof(Hello) <= sizeof(RdmaConnInfo), "hello is staged in the info buffer");
      const int rc = io_step(c->ctrl_fd, &c->theirs, sizeof(Hello), &c->io_done, false);
      if (rc < 0) { drop("closed before the hello"); continue; }
      if (rc == 0) { ++i; continue; }
      Hello hello;
      memcpy(&hello, &c->theirs, sizeof hello);
      if (hello.magic != kHelloMagic || hello.kind != 2 || hello.ndev < 1 || hello.ndev > kMaxDev) { drop("bad hello"); continue; }
      c->peer_dev = hello.sender_dev;
      c->io_done = 0;
      c->stage = 1;
    }
    if (c->stage == 1) {
      const int rc = io_step(c->ctrl_fd, &c->theirs, sizeof c->theirs, &c->io_done, false);
      if (rc < 0) { drop("closed during the exchange"); continue; }
      if (rc == 0) { ++i; continue; }
      if (c->theirs.magic != kInfoMagic || c->theirs.ndev < 1 || c->theirs.ndev > g_ndev || c->theirs.nqps < 1 || c->theirs.nqps > kRdmaMaxQps) {
        drop("bad connection info");
        continue;
      }
      c->ndev = c->theirs.ndev;
      c->nqps = c->theirs.nqps;
      c->ctrl_dev = c->own_dev % c->ndev;
      bool ok = make_endpoints(c);
      c->done = reinterpret_cast<RdmaDoneRec*>(alloc_zeroed(sizeof(RdmaDoneRec) * kMaxRequests));
      c->fifo_src = reinterpret_cast<RdmaDesc*>(alloc_zeroed(sizeof(RdmaDesc) * kMaxRequests));
      ok = ok && c->done && c->fifo_src;
      if (ok) {
        c->done_mr = rdma_reg(c->done, sizeof(RdmaDoneRec) * kMaxRequests);
        c->fifo_src_mr = rdma_reg(c->fifo_src, sizeof(RdmaDesc) * kMaxRequests);
        ok = c->done_mr && c->fifo_src_mr;
      }
      ok = ok && connect_endpoints(c);
      if (ok) {
        // zero-length receives for every write-with-immediate that can be outstanding, on every queue pair.  (Receives
        // cannot be posted to a queue pair that is still in the RESET state, hence after the transitions; no immediate
        // can arrive earlier, because the sender only writes in answer to descriptors this side has not posted yet.)
        for (int d = 0; d < c->ndev && ok; ++d)
          for (int q = 0; q < c->nqps && ok; ++q)
            for (int k = 0; k < kMaxRequests && ok; ++k) ok = g_prov->post_recv(c->dev[d].qp[q], kWrRecv) == 0;
      }
      if (ok && !params().gdr_flush_disable) {
        rdma::QpCaps fc;
        fc.max_send_wr = kMaxRequests;
        fc.max_recv_wr = 1;
        c->flush_qp = g_prov->create_qp(g_pd[c->ctrl_dev], c->dev[c->ctrl_dev].cq, fc);
        c->flush_buf = reinterpret_cast<uint8_t*>(alloc_zeroed(64));
        rdma::QpInfo self;
        rdma::QpConnectParams qp;
        ok = c->flush_qp && c->flush_buf && g_prov->query_qp_info(c->flush_qp, (int)params().ib_gid_index, &self) == 0 &&
             g_prov->connect_qp(c->flush_qp, self, qp) == 0;
        if (ok) c->flush_mr = rdma_reg(c->flush_buf, 64);
        ok = ok && c->flush_mr;
      }
      if (!ok) { drop("cannot set up queue pairs"); continue; }
      c->remote_fifo_addr = c->theirs.fifo_addr;
      memcpy(c->remote_fifo_rkey, c->theirs.fifo_rkey, sizeof c->remote_fifo_rkey);
      c->mine.done_addr = (uint64_t)(uintptr_t)c->done;
      for (int d = 0; d < c->ndev; ++d) c->mine.done_rkey[d] = c->done_mr->mr[d]->rkey;
      size_t sent = 0;
      // a few KB into an empty socket buffer: completes at once; anything else is treated as a failure
      if (io_step(c->ctrl_fd, &c->mine, sizeof c->mine, &sent, true) != 1) { drop("cannot send the connection info"); continue; }
      c->io_done = 0;
      c->stage = 2;
    }
    if (c->stage == 2) {
      uint8_t ready = 0;
      const int rc = io_step(c->ctrl_fd, &ready, 1, &c->io_done, false);
      if (rc < 0) { drop("closed before ready"); continue; }
      if (rc == 0) { ++i; continue; }
      lc->pending.erase(lc->pending.begin() + i);
      c->stage = 3;
      c->cur_dev = -1;
      *out = c;
      return ncclSuccess;
    }
    ++i;
  }
  return ncclSuccess;
}

// -----------------------------------------------------------------------------------------------------
ncclResult_t rdma_isend(RdmaComm* c, ConnManager* cm, void* data, int size, int tag, RdmaMrSet* mr, RdmaRequest** out) {
  *out = nullptr;
  ScopedTimer tm(&c->timers, T_ISEND, params().timers != 0);
  if (c->error) return (ncclResult_t)c->error;
  if (size < 0 || !mr) return ncclInvalidArgument;
  poll_all(c, cm);
  if (c->error) return (ncclResult_t)c->error;
  RdmaDesc* slot = &c->fifo[c->fifo_head % kMaxRequests];
  // the NIC writes this memory; the sequence word is the last one of the entry to land
  if (__atomic_load_n(&slot->seq, __ATOMIC_ACQUIRE) != c->fifo_head + 1) return ncclSuccess;   // the receiver has not posted yet
  RdmaDesc d;
  memcpy(&d, slot, sizeof d);
  if (d.tag != tag) {
    FL_WARN("rdma isend: tag mismatch (posted %d, sending %d)", d.tag, tag);
    return ncclInternalError;
  }
  if ((uint64_t)size > d.size) {
    FL_WARN("rdma isend: message of %d bytes does not fit the posted receive of %llu bytes", size, (unsigned long long)d.size);
    return ncclInvalidUsage;                                       // src/plugin.cc:1555-1570
  }
  RdmaRequest* r = get_request(c);
  if (!r) return ncclSuccess;
  c->fifo_head++;
  r->is_send = true;
  r->size = (uint64_t)size;
  r->tag = tag;

  // plan: stripes over devices, each stripe over the queue pairs of its device
  const Params& p = params();
  const int first = cm->bid_tx(c->channel_id, c->own_dev, d.proposed_dev) % c->ndev;
  int nstripes = (int)p.degree;
  if (nstripes > c->ndev) nstripes = c->ndev;
  if (nstripes < 1) nstripes = 1;
  while (nstripes > 1 && (uint64_t)size / (uint64_t)nstripes < (uint64_t)p.min_stripe_bytes) --nstripes;
  const int per_dev_qps = (p.ib_split_data_on_qps && c->nqps > 1 && (uint64_t)size >= 128ull * c->nqps * nstripes) ? c->nqps : 1;
  const int npieces = nstripes * per_dev_qps;
  const uint64_t per = npieces > 1 ? ((uint64_t)size / (uint64_t)npieces) & ~127ull : (uint64_t)size;
  c->done_src[d.slot % kMaxRequests].size = (uint64_t)size;
  c->done_src[d.slot % kMaxRequests].tx_mask = cm->tx_mask(c->own_dev);
  r->data = reinterpret_cast<const uint8_t*>(data);
  r->mr = mr;
  r->desc = d;
  r->bad_key = p.fault_bad_rkey_after > 0 && (int64_t)c->msg_index + 1 == p.fault_bad_rkey_after;

  uint64_t off = 0;
  int dev = first, piece = 0;
  uint64_t used = 0;
  for (int s = 0; s < nstripes; ++s) {
    if (s > 0) {                              // further stripes: a device the monitor showed idle, kept for the connection
      int& held = c->extra_dev[s];
      if (held >= 0 && (c->dead[held] || ((used >> held) & 1ull))) {
        cm->release_tx(held);
        held = -1;
      }
      if (held < 0) {
        const int b = cm->borrow_tx(c->own_dev, used, dev);
        if (b >= 0 && b < c->ndev && !c->dead[b]) held = b;
        else if (b >= 0) cm->release_tx(b);
      }
      if (held >= 0) dev = held;
    }
    dev = rdma_next_alive(c, dev);            // devices given up earlier are skipped
    if (dev < 0) {
      fail(c, ncclRemoteError, "every device of the connection is gone");
      r->used = false;
      return ncclRemoteError;
    }
    for (int k = 0; k < per_dev_qps; ++k, ++piece) {
      const uint64_t len = piece == npieces - 1 ? (uint64_t)size - off : per;
      const int q = per_dev_qps > 1 ? k : (int)(c->msg_index % (uint64_t)c->nqps);
      RdmaPiece pc;
      pc.dev = dev; pc.q = q; pc.off = off; pc.len = len;
      r->pieces.push_back(pc);
      off += len;
    }
    used |= 1ull << dev;
    dev = (dev + (int)(p.step > 0 ? p.step : 1)) % c->ndev;
  }
  for (int pi = 0; pi < npieces; ++pi) {
    if (!post_piece(c, r, pi)) {
      fail(c, ncclSystemError, "post_send failed");
      r->used = false;
      return ncclSystemError;
    }
    cm->mark_tx(r->pieces[pi].dev, r->pieces[pi].len);
  }
  r->pieces_total = npieces;
  c->msg_index++;
  g_messages.fetch_add(1, std::memory_order_relaxed);
  poll_all(c, cm);
  *out = r;
  return ncclSuccess;
}

ncclResult_t rdma_irecv(RdmaComm* c, ConnManager* cm, void* data, int size, int tag, RdmaMrSet* mr, RdmaRequest** out) {
  *out = nullptr;
  ScopedTimer tm(&c->timers, T_IRECV, params().timers != 0);
  if (c->error) return (ncclResult_t)c->error;
  if (size < 0 || !mr) return ncclInvalidArgument;
  RdmaRequest* r = get_request(c);
  if (!r) return ncclSuccess;
  r->is_send = false;
  r->size = (uint64_t)size;
  r->tag = tag;
  const bool quiescent = c->posted == c->completed;
  if (c->cur_dev < 0 || (c->n_finished >= kFinishedBatch && quiescent)) {
    c->cur_dev = cm->refresh_rx(c->channel_id, c->own_dev, c->cur_dev, c->peer_tx_mask, quiescent);
    c->n_finished = 0;
  }
  r->rx_dev = c->cur_dev;
  const uint64_t idx = c->fifo_tail;
  RdmaDesc* d = &c->fifo_src[idx % kMaxRequests];
  memset(d, 0, sizeof *d);
  d->addr = (uint64_t)(uintptr_t)data;
  d->size = r->size;
  d->tag = tag;
  d->slot = r->slot;
  d->proposed_dev = c->cur_dev;
  for (int k = 0; k < c->ndev; ++k) d->rkey[k] = mr->mr[k]->rkey;
  d->seq = idx + 1;
  r->fifo_idx = idx;
  if (c->dead[c->ctrl_dev] && rdma_next_alive(c, c->ctrl_dev) >= 0) c->ctrl_dev = rdma_next_alive(c, c->ctrl_dev);
  {
    ScopedTimer tp(&c->timers, T_POST_DESC, params().timers != 0);
    if (!post_descriptor(c, idx)) {
      fail(c, ncclSystemError, "descriptor write failed");
      r->used = false;
      return ncclSystemError;
    }
  }
  c->fifo_tail++;
  cm->mark_rx(c->cur_dev, r->size);
  c->posted++;
  poll_all(c, cm);
  *out = r;
  return ncclSuccess;
}

ncclResult_t rdma_iflush(RdmaComm* c, ConnManager* cm, void* data, int size, RdmaMrSet* mr, RdmaRequest** out) {
  *out = nullptr;
  ScopedTimer tm(&c->timers, T_FLUSH, params().timers != 0);
  if (!c->flush_qp || size <= 0 || !mr) return ncclSuccess;
  if (c->error) return (ncclResult_t)c->error;
  RdmaRequest* r = get_request(c);
  if (!r) return ncclInternalError;
  r->is_flush = true;
  r->is_send = true;                       // nothing of the receive bookkeeping applies
  r->size = 0;
  rdma::SendWr wr;
  wr.wr_id = kWrFlush | r->slot;
  wr.op = rdma::kRead;
  wr.laddr = c->flush_buf;
  wr.len = 1;
  wr.lkey = c->flush_mr->mr[c->ctrl_dev]->lkey;
  wr.raddr = (uint64_t)(uintptr_t)data;
  wr.rkey = mr->mr[c->ctrl_dev]->rkey;
  wr.signaled = true;
  if (g_prov->post_send(c->flush_qp, &wr, 1) != 0) {
    r->used = false;
    fail(c, ncclSystemError, "flush read failed");
    return ncclSystemError;
  }
  poll_all(c, cm);
  *out = r;
  return ncclSuccess;
}

ncclResult_t rdma_test(RdmaRequest* r, ConnManager* cm, int* done, int* size) {
  RdmaComm* c = r->comm;
  *done = 0;
  poll_all(c, cm);
  if (r->pieces_total >= 0 && r->pieces_done >= r->pieces_total) {
    if (!r->is_send) {
      const RdmaDoneRec rec = c->done[r->slot];
      if (rec.size > r->size) {
        fail(c, ncclInvalidUsage, "message larger than the posted receive");
        return ncclInvalidUsage;
      }
      r->total = rec.size;
      c->peer_tx_mask = rec.tx_mask;
      c->completed++;
      c->n_finished++;
      cm->done_rx(r->rx_dev, r->size);
    }
    *done = 1;
    if (size) *size = (int)(r->is_send ? r->size : r->total);
    r->used = false;
    return ncclSuccess;
  }
  if (c->error) return (ncclResult_t)c->error;
  const uint64_t limit_ns = (uint64_t)params().net_timeout_ms * 1000000ull;
  if (limit_ns && now_ns() - r->last_progress_ns > limit_ns) {
    FL_WARN("rdma %s request on channel %d made no progress for %ld ms: giving up", r->is_send ? "send" : "recv", c->channel_id,
            (long)params().net_timeout_ms);
    c->error = ncclRemoteError;
    return ncclRemoteError;
  }
  return ncclSuccess;
}

void rdma_close(RdmaComm* c) {
  if (!c) return;
  if (params().timers && c->stage == 3) c->timers.print(c->is_send ? "rdma send" : "rdma recv");
  if (c->flush_qp) g_prov->destroy_qp(c->flush_qp);      // queue pairs go before the completion queue they use
  for (int d = 0; d < kMaxDev; ++d) {
    for (int q = 0; q < kRdmaMaxQps; ++q)
      if (c->dev[d].qp[q]) g_prov->destroy_qp(c->dev[d].qp[q]);
    if (c->dev[d].cq) g_prov->destroy_cq(c->dev[d].cq);
  }
  rdma_dereg(c->flush_mr);
  free(c->flush_buf);
  rdma_dereg(c->fifo_mr);
  rdma_dereg(c->done_src_mr);
  rdma_dereg(c->done_mr);
  rdma_dereg(c->fifo_src_mr);
  free(c->fifo);
  free(c->done_src);
  free(c->done);
  free(c->fifo_src);
  if (c->ctrl_fd >= 0) close(c->ctrl_fd);
  delete c;
}

void rdma_close_listen(RdmaListenComm* lc) {
  if (!lc) return;
  for (RdmaComm* c : lc->pending) rdma_close(c);
  if (lc->fd >= 0) close(lc->fd);
  delete lc;
}

unsigned long long rdma_failovers() { return g_failovers.load(); }

void rdma_counters(unsigned long long* m, unsigned long long* p, unsigned long long* w) {
  *m = g_messages.load();
  *p = g_pieces.load();
  *w = g_work_requests.load();
}

}  // namespace flnet

// Registration counters: registrations made, requests answered from the cache, registrations that went through a dma-buf.
extern "C" __attribute__((visibility("default"))) void fuselink_rdma_mr_counters(unsigned long long* registrations, unsigned long long* cache_hits,
                                                                               unsigned long long* dmabuf) {
  flnet::rdma_mr_counters(registrations, cache_hits, dmabuf);
}
extern "C" __attribute__((visibility("default"))) unsigned long long fuselink_rdma_failovers(void) { return flnet::rdma_failovers(); }

// Counters for tests and tools: messages sent, pieces they were cut into, work requests posted for them.
extern "C" __attribute__((visibility("default"))) void fuselink_rdma_counters(unsigned long long* messages, unsigned long long* pieces,
                                                                            unsigned long long* work_requests) {
  flnet::rdma_counters(messages, pieces, work_requests);
}
