// Entry points of the TCP transport: listen / connect / accept, isend / irecv / test (the progress engine they drive is
// in tcp_transport.cc, the protocol in tcp_transport.h).  plugin.cc maps the ncclNet tables onto these and onto their RDMA
// counterparts in rdma_transport.cc.
#include <arpa/inet.h>
#include <errno.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <random>

#include "logging.h"
#include "nvl_channel.h"
#include "params.h"
#include "tcp_transport.h"
#include "../mem/vmm.h"

namespace flnet {
namespace {

constexpr uint64_t kHelloMagic = 0x464c4e4b48454c4full;  // "FLNKHELO"
constexpr uint32_t kDescMagic = 0x464c4453u;
constexpr uint32_t kFrameMagic = 0x464c4652u;
constexpr uint32_t kFrameDirectMagic = 0x464c4452u;

std::atomic<uint64_t> g_direct_bytes{0};     // payload bytes that went through the direct path (sender side)
std::atomic<uint64_t> g_direct_msgs{0};

Request* get_request(Comm* c) {
  // slots are handed out round-robin so a slot is not reused while frames of its previous use may be in flight
  static thread_local int hint = 0;
  for (int i = 0; i < kMaxRequests; ++i) {
    const int s = (hint + i) % kMaxRequests;
    if (!c->reqs[s].used) {
      hint = s + 1;
      Request& r = c->reqs[s];
      r = Request();
      r.used = true;
      r.comm = c;
      r.slot = (uint32_t)s;
      r.last_progress_ns = now_ns();
      return &r;
    }
  }
  return nullptr;
}

}  // namespace

uint64_t random_u64() {
  static std::mt19937_64 rng{std::random_device{}()};
  static std::mutex mu;
  std::lock_guard<std::mutex> l(mu);
  return rng();
}

uint64_t tcp_direct_bytes() { return g_direct_bytes.load(); }
uint64_t tcp_direct_msgs() { return g_direct_msgs.load(); }

ncclResult_t tcp_listen(int dev, int ndev, int channel_id, bool offer_nvl, Handle* h, ListenComm** out) {
  *out = nullptr;
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
    FL_WARN("listen: bind/listen failed: %s", strerror(errno));
    close(fd);
    return ncclSystemError;
  }
  socklen_t len = sizeof addr;
  getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  set_nonblock_nodelay(fd);
  ListenComm* lc = new ListenComm();
  lc->fd = fd;
  lc->dev = dev;
  lc->channel_id = channel_id;                         // global channel id, carried in the handle (src/plugin.cc:690-698)
  h->magic = kHandleMagic;
  h->addr = addr;
  h->channel_id = lc->channel_id;
  h->ndev = ndev;
  h->listen_dev = dev;
  if (offer_nvl) {
    // same-host side channel for cuMem handles; failing to set it up only means every peer stays on TCP
    const uint64_t token = random_u64() | 1ull;
    int ufd = socket(AF_UNIX, SOCK_SEQPACKET | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
    sockaddr_un sa;
    socklen_t sl;
    nvl_sockaddr(token, &sa, &sl);
    if (ufd >= 0 && bind(ufd, reinterpret_cast<sockaddr*>(&sa), sl) == 0 && listen(ufd, 64) == 0) {
      lc->uds_fd = ufd;
      lc->nvl_token = token;
      h->nvl_token = token;
    } else if (ufd >= 0) {
      close(ufd);
    }
  }
  *out = lc;
  return ncclSuccess;
}

// connect(): re-entered until *send_comm != NULL.  Stage 0 starts one control and ndev data connections,
// stage 1 finishes the TCP handshakes and sends the hellos.  All data sockets are set up eagerly (the
// reference builds its per-NIC side comms eagerly too, src/plugin.cc:727-753) so switching device later costs
// nothing.
ncclResult_t tcp_connect(int dev, int ndev, bool want_nvl, Handle* h, Comm** out) {
  *out = nullptr;
  Comm* c = reinterpret_cast<Comm*>(h->connect_state);
  if (!c) {
    c = new Comm();
    c->is_send = true;
    c->own_dev = dev;
    c->peer_dev = h->listen_dev;
    c->ndev = h->ndev < ndev ? h->ndev : ndev;
    c->channel_id = h->channel_id;
    c->uid = random_u64();
    const int nsock = 1 + c->ndev;
    for (int i = 0; i < nsock; ++i) {
      int fd = socket(AF_INET6, SOCK_STREAM, 0);
      if (fd < 0) { comm_close(c); return ncclSystemError; }
      set_nonblock_nodelay(fd);
      int rc = connect(fd, reinterpret_cast<sockaddr*>(&h->addr), sizeof h->addr);
      if (rc != 0 && errno != EINPROGRESS) {
        FL_WARN("connect: %s", strerror(errno));
        close(fd);
        comm_close(c);
        return ncclSystemError;
      }
      c->pending_fds.push_back(fd);
      c->hello_sent.push_back(0);
    }
    if (h->nvl_token && want_nvl) {
      // the abstract Unix address only resolves on the listener's own machine; a refusal means "remote peer"
      int ufd = socket(AF_UNIX, SOCK_SEQPACKET | SOCK_CLOEXEC, 0);
      sockaddr_un sa;
      socklen_t sl;
      nvl_sockaddr(h->nvl_token, &sa, &sl);
      const uint64_t hello[2] = {kNvlMagic, c->uid};
      if (ufd >= 0 && connect(ufd, reinterpret_cast<sockaddr*>(&sa), sl) == 0 &&
          send(ufd, hello, sizeof hello, MSG_NOSIGNAL) == (ssize_t)sizeof hello) {
        c->nvl_fd = ufd;
      } else if (ufd >= 0) {
        close(ufd);
      }
    }
    h->connect_state = c;
  }
  bool all = true;
  for (size_t i = 0; i < c->pending_fds.size(); ++i) {
    if (c->hello_sent[i] == sizeof(Hello)) continue;
    const int fd = c->pending_fds[i];
    pollfd pfd{fd, POLLOUT, 0};
    if (poll(&pfd, 1, 0) <= 0 || !(pfd.revents & (POLLOUT | POLLERR | POLLHUP))) { all = false; continue; }
    int err = 0;
    socklen_t el = sizeof err;
    getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &el);
    if ((err == ECONNREFUSED || err == ETIMEDOUT) && c->connect_retries < params().connect_retries) {
      // the listener may not be up yet (or its backlog is full): try again a little later, within a budget
      c->connect_retries++;
      close(fd);
      usleep(1000);
      int nfd = socket(AF_INET6, SOCK_STREAM, 0);
      if (nfd >= 0) {
        set_nonblock_nodelay(nfd);
        int rc2 = connect(nfd, reinterpret_cast<sockaddr*>(&h->addr), sizeof h->addr);
        if (rc2 != 0 && errno != EINPROGRESS) { close(nfd); nfd = -1; }
      }
      if (nfd >= 0) {
        c->pending_fds[i] = nfd;
        all = false;
        continue;
      }
      err = errno ? errno : ECONNREFUSED;
    }
    if (err) {
      FL_WARN("connect to listener failed after %d retries: %s", c->connect_retries, strerror(err));
      c->pending_fds[i] = -1;
      h->connect_state = nullptr;
      comm_close(c);
      return ncclSystemError;
    }
    Hello hello;
    memset(&hello, 0, sizeof hello);
    hello.magic = kHelloMagic;
    hello.comm_uid = c->uid;
    hello.kind = i == 0 ? 0 : 1;
    hello.dev = i == 0 ? (c->nvl_fd >= 0 ? -2 : -1) : (int)i - 1;   // control hello: -2 announces a side channel
    hello.sender_dev = c->own_dev;
    hello.ndev = c->ndev;
    ssize_t r = send(fd, reinterpret_cast<uint8_t*>(&hello) + c->hello_sent[i], sizeof hello - c->hello_sent[i], MSG_DONTWAIT | MSG_NOSIGNAL);
    if (r > 0) c->hello_sent[i] += (size_t)r;
    if (c->hello_sent[i] < sizeof(Hello)) all = false;
  }
  if (!all) return ncclSuccess;
  c->ctrl_fd = c->pending_fds[0];
  for (int d = 0; d < c->ndev; ++d) c->data[d].fd = c->pending_fds[1 + d];
  c->pending_fds.clear();
  h->connect_state = nullptr;
  *out = c;
  return ncclSuccess;
}

ncclResult_t tcp_accept(ListenComm* lc, Comm** out) {
  *out = nullptr;
  for (;;) {
    int fd = accept(lc->fd, nullptr, nullptr);
    if (fd < 0) break;
    set_nonblock_nodelay(fd);
    PendingSock ps;
    ps.fd = fd;
    ps.got = 0;
    ps.since_ns = now_ns();
    lc->pending.push_back(ps);
  }
  while (lc->uds_fd >= 0) {
    int ufd = accept4(lc->uds_fd, nullptr, nullptr, SOCK_CLOEXEC);
    if (ufd < 0) break;
    lc->nvl_pending.push_back({ufd, 0});
  }
  for (size_t i = 0; i < lc->nvl_pending.size();) {
    auto& np = lc->nvl_pending[i];
    if (np.uid == 0) {
      uint64_t hello[2] = {0, 0};
      ssize_t r = recv(np.fd, hello, sizeof hello, MSG_DONTWAIT);
      if (r == (ssize_t)sizeof hello && hello[0] == kNvlMagic && hello[1] != 0) {
        np.uid = hello[1];
      } else if (r >= 0 || (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) {
        close(np.fd);
        lc->nvl_pending.erase(lc->nvl_pending.begin() + i);
        continue;
      }
    }
    ++i;
  }
  for (size_t i = 0; i < lc->pending.size();) {
    PendingSock& ps = lc->pending[i];
    ssize_t r = recv(ps.fd, reinterpret_cast<uint8_t*>(&ps.hello) + ps.got, sizeof(Hello) - ps.got, MSG_DONTWAIT);
    if (r > 0) ps.got += (size_t)r;
    else if (r == 0 || (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) {
      close(ps.fd);                                    // stray or broken connection: drop it (socket.cc:431-437)
      lc->pending.erase(lc->pending.begin() + i);
      continue;
    }
    if (ps.got < sizeof(Hello)) {
      if (now_ns() - ps.since_ns > kHelloTimeoutNs) {   // connected and never introduced itself
        close(ps.fd);
        lc->pending.erase(lc->pending.begin() + i);
        continue;
      }
      ++i;
      continue;
    }
    if (ps.hello.magic != kHelloMagic || ps.hello.ndev < 1 || ps.hello.ndev > kMaxDev ||
        (ps.hello.kind == 1 && (ps.hello.dev < 0 || ps.hello.dev >= ps.hello.ndev))) {
      FL_WARN("accept: dropping a connection with a bad hello");
      close(ps.fd);
      lc->pending.erase(lc->pending.begin() + i);
      continue;
    }
    ListenComm::Partial* part = nullptr;
    for (auto& p : lc->partials) if (p.uid == ps.hello.comm_uid) part = &p;
    if (!part) {
      Comm* c = new Comm();
      c->is_send = false;
      c->own_dev = lc->dev;
      c->peer_dev = ps.hello.sender_dev;
      c->ndev = ps.hello.ndev;
      c->channel_id = lc->channel_id;
      c->uid = ps.hello.comm_uid;
      lc->partials.push_back({ps.hello.comm_uid, c, 0, now_ns()});
      part = &lc->partials.back();
    }
    if (ps.hello.kind == 0 && ps.hello.dev == -2) part->comm->nvl_fd = -2;   // a side channel belongs to this connection
    if (ps.hello.kind == 0) part->comm->ctrl_fd = ps.fd;
    else part->comm->data[ps.hello.dev].fd = ps.fd;
    part->have++;
    lc->pending.erase(lc->pending.begin() + i);
  }
  for (size_t i = 0; i < lc->partials.size();) {        // connections whose remaining sockets never came
    if (now_ns() - lc->partials[i].since_ns > kPartialTimeoutNs && lc->partials[i].have < 1 + lc->partials[i].comm->ndev) {
      FL_WARN("accept: dropping a connection that stayed incomplete (%d of %d sockets)", lc->partials[i].have, 1 + lc->partials[i].comm->ndev);
      comm_close(lc->partials[i].comm);
      lc->partials.erase(lc->partials.begin() + i);
    } else {
      ++i;
    }
  }
  for (size_t i = 0; i < lc->partials.size(); ++i) {
    if (lc->partials[i].have == 1 + lc->partials[i].comm->ndev) {
      Comm* c = lc->partials[i].comm;
      if (c->nvl_fd == -2) {
        // the sender connected its side channel before it sent the hello, so it is in the backlog by now
        for (size_t k = 0; k < lc->nvl_pending.size(); ++k) {
          if (lc->nvl_pending[k].uid == c->uid) {
            c->nvl_fd = lc->nvl_pending[k].fd;
            lc->nvl_pending.erase(lc->nvl_pending.begin() + k);
            break;
          }
        }
        if (c->nvl_fd == -2) continue;             // its hello has not been read yet: next call
      }
      lc->partials.erase(lc->partials.begin() + i);
      c->cur_dev = -1;
      *out = c;
      return ncclSuccess;
    }
  }
  return ncclSuccess;
}

ncclResult_t tcp_isend(Comm* c, ConnManager* cm, void* data, int size, int tag, const TcpMem* mem, Request** out) {
  *out = nullptr;
  ScopedTimer tm(&c->timers, T_ISEND, params().timers != 0);
  if (c->error) return (ncclResult_t)c->error;
  if (size < 0) return ncclInvalidArgument;
  comm_progress(c, cm);
  if (c->error) return (ncclResult_t)c->error;
  if (c->fifo.empty()) return ncclSuccess;          // the receiver has not posted yet: try again later
  const RecvDesc d = c->fifo.front();
  if (d.tag != tag) {
    FL_WARN("isend: tag mismatch (posted %d, sending %d)", d.tag, tag);
    return ncclInternalError;
  }
  if ((uint64_t)size > d.size) {
    FL_WARN("isend: message of %d bytes does not fit the posted receive of %llu bytes", size, (unsigned long long)d.size);
    return ncclInvalidUsage;
  }
  const TcpMem* mh = mem;
  if (c->nvl_fd >= 0 && !c->peer_mrs.empty()) nvl_ingest(c, 0);     // notices of regions the peer has deregistered
  // Direct path: the receiver exported the buffer of this descriptor.  Its announcement travels on another
  // socket than the descriptor, so it may not be here yet: come back later rather than fall back.
  uint8_t* direct_dst = nullptr;
  if ((d.flags & kDescDirectOk) && c->nvl_fd >= 0 && size > 0) {
    const Comm::PeerMr* pm = nullptr;
    for (int pass = 0; pass < 2 && !pm; ++pass) {
      for (auto& m : c->peer_mrs) if (m.id == d.mr_id) pm = &m;
      if (!pm && pass == 0) nvl_ingest(c, mh && mh->type == NCCL_PTR_CUDA ? fl_vmm_pointer_device(data) : 0);
    }
    if (!pm && c->nvl_fd >= 0) return ncclSuccess;
    if (pm && pm->base && d.mr_off + (uint64_t)size <= pm->size) direct_dst = reinterpret_cast<uint8_t*>(pm->base) + d.mr_off;
  }
  Request* r = get_request(c);
  if (!r) {
    FL_WARN("isend: out of request slots");        // src/plugin.cc:1082-1084
    return ncclInternalError;
  }
  c->fifo.pop_front();
  r->is_send = true;
  r->data = reinterpret_cast<uint8_t*>(data);
  r->size = (uint64_t)size;
  r->tag = tag;
  if (direct_dst && fl_vmm_memcpy(direct_dst, data, (size_t)size) == 0) {
    // the payload is in place: one header-only frame on the proposed device tells the receiver
    int dev0 = next_alive_dev(c, cm->bid_tx(c->channel_id, c->own_dev, d.proposed_dev) % c->ndev);
    if (dev0 < 0) dev0 = 0;
    Stripe st;
    st.dev = dev0;
    st.hdr.magic = kFrameDirectMagic;
    st.hdr.slot = d.slot;
    st.hdr.total = (uint64_t)size;
    st.hdr.offset = 0;
    st.hdr.len = 0;
    st.hdr.tx_mask = cm->tx_mask(c->own_dev);
    r->stripes.push_back(st);
    c->data[dev0].txq.emplace_back(r, 0);
    r->moved = (uint64_t)size;
    g_direct_bytes.fetch_add((uint64_t)size, std::memory_order_relaxed);
    g_direct_msgs.fetch_add(1, std::memory_order_relaxed);
    c->msg_index++;
    comm_progress(c, cm);
    *out = r;
    return ncclSuccess;
  }
  if (direct_dst) FL_WARN("isend: direct store failed (%s): message goes through the staged path", fl_vmm_last_error());
  if (mh && mh->type == NCCL_PTR_CUDA && size > 0) {
    // device memory cannot be handed to send(2): bounce it through host memory
    r->stage.resize((size_t)size);
    if (fl_vmm_memcpy(r->stage.data(), data, (size_t)size) != 0) {
      FL_WARN("isend: device -> host staging copy failed: %s", fl_vmm_last_error());
      r->used = false;
      return ncclUnhandledCudaError;
    }
    r->data = r->stage.data();
  }
  // path: the device the receiver proposed, if usable; extra stripes on following devices
  const Params& p = params();
  const int first = cm->bid_tx(c->channel_id, c->own_dev, d.proposed_dev) % c->ndev;
  int nstripes = (int)p.degree;
  if (nstripes > c->ndev) nstripes = c->ndev;
  while (nstripes > 1 && (uint64_t)size / (uint64_t)nstripes < (uint64_t)p.min_stripe_bytes) --nstripes;
  const uint64_t mask = cm->tx_mask(c->own_dev);
  const uint64_t per = nstripes > 1 ? ((uint64_t)size / (uint64_t)nstripes) & ~127ull : (uint64_t)size;  // 128-B multiples (src/plugin.cc:1467-1472)
  uint64_t off = 0;
  int dev = first;
  uint64_t used = 0;
  for (int s = 0; s < nstripes; ++s) {
    if (s > 0) {
      // further stripes go to a device the monitor showed idle when the connection first needed it; it is kept (its
      // lease is renewed by the traffic itself) so that concurrent jobs settle on disjoint devices
      int& held = c->extra_dev[s];
      if (held >= 0 && (c->data[held].fd < 0 || ((used >> held) & 1ull))) {
        cm->release_tx(held);
        held = -1;
      }
      if (held < 0) {
        const int b = cm->borrow_tx(c->own_dev, used, dev);
        if (b >= 0 && c->data[b].fd >= 0) held = b;
        else if (b >= 0) cm->release_tx(b);
      }
      if (held >= 0) dev = held;
    }
    dev = next_alive_dev(c, dev);                     // a device whose socket broke earlier is skipped
    if (dev < 0) {
      r->used = false;
      c->error = ncclRemoteError;
      FL_WARN("isend: every data connection of channel %d is gone", c->channel_id);
      return ncclRemoteError;
    }
    Stripe st;
    st.dev = dev;
    st.hdr.magic = kFrameMagic;
    st.hdr.slot = d.slot;
    st.hdr.total = (uint64_t)size;
    st.hdr.offset = off;
    st.hdr.len = s == nstripes - 1 ? (uint64_t)size - off : per;
    st.hdr.tx_mask = mask;
    off += st.hdr.len;
    r->stripes.push_back(st);
    used |= 1ull << dev;
    dev = (dev + (int)(p.step > 0 ? p.step : 1)) % c->ndev;
  }
  for (size_t s = 0; s < r->stripes.size(); ++s) {
    c->data[r->stripes[s].dev].txq.emplace_back(r, (int)s);
    cm->mark_tx(r->stripes[s].dev, r->stripes[s].hdr.len);
  }
  c->msg_index++;
  comm_progress(c, cm);
  *out = r;
  return ncclSuccess;
}

ncclResult_t tcp_irecv(Comm* c, ConnManager* cm, void* data, int size, int tag, TcpMem* mem, Request** out) {
  *out = nullptr;
  ScopedTimer tm(&c->timers, T_IRECV, params().timers != 0);
  if (c->error) return (ncclResult_t)c->error;
  if (size < 0) return ncclInvalidArgument;
  Request* r = get_request(c);
  if (!r) return ncclSuccess;                      // everything in flight: NCCL retries
  r->is_send = false;
  r->data = reinterpret_cast<uint8_t*>(data);
  r->size = (uint64_t)size;
  r->tag = tag;
  TcpMem* mh = mem;
  if (mh && mh->type == NCCL_PTR_CUDA && size > 0) {
    r->stage.resize((size_t)size);
    r->user = r->data;                       // bytes land in the bounce buffer and are copied up when complete
    r->data = r->stage.data();
  }
  // choose the device for this message: re-evaluated every kFinishedBatch completions and only when the
  // connection is quiescent, so a path switch never races with data in flight (src/plugin.cc:1700-1716)
  {
    ScopedTimer ts(&c->timers, T_SELECT, params().timers != 0);
    const bool quiescent = c->posted == c->completed;
    if (c->cur_dev < 0 || (c->n_finished >= kFinishedBatch && quiescent)) {
      c->cur_dev = cm->refresh_rx(c->channel_id, c->own_dev, c->cur_dev, c->peer_tx_mask, quiescent);
      c->n_finished = 0;
    }
  }
  RecvDesc d;
  memset(&d, 0, sizeof d);
  d.magic = kDescMagic;
  d.slot = r->slot;
  d.tag = r->tag;
  d.proposed_dev = c->cur_dev;
  d.size = r->size;
  d.seq = c->post_seq++;
  if (mh && mh->mr_id && mh->region && c->nvl_fd >= 0 && size > 0) {
    bool known = false;
    for (uint32_t id : c->exported) if (id == mh->mr_id) known = true;
    if (!known) {
      // first use of this region on this connection: send its descriptors ahead of the receive that names it
      NvlExportMsg msg;
      memset(&msg, 0, sizeof msg);
      msg.magic = kNvlMagic;
      msg.mr_id = mh->mr_id;
      msg.nslabs = fl_vmm_num_slabs(mh->region);
      msg.size = fl_vmm_size(mh->region);
      msg.slab_bytes = fl_vmm_slab_bytes(mh->region);
      int fds[16];
      int nf = 0;
      bool ok = msg.nslabs >= 1 && msg.nslabs <= 16;
      for (int i = 0; ok && i < msg.nslabs; ++i) {
        if (fl_vmm_export_fd(mh->region, i, &fds[nf]) == 0) ++nf;
        else ok = false;
      }
      if (ok && nvl_send_fds(c->nvl_fd, msg, fds, nf) == 0) {
        c->exported.push_back(mh->mr_id);
        known = true;
      } else {
        FL_INFO("direct path: region %u cannot be exported (%s): staged path", mh->mr_id, fl_vmm_last_error());
        mh->mr_id = 0;                               // do not try again for every message
      }
      for (int i = 0; i < nf; ++i) close(fds[i]);
    }
    if (known) {
      d.mr_id = mh->mr_id;
      d.flags |= kDescDirectOk;
      d.mr_off = (uint64_t)(reinterpret_cast<uint8_t*>(data) - reinterpret_cast<uint8_t*>(fl_vmm_ptr(mh->region)));
    }
  }
  {
    ScopedTimer tp(&c->timers, T_POST_DESC, params().timers != 0);
    const uint8_t* p = reinterpret_cast<const uint8_t*>(&d);
    c->ctrl_tx.insert(c->ctrl_tx.end(), p, p + sizeof d);
    cm->touch_rx(c->cur_dev);                 // bytes are accounted on the device their stripes really arrive on
    c->posted++;
    comm_progress(c, cm);
  }
  *out = r;
  return ncclSuccess;
}

ncclResult_t tcp_test(Request* r, ConnManager* cm, int* done, int* sizes) {
  Comm* c = r->comm;
  *done = 0;
  {
    ScopedTimer tm(&c->timers, T_PROGRESS, params().timers != 0);
    comm_progress(c, cm);
  }
  if (r->done) {
    if (r->user && !r->direct && r->total != UINT64_MAX && r->total > 0) {
      if (fl_vmm_memcpy(r->user, r->stage.data(), (size_t)r->total) != 0) {
        FL_WARN("test: host -> device staging copy failed: %s", fl_vmm_last_error());
        return ncclUnhandledCudaError;
      }
    }
    *done = 1;
    if (sizes) *sizes = (int)(r->is_send ? r->size : r->total);
    if (!r->is_send) {
      c->completed++;
      c->n_finished++;
    }
    r->used = false;
    return ncclSuccess;
  }
  if (c->error) return (ncclResult_t)c->error;
  const uint64_t limit_ns = (uint64_t)params().net_timeout_ms * 1000000ull;
  if (limit_ns && now_ns() - r->last_progress_ns > limit_ns) {
    FL_WARN("%s request on channel %d made no progress for %ld ms: giving up", r->is_send ? "send" : "recv", c->channel_id,
            (long)params().net_timeout_ms);
    c->error = ncclRemoteError;
    return ncclRemoteError;
  }
  return ncclSuccess;
}

void tcp_close_listen(ListenComm* lc) {
  if (!lc) return;
  for (auto& ps : lc->pending) close(ps.fd);
  for (auto& p : lc->partials) comm_close(p.comm);
  for (auto& np : lc->nvl_pending) close(np.fd);
  if (lc->uds_fd >= 0) close(lc->uds_fd);
  if (lc->fd >= 0) close(lc->fd);
  delete lc;
}

}  // namespace flnet
