// Software NIC: reliable-connected queue pairs between processes of one machine, over Unix stream sockets.
//
// Every process owns one listener in the abstract namespace ("fuselink-softnic-<pid>").  Connecting a queue
// pair opens a stream to the peer's listener; work requests travel on it as {header, payload} records, the
// responder checks the remote key and the bounds, stores the payload at the requested address, consumes a
// posted receive for a write-with-immediate, and answers every request with an ACK (or a NAK that moves the
// requester's queue pair to the error state, as a remote access error does on hardware).  A completion is
// reported when the ACK arrives, so "signalled completion" keeps its meaning: the bytes are in place.
//
// Bytes only move inside progress(), which the transport calls from its own entry points; there is no
// thread.  The whole NIC sits behind one mutex (the transport may be entered from several proxy threads).
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <vector>

#include "logging.h"
#include "nic_rate.h"
#include "params.h"
#include "rdma_provider.h"

namespace flnet {
namespace rdma {

namespace {

// the opaque handles of the interface are these objects
struct SoftPd { int dev; };
struct SoftCq { int dev; std::deque<Completion> done; };
inline SoftCq* impl(Cq* c) { return reinterpret_cast<SoftCq*>(c); }

constexpr uint32_t kWireMagic = 0x534e4943u;   // "SNIC"
constexpr uint32_t kAck = 1, kNak = 2;

struct WireHdr {
  uint32_t magic;
  uint32_t op;
  uint32_t len;
  uint32_t rkey;
  uint64_t raddr;
  uint32_t imm;
  uint32_t pad;
};
struct WireHello {
  uint32_t magic;
  uint32_t target_qpn;
  uint32_t source_qpn;
  uint32_t pad;
};
struct WireAck {
  uint32_t magic;
  uint32_t kind;     // kAck / kNak
};

struct OutMsg {
  WireHdr hdr;
  const uint8_t* payload;
  std::vector<uint8_t> copy;       // inline data
  size_t hdr_sent = 0, sent = 0;
};
struct Inflight {
  uint64_t wr_id;
  bool signaled;
  uint32_t len;
  uint8_t* read_dst;               // RDMA read: where the returned bytes go (null for writes)
};

struct SoftMr {
  uint8_t* addr;                   // what work requests and the peer call this memory (the I/O virtual address)
  size_t len;
  int access;
  uint8_t* local = nullptr;        // where the bytes are in this process; differs from addr for a dma-buf registration
  void* map = nullptr;             // dma-buf: this NIC's own mapping of the buffer
  size_t map_len = 0;
  uint8_t* at(const uint8_t* a) const { return local + (a - addr); }
};

struct Inbound {                    // one accepted stream, attached to the queue pair its hello names
  int fd = -1;
  WireHello hello;
  size_t hello_got = 0;
  struct QpImpl* qp = nullptr;
  WireHdr hdr;
  size_t hdr_got = 0;
  bool in_payload = false, bad = false, wait_recv = false;
  uint32_t payload_got = 0;
  uint8_t* dst = nullptr;
  std::vector<uint8_t> ack_tx;      // ACK bytes the socket has not taken yet
};

struct QpImpl {
  uint32_t qpn = 0;
  int dev = 0;
  SoftCq* cq = nullptr;
  int out_fd = -1;
  bool error = false;
  std::deque<OutMsg> sendq;
  std::deque<Inflight> inflight;    // handed to the socket (at least partly), not yet acknowledged
  std::deque<uint64_t> rq;          // posted zero-length receives
  WireAck ack_rx;
  size_t ack_got = 0;
  uint32_t read_left = 0;           // bytes of a read response still to arrive behind its ACK
  uint32_t read_got = 0;
  QpCaps caps;
};

int set_nonblock(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  return fl < 0 ? -1 : fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}

void nic_addr(uint64_t pid, sockaddr_un* sa, socklen_t* len) {
  memset(sa, 0, sizeof *sa);
  sa->sun_family = AF_UNIX;
  const int n = snprintf(sa->sun_path + 1, sizeof sa->sun_path - 1, "fuselink-softnic-%llu", (unsigned long long)pid);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

class SoftProvider : public Provider {
 public:
  SoftProvider() {
    ndev_ = (int)param_i64("FUSELINK_SOFT_NDEV", 4);
    fault_dev_ = (int)param_i64("FUSELINK_SOFT_FAULT_DEV", -1);               // test hook: this device breaks ...
    fault_after_ = (uint64_t)param_i64("FUSELINK_SOFT_FAULT_AFTER_BYTES", 0);  // ... once it has carried this many bytes
    if (ndev_ < 1) ndev_ = 1;
    if (ndev_ > 16) ndev_ = 16;
    listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    sockaddr_un sa;
    socklen_t sl;
    nic_addr((uint64_t)getpid(), &sa, &sl);
    if (listen_fd_ < 0 || bind(listen_fd_, reinterpret_cast<sockaddr*>(&sa), sl) != 0 || listen(listen_fd_, 1024) != 0) {
      FL_WARN("software NIC: cannot listen (%s)", strerror(errno));
      if (listen_fd_ >= 0) close(listen_fd_);
      listen_fd_ = -1;
      ndev_ = 0;
    } else {
      set_nonblock(listen_fd_);
    }
  }
  const char* name() const override { return "soft"; }
  int device_count() override { return ndev_; }
  DeviceInfo device(int dev) override {
    DeviceInfo d;
    char buf[64];
    snprintf(buf, sizeof buf, "softnic_%d", dev);
    d.name = buf;
    snprintf(buf, sizeof buf, "/sys/devices/virtual/infiniband/softnic_%d", dev);
    d.pci_path = buf;
    d.guid = 0x534e494300000000ull + (uint64_t)dev;
    d.speed_mbps = 100000;
    d.max_qp = 65536;
    d.link = kLinkEthernet;
    d.relaxed_ordering = true;
    return d;
  }

  Pd* alloc_pd(int dev) override { return reinterpret_cast<Pd*>(new SoftPd{dev}); }
  void dealloc_pd(Pd* pd) override { delete reinterpret_cast<SoftPd*>(pd); }

  Mr* reg_mr(Pd* pd, void* addr, size_t len, int access) override {
    (void)pd;
    std::lock_guard<std::mutex> l(mu_);
    Mr* m = new Mr();
    m->lkey = m->rkey = next_key_++;
    m->addr = addr;
    m->len = len;
    SoftMr sm{reinterpret_cast<uint8_t*>(addr), len, access};
    sm.local = sm.addr;
    mrs_[m->rkey] = sm;
    return m;
  }
  // A dma-buf is reached through a mapping of its own, never through the address the application uses: the way a NIC
  // gets to device memory through the exporter's pages.  Anything mmap can map stands in for the dma-buf (the memfd
  // slabs of the fake cuMem driver in the tests).
  Mr* reg_dmabuf_mr(Pd* pd, int fd, uint64_t offset, size_t len, uint64_t iova, int access) override {
    (void)pd;
    if (fd < 0 || !len) { errno = EBADF; return nullptr; }
    const uint64_t page = (uint64_t)sysconf(_SC_PAGESIZE);
    const uint64_t lo = offset / page * page;
    const size_t map_len = (size_t)(offset - lo) + len;
    void* map = mmap(nullptr, map_len, PROT_READ | PROT_WRITE, MAP_SHARED, fd, (off_t)lo);
    if (map == MAP_FAILED) return nullptr;
    std::lock_guard<std::mutex> l(mu_);
    Mr* m = new Mr();
    m->lkey = m->rkey = next_key_++;
    m->addr = reinterpret_cast<void*>(iova);
    m->len = len;
    SoftMr sm{reinterpret_cast<uint8_t*>(iova), len, access};
    sm.local = static_cast<uint8_t*>(map) + (offset - lo);
    sm.map = map;
    sm.map_len = map_len;
    mrs_[m->rkey] = sm;
    return m;
  }
  bool dmabuf_supported(int) override { return true; }
  bool peer_memory_supported() override { return param_i64("FUSELINK_SOFT_PEERMEM", 1) != 0; }
  void dereg_mr(Mr* mr) override {
    if (!mr) return;
    std::lock_guard<std::mutex> l(mu_);
    auto it = mrs_.find(mr->rkey);
    if (it != mrs_.end()) {
      if (it->second.map) munmap(it->second.map, it->second.map_len);
      mrs_.erase(it);
    }
    delete mr;
  }

  Cq* create_cq(int dev, int depth) override {
    (void)depth;
    SoftCq* c = new SoftCq();
    c->dev = dev;
    return reinterpret_cast<Cq*>(c);
  }
  void destroy_cq(Cq* cq) override { delete impl(cq); }

  Qp* create_qp(Pd* pd, Cq* cq, const QpCaps& caps) override {
    std::lock_guard<std::mutex> l(mu_);
    QpImpl* q = new QpImpl();
    q->qpn = next_qpn_++;
    q->dev = reinterpret_cast<SoftPd*>(pd)->dev;
    q->cq = impl(cq);
    q->caps = caps;
    qps_[q->qpn] = q;
    return reinterpret_cast<Qp*>(q);
  }
  void destroy_qp(Qp* qp) override {
    if (!qp) return;
    std::lock_guard<std::mutex> l(mu_);
    QpImpl* q = reinterpret_cast<QpImpl*>(qp);
    if (q->out_fd >= 0) close(q->out_fd);
    for (auto& in : inbound_) {
      if (in.qp == q) {
        close(in.fd);
        in.fd = -1;
        in.qp = nullptr;
      }
    }
    qps_.erase(q->qpn);
    delete q;
  }

  int query_qp_info(Qp* qp, int gid_index, QpInfo* out) override {
    (void)gid_index;
    QpImpl* q = reinterpret_cast<QpImpl*>(qp);
    memset(out, 0, sizeof *out);
    out->qpn = q->qpn;
    out->link = kLinkEthernet;
    out->port = 1;
    out->mtu = 5;
    out->gid[15] = (uint8_t)q->dev;
    out->cookie = (uint64_t)getpid();
    return 0;
  }

  int connect_qp(Qp* qp, const QpInfo& remote, const QpConnectParams& p) override {
    (void)p;
    QpImpl* q = reinterpret_cast<QpImpl*>(qp);
    int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    sockaddr_un sa;
    socklen_t sl;
    nic_addr(remote.cookie, &sa, &sl);
    if (connect(fd, reinterpret_cast<sockaddr*>(&sa), sl) != 0) {
      FL_WARN("software NIC: peer process %llu is not reachable (%s)", (unsigned long long)remote.cookie, strerror(errno));
      close(fd);
      return -1;
    }
    WireHello h{kWireMagic, remote.qpn, q->qpn, 0};
    if (send(fd, &h, sizeof h, MSG_NOSIGNAL) != (ssize_t)sizeof h) {
      close(fd);
      return -1;
    }
    set_nonblock(fd);
    int buf = 4 << 20;
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof buf);
    std::lock_guard<std::mutex> l(mu_);
    q->out_fd = fd;
    return 0;
  }

  int post_send(Qp* qp, const SendWr* wrs, int n) override {
    std::lock_guard<std::mutex> l(mu_);
    QpImpl* q = reinterpret_cast<QpImpl*>(qp);
    if (q->out_fd < 0) return -1;
    if ((int)(q->sendq.size() + q->inflight.size()) + n > q->caps.max_send_wr) return -ENOMEM;   // send queue full
    for (int i = 0; i < n; ++i) {
      const SendWr& w = wrs[i];
      if (w.inline_data && (int)w.len > q->caps.max_inline) return -EINVAL;
      OutMsg m;
      m.hdr = WireHdr{kWireMagic, (uint32_t)w.op, w.len, w.rkey, w.raddr, w.imm, 0};
      m.payload = reinterpret_cast<const uint8_t*>(w.laddr);
      if (w.len && w.laddr) {                      // a dma-buf registration is read and written through its own mapping
        auto lm = mrs_.find(w.lkey);
        if (lm != mrs_.end() && lm->second.map) {
          if (m.payload < lm->second.addr || m.payload + w.len > lm->second.addr + lm->second.len) return -EINVAL;
          m.payload = lm->second.at(m.payload);
        }
      }
      uint8_t* read_dst = nullptr;
      if (w.op == kRead) {                         // the request carries no payload; the response does
        read_dst = const_cast<uint8_t*>(m.payload);
        m.payload = nullptr;
        m.hdr.pad = w.len;                         // bytes wanted
        m.hdr.len = 0;
      } else if (w.inline_data && w.len) {
        m.copy.assign(m.payload, m.payload + w.len);
        m.payload = nullptr;
      }
      q->sendq.push_back(std::move(m));
      q->inflight.push_back(Inflight{w.wr_id, w.signaled, w.len, read_dst});
    }
    progress_locked();
    return 0;
  }

  int post_recv(Qp* qp, uint64_t wr_id) override {
    std::lock_guard<std::mutex> l(mu_);
    QpImpl* q = reinterpret_cast<QpImpl*>(qp);
    if ((int)q->rq.size() >= q->caps.max_recv_wr) return -ENOMEM;
    q->rq.push_back(wr_id);
    return 0;
  }

  int poll_cq(Cq* cq_h, int max, Completion* out) override {
    std::lock_guard<std::mutex> l(mu_);
    progress_locked();
    SoftCq* cq = impl(cq_h);
    int n = 0;
    while (n < max && !cq->done.empty()) {
      out[n++] = cq->done.front();
      cq->done.pop_front();
    }
    return n;
  }

  void progress() override {
    std::lock_guard<std::mutex> l(mu_);
    progress_locked();
  }

  int wait_async_event(int dev, int timeout_ms, std::string* what) override {
    std::unique_lock<std::mutex> l(ev_mu_);
    if (!ev_cv_.wait_for(l, std::chrono::milliseconds(timeout_ms), [&] { return !events_[dev].empty() || closing_; })) return 0;
    if (closing_ || events_[dev].empty()) return -1;
    *what = events_[dev].front();
    events_[dev].pop_front();
    return 1;
  }
  void inject_event(int dev, const char* what) {
    std::lock_guard<std::mutex> l(ev_mu_);
    events_[dev].push_back(what);
    ev_cv_.notify_all();
  }

 private:
  void fail_qp(QpImpl* q, int status) {
    // the request at the head failed with `status`, everything behind it is flushed (verbs error state)
    bool first = true;
    for (auto& f : q->inflight) {
      Completion c;
      c.wr_id = f.wr_id;
      c.status = first ? status : kWcFlushed;
      c.qpn = q->qpn;
      if (first || f.signaled) q->cq->done.push_back(c);
      first = false;
    }
    q->inflight.clear();
    q->sendq.clear();
    q->error = true;
  }

  void requester_progress(QpImpl* q) {
    if (q->out_fd < 0 || q->error) return;
    while (!q->sendq.empty()) {
      OutMsg& m = q->sendq.front();
      if (m.hdr_sent < sizeof m.hdr) {
        ssize_t r = send(q->out_fd, reinterpret_cast<uint8_t*>(&m.hdr) + m.hdr_sent, sizeof m.hdr - m.hdr_sent, MSG_DONTWAIT | MSG_NOSIGNAL);
        if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) break;
        if (r <= 0) { fail_qp(q, kWcRetryExceeded); return; }
        m.hdr_sent += (size_t)r;
        if (m.hdr_sent < sizeof m.hdr) break;
      }
      const uint8_t* p = m.payload ? m.payload : m.copy.data();
      if (q->dev == fault_dev_ && !fault_fired_ && fault_after_ && dev_bytes_ + m.hdr.len - m.sent > fault_after_) {
        // the link of this device goes down in the middle of a message: what a cable pull does to a queue pair
        const size_t allowed = fault_after_ > dev_bytes_ ? (size_t)(fault_after_ - dev_bytes_) : 0;
        if (allowed && m.sent < m.hdr.len) (void)!send(q->out_fd, p + m.sent, allowed < m.hdr.len - m.sent ? allowed : m.hdr.len - m.sent, MSG_DONTWAIT | MSG_NOSIGNAL);
        fault_fired_ = true;
        close(q->out_fd);
        q->out_fd = -1;
        fail_qp(q, kWcRetryExceeded);
        return;
      }
      if (m.sent < m.hdr.len) {
        const size_t may = nic_allowance(q->dev, m.hdr.len - m.sent);   // emulated line rate of this device, if one is set
        if (may == 0) break;
        ssize_t r = send(q->out_fd, p + m.sent, may, MSG_DONTWAIT | MSG_NOSIGNAL);
        if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) break;
        if (r <= 0) { fail_qp(q, kWcRetryExceeded); return; }
        m.sent += (size_t)r;
        if (q->dev == fault_dev_) dev_bytes_ += (uint64_t)r;
        if (m.sent < m.hdr.len) break;
      }
      q->sendq.pop_front();
    }
    for (;;) {          // acknowledgements (a read's ACK is followed by the bytes it asked for)
      if (q->read_left) {
        const size_t want = q->read_left < sizeof bounce_ ? q->read_left : sizeof bounce_;
        ssize_t r = recv(q->out_fd, bounce_, want, MSG_DONTWAIT);
        if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) break;
        if (r <= 0) { fail_qp(q, kWcRetryExceeded); return; }
        Inflight& f = q->inflight.front();
        dma_place(f.read_dst + q->read_got, bounce_, (size_t)r);
        q->read_got += (uint32_t)r;
        q->read_left -= (uint32_t)r;
        if (q->read_left) continue;
        complete_head(q);
        continue;
      }
      ssize_t r = recv(q->out_fd, reinterpret_cast<uint8_t*>(&q->ack_rx) + q->ack_got, sizeof(WireAck) - q->ack_got, MSG_DONTWAIT);
      if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) break;
      if (r <= 0) {
        if (!q->inflight.empty()) fail_qp(q, kWcRetryExceeded);     // the peer went away with work outstanding
        else { close(q->out_fd); q->out_fd = -1; }
        return;
      }
      q->ack_got += (size_t)r;
      if (q->ack_got < sizeof(WireAck)) continue;
      q->ack_got = 0;
      if (q->ack_rx.magic != kWireMagic || q->inflight.empty()) { fail_qp(q, kWcGeneral); return; }
      if (q->ack_rx.kind == kNak) { fail_qp(q, kWcRemoteAccess); return; }
      if (q->inflight.front().read_dst && q->inflight.front().len) {
        q->read_left = q->inflight.front().len;
        q->read_got = 0;
        continue;
      }
      complete_head(q);
    }
  }
  void complete_head(QpImpl* q) {
    Inflight f = q->inflight.front();
    q->inflight.pop_front();
    if (f.signaled) {
      Completion c;
      c.wr_id = f.wr_id;
      c.byte_len = f.len;
      c.qpn = q->qpn;
      q->cq->done.push_back(c);
    }
  }

  void queue_ack(Inbound& in, uint32_t kind) {
    WireAck a{kWireMagic, kind};
    const uint8_t* p = reinterpret_cast<const uint8_t*>(&a);
    in.ack_tx.insert(in.ack_tx.end(), p, p + sizeof a);
  }
  bool flush_acks(Inbound& in) {
    while (!in.ack_tx.empty()) {
      ssize_t r = send(in.fd, in.ack_tx.data(), in.ack_tx.size(), MSG_DONTWAIT | MSG_NOSIGNAL);
      if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return true;
      if (r <= 0) return false;
      in.ack_tx.erase(in.ack_tx.begin(), in.ack_tx.begin() + r);
    }
    return true;
  }

  // returns false when the stream is finished (closed or broken)
  bool responder_progress(Inbound& in) {
    if (in.hello_got < sizeof in.hello) {
      ssize_t r = recv(in.fd, reinterpret_cast<uint8_t*>(&in.hello) + in.hello_got, sizeof in.hello - in.hello_got, MSG_DONTWAIT);
      if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return true;
      if (r <= 0) return false;
      in.hello_got += (size_t)r;
      if (in.hello_got < sizeof in.hello) return true;
      auto it = qps_.find(in.hello.target_qpn);
      if (in.hello.magic != kWireMagic || it == qps_.end()) return false;
      in.qp = it->second;
    }
    if (!flush_acks(in)) return false;
    for (;;) {
      if (in.wait_recv) {                       // a write-with-immediate is complete but no receive was posted (RNR): retry
        if (in.qp->rq.empty()) return true;
        finish_imm(in);
      }
      if (!in.in_payload) {
        ssize_t r = recv(in.fd, reinterpret_cast<uint8_t*>(&in.hdr) + in.hdr_got, sizeof in.hdr - in.hdr_got, MSG_DONTWAIT);
        if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return flush_acks(in);
        if (r <= 0) return false;
        in.hdr_got += (size_t)r;
        if (in.hdr_got < sizeof in.hdr) return true;
        in.hdr_got = 0;
        if (in.hdr.magic != kWireMagic) return false;
        in.bad = false;
        in.dst = nullptr;
        if (in.hdr.op == (uint32_t)kRead) {        // answer: ACK + the bytes, or NAK
          const uint32_t want = in.hdr.pad;
          auto it = mrs_.find(in.hdr.rkey);
          const uint8_t* a = reinterpret_cast<const uint8_t*>(in.hdr.raddr);
          if (it == mrs_.end() || !(it->second.access & kAccessRemoteRead) || a < it->second.addr || a + want > it->second.addr + it->second.len) {
            queue_ack(in, kNak);
          } else {
            queue_ack(in, kAck);
            const size_t at = in.ack_tx.size();
            in.ack_tx.resize(at + want);
            dma_fetch(in.ack_tx.data() + at, it->second.at(a), want);
          }
          flush_acks(in);
          continue;
        }
        if (in.hdr.len) {
          auto it = mrs_.find(in.hdr.rkey);
          uint8_t* a = reinterpret_cast<uint8_t*>(in.hdr.raddr);
          if (it == mrs_.end() || !(it->second.access & kAccessRemoteWrite) || a < it->second.addr ||
              a + in.hdr.len > it->second.addr + it->second.len)
            in.bad = true;                      // wrong key or out of bounds: the payload is drained and refused
          else
            in.dst = it->second.at(a);
        }
        in.in_payload = true;
        in.payload_got = 0;
      }
      while (in.payload_got < in.hdr.len) {
        // through a bounce buffer: the placement into the application's memory is the NIC's DMA (see dma_place)
        const size_t want = in.hdr.len - in.payload_got;
        ssize_t r = recv(in.fd, bounce_, want < sizeof bounce_ ? want : sizeof bounce_, MSG_DONTWAIT);
        if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return flush_acks(in);
        if (r <= 0) return false;
        if (!in.bad) dma_place(in.dst + in.payload_got, bounce_, (size_t)r);
        in.payload_got += (uint32_t)r;
      }
      in.in_payload = false;
      if (in.bad) {
        queue_ack(in, kNak);
        flush_acks(in);
        continue;
      }
      if (in.hdr.op == (uint32_t)kWriteImm) {
        if (in.qp->rq.empty()) { in.wait_recv = true; return true; }
        finish_imm(in);
      } else {
        queue_ack(in, kAck);
      }
    }
  }
  // What a NIC's DMA engine does: bytes land in ascending order and the last word becomes visible after everything
  // before it, so a reader that polls the end of a record (the descriptor FIFO's sequence word) sees a complete
  // record.  The application reads such memory without a lock, exactly as it does with hardware; the copy is kept out
  // of ThreadSanitizer's view for that reason (it is device traffic, not a program store the reader could lock against),
  // and the reader pairs it with an acquire load.
  __attribute__((no_sanitize("thread"))) static void dma_place(uint8_t* dst, const uint8_t* src, size_t n) {
    size_t body = n >= 8 && ((reinterpret_cast<uintptr_t>(dst) + n) & 7) == 0 ? n - 8 : n;
    volatile uint8_t* d = dst;
    for (size_t i = 0; i < body; ++i) d[i] = src[i];
    if (body < n) {
      uint64_t last;
      __builtin_memcpy(&last, src + body, 8);
      __atomic_store_n(reinterpret_cast<uint64_t*>(dst + body), last, __ATOMIC_RELEASE);
    }
  }

  // the NIC reading application memory (the other direction of dma_place)
  __attribute__((no_sanitize("thread"))) static void dma_fetch(uint8_t* dst, const uint8_t* src, size_t n) {
    const volatile uint8_t* s = src;
    for (size_t i = 0; i < n; ++i) dst[i] = s[i];
  }

  void finish_imm(Inbound& in) {
    in.wait_recv = false;
    Completion c;
    c.wr_id = in.qp->rq.front();
    in.qp->rq.pop_front();
    c.is_recv = true;
    c.imm = in.hdr.imm;
    c.byte_len = in.hdr.len;
    c.qpn = in.qp->qpn;
    in.qp->cq->done.push_back(c);
    queue_ack(in, kAck);
  }

  // One poll() over every socket of the NIC tells which queue pairs and inbound streams have work; only those are
  // touched.  (Walking all of them with a recv each costs a system call per socket per call, which dominates once a
  // process holds dozens of queue pairs.)
  void progress_locked() {
    if (listen_fd_ < 0) return;
    pfds_.clear();
    pfds_.push_back(pollfd{listen_fd_, POLLIN, 0});
    pqps_.clear();
    for (auto& kv : qps_) {
      QpImpl* q = kv.second;
      if (q->out_fd < 0 || q->error) continue;
      pfds_.push_back(pollfd{q->out_fd, (short)(POLLIN | (q->sendq.empty() ? 0 : POLLOUT)), 0});
      pqps_.push_back(q);
    }
    const size_t in0 = pfds_.size();
    for (auto& in : inbound_) {
      // a stream parked on "no receive posted" (RNR) has to be looked at again even without new bytes
      const short ev = (short)(POLLIN | (in.ack_tx.empty() ? 0 : POLLOUT));
      pfds_.push_back(pollfd{in.fd, ev, (short)(in.wait_recv && in.qp && !in.qp->rq.empty() ? POLLIN : 0)});
    }
    if (poll(pfds_.data(), pfds_.size(), 0) < 0) return;
    if (pfds_[0].revents) {
      for (;;) {
        int fd = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd < 0) break;
        set_nonblock(fd);
        int buf = 4 << 20;
        setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof buf);
        inbound_.emplace_back();
        inbound_.back().fd = fd;
      }
    }
    for (size_t i = 0; i < pqps_.size(); ++i)
      if (pfds_[1 + i].revents) requester_progress(pqps_[i]);
    bool answered = false;
    size_t k = in0;
    for (auto it = inbound_.begin(); it != inbound_.end();) {
      const bool listed = k < pfds_.size() && pfds_[k].fd == it->fd;
      const bool ready = !listed || pfds_[k].revents || (it->wait_recv && it->qp && !it->qp->rq.empty());
      if (listed) ++k;
      if (it->fd >= 0 && !ready) { ++it; continue; }
      if (it->fd < 0 || !responder_progress(*it)) {
        if (it->fd >= 0) close(it->fd);
        it = inbound_.erase(it);
      } else {
        answered = true;
        ++it;
      }
    }
    // ACKs produced above for requesters in this same process are picked up by the next call's poll()
    (void)answered;
  }

  std::vector<pollfd> pfds_;
  std::vector<QpImpl*> pqps_;
  std::mutex mu_;
  int fault_dev_ = -1;
  uint64_t fault_after_ = 0, dev_bytes_ = 0;
  bool fault_fired_ = false;
  uint8_t bounce_[64 * 1024];
  int ndev_ = 0;
  int listen_fd_ = -1;
  uint32_t next_key_ = 0x1000, next_qpn_ = 0x100;
  std::map<uint32_t, SoftMr> mrs_;
  std::map<uint32_t, QpImpl*> qps_;
  std::deque<Inbound> inbound_;
  std::mutex ev_mu_;
  std::condition_variable ev_cv_;
  std::map<int, std::deque<std::string>> events_;
  bool closing_ = false;
};

SoftProvider* g_soft = nullptr;

}  // namespace

Provider* make_soft_provider() {
  if (!g_soft) g_soft = new SoftProvider();
  return g_soft;
}

}  // namespace rdma
}  // namespace flnet

// Test hook: raise an asynchronous event on a software device (what a port going down does on hardware).
extern "C" __attribute__((visibility("default"))) void fuselink_soft_inject_event(int dev, const char* what) {
  if (flnet::rdma::g_soft) flnet::rdma::g_soft->inject_event(dev, what ? what : "event");
}
