// Non-blocking progress engine of the TCP transport (see tcp_transport.h for the protocol).
#include "tcp_transport.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/tcp.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <mutex>

#include "nic_rate.h"
#include "params.h"
#include "../mem/vmm.h"

namespace flnet {

constexpr uint32_t kDescMagic = 0x464c4453u;   // "FLDS"
constexpr uint32_t kFrameMagic = 0x464c4652u;  // "FLFR"
constexpr uint32_t kFrameDirectMagic = 0x464c4452u;  // "FLDR": no payload follows, the bytes were written into the exported buffer

int set_nonblock_nodelay(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  if (fl < 0 || fcntl(fd, F_SETFL, fl | O_NONBLOCK) < 0) return -1;
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  int buf = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof buf);
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof buf);
  return 0;
}

static void map_v4(const sockaddr_in* v4, sockaddr_in6* out) {
  memset(out, 0, sizeof *out);
  out->sin6_family = AF_INET6;
  out->sin6_addr.s6_addr[10] = 0xff;
  out->sin6_addr.s6_addr[11] = 0xff;
  memcpy(&out->sin6_addr.s6_addr[12], &v4->sin_addr, 4);
}

// Whether `a` (IPv4, mapped) lies in the subnet of the interface address `ifa` / `mask`.
static bool same_subnet_v4(const sockaddr_in* ifa, const sockaddr_in* mask, const in_addr& a) {
  return (ifa->sin_addr.s_addr & mask->sin_addr.s_addr) == (a.s_addr & mask->sin_addr.s_addr);
}

// Interface selection: NCCL_SOCKET_IFNAME is a comma list of prefixes ("^" excludes, "=" exact), as in the
// reference's OOB code (src/extern/socket.cc:86-99,323-357).  Without it the reference's order of preference
// applies: an "ib*" interface, else the interface in the subnet of the address in NCCL_COMM_ID ("ip:port", the
// rendezvous address some launchers export), else anything that is neither docker nor loopback, else docker,
// else loopback.
int pick_listen_addr(sockaddr_in6* out) {
  const Params& p = params();
  std::string spec = p.socket_ifname;
  bool exclude = false, exact = false;
  if (!spec.empty() && spec[0] == '^') { exclude = true; spec = spec.substr(1); }
  if (!spec.empty() && spec[0] == '=') { exact = true; spec = spec.substr(1); }
  std::vector<std::string> names;
  size_t pos = 0;
  while (pos <= spec.size() && !spec.empty()) {
    size_t c = spec.find(',', pos);
    if (c == std::string::npos) c = spec.size();
    if (c > pos) names.push_back(spec.substr(pos, c - pos));
    pos = c + 1;
  }
  auto matches = [&](const char* ifn) {
    for (auto& n : names) {
      if (exact ? n == ifn : strncmp(ifn, n.c_str(), n.size()) == 0) return true;
    }
    return false;
  };
  const bool want6 = p.socket_family == "AF_INET6";
  ifaddrs* ifs = nullptr;
  bool found = false;
  sockaddr_in6 loop;
  bool have_loop = false;
  // the address NCCL_COMM_ID names, if it is an IPv4 "a.b.c.d:port"
  in_addr comm_id_addr;
  bool have_comm_id = false;
  if (names.empty()) {
    const char* cid = getenv("NCCL_COMM_ID");
    if (cid && strlen(cid) > 1) {
      std::string host(cid);
      const size_t colon = host.rfind(':');
      if (colon != std::string::npos && host.find(':') == colon) host = host.substr(0, colon);
      have_comm_id = inet_pton(AF_INET, host.c_str(), &comm_id_addr) == 1;
    }
  }
  int best_rank = 100;   // without NCCL_SOCKET_IFNAME: 0 ib*, 1 subnet of NCCL_COMM_ID, 2 other, 3 docker (loopback apart)
  if (getifaddrs(&ifs) == 0) {
    for (ifaddrs* i = ifs; i && !found; i = i->ifa_next) {
      if (!i->ifa_addr || !(i->ifa_flags & IFF_UP)) continue;
      const int fam = i->ifa_addr->sa_family;
      if (fam != AF_INET && fam != AF_INET6) continue;
      if (want6 != (fam == AF_INET6) && !p.socket_family.empty()) continue;
      sockaddr_in6 a;
      if (fam == AF_INET) map_v4(reinterpret_cast<sockaddr_in*>(i->ifa_addr), &a);
      else { a = *reinterpret_cast<sockaddr_in6*>(i->ifa_addr); if (IN6_IS_ADDR_LINKLOCAL(&a.sin6_addr)) continue; }
      const bool is_loop = i->ifa_flags & IFF_LOOPBACK;
      if (!names.empty()) {
        const bool m = matches(i->ifa_name);
        if (m == exclude) continue;
        *out = a; found = true;
      } else if (is_loop) {
        if (!have_loop && fam == AF_INET) { loop = a; have_loop = true; }
      } else if (fam == AF_INET || want6) {
        int rank = 2;
        if (strncmp(i->ifa_name, "ib", 2) == 0) rank = 0;
        else if (have_comm_id && fam == AF_INET && i->ifa_netmask &&
                 same_subnet_v4(reinterpret_cast<sockaddr_in*>(i->ifa_addr), reinterpret_cast<sockaddr_in*>(i->ifa_netmask), comm_id_addr))
          rank = 1;
        else if (strncmp(i->ifa_name, "docker", 6) == 0) rank = 3;
        if (rank < best_rank) { best_rank = rank; *out = a; }
      }
    }
    freeifaddrs(ifs);
  }
  if (best_rank < 100) found = true;
  if (!found) {
    if (have_loop) { *out = loop; return 0; }
    sockaddr_in v4;
    memset(&v4, 0, sizeof v4);
    v4.sin_family = AF_INET;
    v4.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    map_v4(&v4, out);
  }
  return 0;
}

// returns bytes moved, 0 if it would block, -1 on error / peer closed
static ssize_t nb_send(int fd, const void* p, size_t n) {
  ssize_t r = send(fd, p, n, MSG_DONTWAIT | MSG_NOSIGNAL);
  if (r >= 0) return r;
  if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return 0;
  return -1;
}
static ssize_t nb_recv(int fd, void* p, size_t n) {
  ssize_t r = recv(fd, p, n, MSG_DONTWAIT);
  if (r > 0) return r;
  if (r == 0) return -1;  // orderly shutdown by the peer while we still expect bytes
  if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return 0;
  return -1;
}

static void fail(Comm* c, ncclResult_t why, const char* what) {
  if (!c->error) {
    c->error = why;
    FL_WARN("%s comm (channel %d, dev %d): %s (errno %d: %s)", c->is_send ? "send" : "recv", c->channel_id, c->own_dev, what,
            errno, strerror(errno));
  }
}

static std::atomic<uint64_t> g_failovers{0};

uint64_t failover_count() { return g_failovers.load(); }

int next_alive_dev(const Comm* c, int from) {
  for (int i = 0; i < c->ndev; ++i) {
    const int d = (from + i) % c->ndev;
    if (c->data[d].fd >= 0) return d;
  }
  return -1;
}

// Recovery from a broken data socket (sender side): the device is marked dead for the selector, and every stripe
// queued on it -- the one in flight from its first byte, since the receiver discards a partial stripe -- moves to the
// next device that is still connected.  What the kernel had already accepted for the broken socket is not known to be
// delivered; a stripe that was counted as sent and then lost shows up as the receiver's request timing out.
static bool failover_tx(Comm* c, ConnManager* cm, int d, const char* why) {
  DataSock& s = c->data[d];
  if (s.fd >= 0) {
    shutdown(s.fd, SHUT_RDWR);
    close(s.fd);
    s.fd = -1;
  }
  cm->set_dead(d, true);
  const int to = params().failover ? next_alive_dev(c, d + 1) : -1;
  if (to < 0) return false;
  size_t moved = 0;
  while (!s.txq.empty()) {
    Request* rq = s.txq.front().first;
    const int si = s.txq.front().second;
    Stripe& st = rq->stripes[si];
    rq->moved -= st.sent;
    st.sent = 0;
    st.hdr_sent = 0;
    st.dev = to;
    c->data[to].txq.emplace_back(rq, si);
    s.txq.pop_front();
    ++moved;
  }
  g_failovers.fetch_add(moved, std::memory_order_relaxed);
  FL_WARN("send comm (channel %d): device %d lost (%s); %zu stripe(s) continue on device %d", c->channel_id, d, why, moved, to);
  return true;
}

// ---- sender ----------------------------------------------------------------------------------------
static void sender_read_descs(Comm* c) {
  for (;;) {
    ssize_t r = nb_recv(c->ctrl_fd, c->ctrl_rx + c->ctrl_rx_got, sizeof(RecvDesc) - c->ctrl_rx_got);
    if (r < 0) {
      // the receiver may close its side once everything it posted has completed; only an error if we still owe data
      bool owing = false;
      for (auto& rq : c->reqs) if (rq.used && !rq.done) owing = true;
      if (owing) fail(c, ncclRemoteError, "control connection lost");
      return;
    }
    if (r == 0) return;
    c->ctrl_rx_got += (size_t)r;
    if (c->ctrl_rx_got == sizeof(RecvDesc)) {
      RecvDesc d;
      memcpy(&d, c->ctrl_rx, sizeof d);
      c->ctrl_rx_got = 0;
      if (d.magic != kDescMagic) { fail(c, ncclInternalError, "bad descriptor magic"); return; }
      c->fifo.push_back(d);
    }
  }
}

static void sender_push(Comm* c, ConnManager* cm) {
  const int64_t fault_after = params().fault_drop_after;
  for (int d = 0; d < c->ndev; ++d) {
    DataSock& s = c->data[d];
    if (s.fd < 0) continue;
    while (!s.txq.empty()) {
      Request* rq = s.txq.front().first;
      Stripe& st = rq->stripes[s.txq.front().second];
      if (st.hdr_sent < sizeof(FrameHdr)) {
        ssize_t r = nb_send(s.fd, reinterpret_cast<uint8_t*>(&st.hdr) + st.hdr_sent, sizeof(FrameHdr) - st.hdr_sent);
        if (r < 0) {
          if (!failover_tx(c, cm, d, "send failed")) { fail(c, ncclRemoteError, "data connection lost while sending"); return; }
          break;
        }
        if (r == 0) break;
        st.hdr_sent += (size_t)r;
        if (st.hdr_sent < sizeof(FrameHdr)) break;
      }
      if (st.sent < st.hdr.len) {
        size_t want = st.hdr.len - st.sent;
        if (fault_after > 0 && !c->fault_fired && s.tx_bytes + want > (uint64_t)fault_after) {
          // test hook: the link "breaks" in the middle of a stripe
          size_t allowed = (uint64_t)fault_after > s.tx_bytes ? (size_t)(fault_after - s.tx_bytes) : 0;
          if (allowed) nb_send(s.fd, rq->data + st.hdr.offset + st.sent, allowed);
          c->fault_fired = true;
          if (!failover_tx(c, cm, d, "injected link failure")) { fail(c, ncclSystemError, "injected link failure"); return; }
          break;
        }
        want = nic_allowance(d, want);
        if (want == 0) break;                                  // this NIC is at its line rate: come back later
        ssize_t r = nb_send(s.fd, rq->data + st.hdr.offset + st.sent, want);
        if (r < 0) {
          if (!failover_tx(c, cm, d, "send failed")) { fail(c, ncclRemoteError, "data connection lost while sending"); return; }
          break;
        }
        if (r == 0) break;
        st.sent += (size_t)r;
        s.tx_bytes += (uint64_t)r;
        rq->moved += (uint64_t)r;
        rq->last_progress_ns = now_ns();
        cm->done_tx(d, (uint64_t)r);
        if (st.sent < st.hdr.len) break;
      }
      rq->stripes_done++;
      if (rq->stripes_done == rq->stripes.size()) rq->done = true;
      s.txq.pop_front();
    }
  }
}

// ---- receiver --------------------------------------------------------------------------------------
static void receiver_flush_ctrl(Comm* c) {
  while (!c->ctrl_tx.empty()) {
    ssize_t r = nb_send(c->ctrl_fd, c->ctrl_tx.data(), c->ctrl_tx.size());
    if (r < 0) { fail(c, ncclRemoteError, "control connection lost"); return; }
    if (r == 0) return;
    c->ctrl_tx.erase(c->ctrl_tx.begin(), c->ctrl_tx.begin() + r);
  }
}

// A stripe counts when its last byte is in, and once: after a failover the sender may repeat one that had arrived.
static void stripe_arrived(Request& rq, uint64_t offset, uint64_t len) {
  if (std::find(rq.got_offsets.begin(), rq.got_offsets.end(), offset) == rq.got_offsets.end()) {
    rq.got_offsets.push_back(offset);
    rq.moved += len;
  }
  if (rq.moved == rq.total) rq.done = true;
}

// Receiver side of the recovery: the broken socket is closed, its half-received stripe forgotten, and the connection
// lives on as long as another data socket does.
static bool failover_rx(Comm* c, ConnManager* cm, int d) {
  DataSock& s = c->data[d];
  close(s.fd);
  s.fd = -1;
  if (s.rx_in_payload) cm->done_rx(d, s.rx_hdr.len - s.rx_payload_got);   // what will never arrive here any more
  s.rx_in_payload = false;
  s.rx_hdr_got = 0;
  s.rx_payload_got = 0;
  cm->set_dead(d, true);
  if (!params().failover || next_alive_dev(c, d + 1) < 0) return false;
  FL_WARN("recv comm (channel %d): device %d lost; waiting for its stripes on the other devices", c->channel_id, d);
  return true;
}

static void receiver_pull(Comm* c, ConnManager* cm) {
  for (int d = 0; d < c->ndev; ++d) {
    DataSock& s = c->data[d];
    if (s.fd < 0) continue;
    for (;;) {
      if (!s.rx_in_payload) {
        ssize_t r = nb_recv(s.fd, reinterpret_cast<uint8_t*>(&s.rx_hdr) + s.rx_hdr_got, sizeof(FrameHdr) - s.rx_hdr_got);
        if (r < 0) {
          bool waiting = false;
          for (auto& rq : c->reqs) if (rq.used && !rq.done) waiting = true;
          if (!waiting) return;                       // the sender is done with this connection
          if (failover_rx(c, cm, d)) break;
          cm->set_dead(d, true);
          fail(c, ncclRemoteError, "data connection closed by the sender");
          return;
        }
        if (r == 0) break;
        s.rx_hdr_got += (size_t)r;
        if (s.rx_hdr_got < sizeof(FrameHdr)) break;
        s.rx_hdr_got = 0;
        if ((s.rx_hdr.magic != kFrameMagic && s.rx_hdr.magic != kFrameDirectMagic) || s.rx_hdr.slot >= (uint32_t)kMaxRequests) {
          fail(c, ncclInternalError, "bad frame header");
          return;
        }
        Request& rq = c->reqs[s.rx_hdr.slot];
        if (!rq.used || rq.is_send) { fail(c, ncclInternalError, "frame for a slot that is not posted"); return; }
        if (s.rx_hdr.total > rq.size || s.rx_hdr.offset + s.rx_hdr.len > s.rx_hdr.total) {
          fail(c, ncclInvalidUsage, "message larger than the posted receive");   // src/plugin.cc:1555-1570
          return;
        }
        rq.total = s.rx_hdr.total;
        c->peer_tx_mask = s.rx_hdr.tx_mask;
        if (s.rx_hdr.magic == kFrameDirectMagic) {      // the sender already stored the payload through its mapping
          rq.direct = true;
          rq.moved = rq.total;
          rq.done = true;
          rq.last_progress_ns = now_ns();
          cm->touch_rx(d);
          continue;
        }
        s.rx_in_payload = true;
        s.rx_payload_got = 0;
        cm->mark_rx(d, s.rx_hdr.len);                 // this stripe is now in flight on device d
        if (s.rx_hdr.len == 0) {
          s.rx_in_payload = false;
          stripe_arrived(rq, s.rx_hdr.offset, 0);
        }
      }
      if (s.rx_in_payload) {
        Request& rq = c->reqs[s.rx_hdr.slot];
        ssize_t r = nb_recv(s.fd, rq.data + s.rx_hdr.offset + s.rx_payload_got, s.rx_hdr.len - s.rx_payload_got);
        if (r < 0) {
          if (failover_rx(c, cm, d)) break;           // the partial stripe is dropped; the sender sends it again elsewhere
          cm->set_dead(d, true);
          fail(c, ncclRemoteError, "data connection closed in the middle of a message");
          return;
        }
        if (r == 0) break;
        s.rx_payload_got += (uint64_t)r;
        rq.last_progress_ns = now_ns();
        cm->done_rx(d, (uint64_t)r);
        if (s.rx_payload_got == s.rx_hdr.len) {
          s.rx_in_payload = false;
          stripe_arrived(rq, s.rx_hdr.offset, s.rx_hdr.len);
        }
      }
    }
  }
}

ncclResult_t comm_progress(Comm* c, ConnManager* cm) {
  if (c->error) return (ncclResult_t)c->error;
  if (c->is_send) {
    sender_read_descs(c);
    if (!c->error) sender_push(c, cm);
  } else {
    receiver_flush_ctrl(c);
    if (!c->error) receiver_pull(c, cm);
  }
  return (ncclResult_t)c->error;
}

void comm_close(Comm* c) {
  if (!c) return;
  if (params().timers) c->timers.print(c->is_send ? "send" : "recv");
  if (c->ctrl_fd >= 0) close(c->ctrl_fd);
  for (int d = 0; d < kMaxDev; ++d)
    if (c->data[d].fd >= 0) close(c->data[d].fd);
  for (int fd : c->pending_fds)
    if (fd >= 0) close(fd);
  if (c->nvl_fd >= 0) close(c->nvl_fd);
  for (auto& m : c->peer_mrs)
    if (m.region) fl_vmm_destroy(reinterpret_cast<FlVmmRegion*>(m.region));
  delete c;
}

}  // namespace flnet
