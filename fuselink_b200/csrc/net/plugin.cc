// ncclNet plugin entry points: `libnccl-net-fuselink.so`, loaded by NCCL with NCCL_NET_PLUGIN=fuselink.
//
// Surface kept from the reference (src/plugin.cc:1997-2018): the table is named "FuseLink" and is exported
// as ncclNetPlugin_v7 with a v6 alias; getDeviceMr / irecvConsumed are NULL; multi-receive (n > 1) is
// rejected (src/plugin.cc:1449-1450,1879-1880).  A v8 table (size_t registration sizes) is exported too so
// that current NCCL releases find a version they probe for.
//
// What differs: devices are the virtual NICs of a transport.  The TCP transport (tcp_transport.*) works on
// any machine and is what the CPU tests drive; the verbs transport (ib_transport.*) is compiled in and
// used only where libibverbs and RDMA devices exist.  Path selection goes through ConnManager and the
// lock-free monitor instead of peeking into NCCL's private proxy structures (src/fuselink.h:18-37): the
// plugin counts its own posted / completed requests to know when a connection is quiescent.
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
#include <map>
#include <mutex>
#include <random>

#include "conn_manager.h"
#include "ib_transport.h"
#include "logging.h"
#include "nccl_net_abi.h"
#include "params.h"
#include "rdma_transport.h"
#include "tcp_transport.h"
#include "../mem/vmm.h"

using namespace flnet;

namespace {

constexpr uint64_t kHelloMagic = 0x464c4e4b48454c4full;  // "FLNKHELO"
constexpr uint32_t kDescMagic = 0x464c4453u;
constexpr uint32_t kFrameMagic = 0x464c4652u;
constexpr uint32_t kFrameDirectMagic = 0x464c4452u;

std::mutex g_mu;
ConnManager* g_cm = nullptr;
int g_ndev = 0;
int g_ngpus = 0;          // devices the cuMem layer sees; 0 = CUDA registrations unavailable
bool g_rdma = false;      // the RDMA transport carries the data (FUSELINK_TRANSPORT=rdma, or auto with verbs devices present)
std::atomic<int> g_channel_counter{0};
char g_names[kMaxDev][32];
char g_pci[kMaxDev][256];
int g_speed[kMaxDev];
uint64_t g_guid[kMaxDev];
int g_max_comms[kMaxDev];

struct MemHandle {
  void* data;
  size_t size;
  int type;
  FlVmmRegion* region;   // CUDA registrations made through the cuMem layer, else null
  uint32_t mr_id;        // non-zero for a region that can be exported to a same-host sender
  RdmaMrSet* rdma;       // RDMA transport: the registration on every device
  void* base;            // start of the cuMem allocation `data` lies in (key of the adoption table), else null
};
std::atomic<uint32_t> g_mr_counter{1};
struct Adopted { FlVmmRegion* region; uint32_t mr_id; int refs; };
std::map<void*, Adopted> g_adopted;          // cuMem allocations taken over by regMr, by base address (under g_mu)
std::atomic<uint64_t> g_direct_bytes{0};     // payload bytes that went through the direct path (sender side)
std::atomic<uint64_t> g_direct_msgs{0};

// ---- same-host side channel ---------------------------------------------------------------------------
// A receive buffer that lives in a cuMem allocation can be written by a sender on the same machine without
// touching host memory: the receiver hands the allocation's file descriptors over a Unix socket
// (SCM_RIGHTS), the sender maps them, stores the payload through that mapping and sends a frame header with
// no payload.  The reference gets the same effect inside one process by copying from the relay GPU's alias
// address (src/fuselink.cc:25-41); across processes the descriptor has to travel, which is what this does.
// The socket lives in the abstract namespace under a random token published in the listen handle, so a
// sender on another host (or in another network namespace) simply fails to connect and stays on TCP.
void nvl_sockaddr(uint64_t token, sockaddr_un* sa, socklen_t* len) {
  memset(sa, 0, sizeof *sa);
  sa->sun_family = AF_UNIX;
  const int n = snprintf(sa->sun_path + 1, sizeof sa->sun_path - 1, "fuselink-nvl-%016llx", (unsigned long long)token);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int nvl_send_fds(int sock, const NvlExportMsg& msg, const int* fds, int nfds) {
  char cbuf[CMSG_SPACE(sizeof(int) * 16)];
  if (nfds > 16) return -1;
  memset(cbuf, 0, sizeof cbuf);
  iovec iov{const_cast<NvlExportMsg*>(&msg), sizeof msg};
  msghdr mh;
  memset(&mh, 0, sizeof mh);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  if (nfds > 0) {
    mh.msg_control = cbuf;
    mh.msg_controllen = CMSG_SPACE(sizeof(int) * nfds);
    cmsghdr* cm = CMSG_FIRSTHDR(&mh);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int) * nfds);
    memcpy(CMSG_DATA(cm), fds, sizeof(int) * nfds);
  }
  ssize_t r;
  do { r = sendmsg(sock, &mh, MSG_NOSIGNAL); } while (r < 0 && errno == EINTR);
  return r == (ssize_t)sizeof msg ? 0 : -1;
}

// returns 1 when a message was read, 0 when nothing is waiting, -1 on error / closed
int nvl_recv_fds(int sock, NvlExportMsg* msg, int* fds, int* nfds) {
  char cbuf[CMSG_SPACE(sizeof(int) * 16)];
  iovec iov{msg, sizeof *msg};
  msghdr mh;
  memset(&mh, 0, sizeof mh);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  mh.msg_control = cbuf;
  mh.msg_controllen = sizeof cbuf;
  ssize_t r = recvmsg(sock, &mh, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
  if (r < 0) return (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) ? 0 : -1;
  if (r == 0) return -1;
  *nfds = 0;
  for (cmsghdr* cm = CMSG_FIRSTHDR(&mh); cm; cm = CMSG_NXTHDR(&mh, cm)) {
    if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) {
      const int n = (int)((cm->cmsg_len - CMSG_LEN(0)) / sizeof(int));
      memcpy(fds, CMSG_DATA(cm), sizeof(int) * n);
      *nfds = n;
    }
  }
  if (r != (ssize_t)sizeof *msg || msg->magic != kNvlMagic || *nfds != msg->nslabs) {
    for (int i = 0; i < *nfds; ++i) close(fds[i]);
    return -1;
  }
  return 1;
}

// sender: map every region the peer has announced so far
void nvl_ingest(Comm* c, int device) {
  while (c->nvl_fd >= 0) {
    NvlExportMsg msg;
    int fds[16], nfds = 0;
    const int rc = nvl_recv_fds(c->nvl_fd, &msg, fds, &nfds);
    if (rc == 0) return;
    if (rc < 0) {
      close(c->nvl_fd);
      c->nvl_fd = -1;                              // direct path off for this connection; TCP carries on
      return;
    }
    if (msg.nslabs == 0) {                         // the peer deregistered the region: unmap it
      for (auto it = c->peer_mrs.begin(); it != c->peer_mrs.end(); ++it) {
        if (it->id == msg.mr_id) {
          if (it->region) fl_vmm_destroy(reinterpret_cast<FlVmmRegion*>(it->region));
          c->peer_mrs.erase(it);
          break;
        }
      }
      continue;
    }
    FlVmmRegion* r = fl_vmm_import(device < 0 ? 0 : device, fds, nfds, (size_t)msg.slab_bytes);
    for (int i = 0; i < nfds; ++i) close(fds[i]);
    if (!r) {
      FL_WARN("direct path: cannot map the peer's region %u (%s); that region stays on the staged path", msg.mr_id, fl_vmm_last_error());
      c->peer_mrs.push_back({msg.mr_id, nullptr, 0, nullptr});
      continue;
    }
    c->peer_mrs.push_back({msg.mr_id, fl_vmm_ptr(r), msg.size, r});
    FL_INFO("direct path: peer region %u (%llu bytes) mapped at %p", msg.mr_id, (unsigned long long)msg.size, fl_vmm_ptr(r));
  }
}

uint64_t random_u64() {
  static std::mt19937_64 rng{std::random_device{}()};
  static std::mutex mu;
  std::lock_guard<std::mutex> l(mu);
  return rng();
}

// ---------------------------------------------------------------------------------------------------
ncclResult_t fl_init(ncclDebugLogger_t logger) {
  std::lock_guard<std::mutex> l(g_mu);
  log_set(logger);
  if (g_cm) return ncclSuccess;
  params_reload();
  const Params& p = params();
  // Transport: "tcp", "rdma", or "auto" = RDMA when the provider finds devices (verbs NICs), else TCP.
  const std::string want = param_str("FUSELINK_TRANSPORT", "auto");
  int n_ib = 0;
  if (want != "tcp" && !(p.ib_disable && param_str("FUSELINK_RDMA_PROVIDER", "verbs") == "verbs")) n_ib = rdma_init(nullptr);
  g_rdma = n_ib > 0;
  if (want == "rdma" && !g_rdma) FL_WARN("FUSELINK_TRANSPORT=rdma but no RDMA device was found: using TCP");
  if (g_rdma) {
    g_ndev = n_ib;
    for (int d = 0; d < g_ndev; ++d) {
      const rdma::DeviceInfo di = rdma_device(d);
      snprintf(g_names[d], sizeof g_names[d], "%s", di.name.c_str());
      snprintf(g_pci[d], sizeof g_pci[d], "%s", di.pci_path.c_str());
      g_speed[d] = di.speed_mbps;
      g_guid[d] = di.guid;
      g_max_comms[d] = di.max_qp;
    }
  } else {
    g_ndev = (int)p.tcp_ndev;
    for (int d = 0; d < g_ndev; ++d) {
      snprintf(g_names[d], sizeof g_names[d], "fuselink-tcp%d", d);
      snprintf(g_pci[d], sizeof g_pci[d], "/sys/devices/virtual/net/fuselink%d", d);
      g_speed[d] = 100000;
      g_guid[d] = 0x464c0000ull + (uint64_t)d;
      g_max_comms[d] = 65536;
    }
  }
  int prio = (int)p.priority_dev;
  if (prio < 0 || prio >= g_ndev) prio = 0;
  g_cm = new ConnManager(g_ndev, prio, p.monitor_enable != 0, p.monitor_shm.c_str(), (int)p.monitor_timeout_us);
  if (p.cuda_ptrs) {
    if (fl_vmm_init(p.vmm_fake ? 1 : 0) == 0) g_ngpus = fl_vmm_device_count();
    else FL_WARN("CUDA registrations requested but the cuMem layer is unavailable: %s", fl_vmm_last_error());
  }
  FL_INFO("FuseLink plugin: %d device(s) over %s, degree %ld step %ld, monitor %s", g_ndev, g_rdma ? "RDMA" : "TCP (virtual NICs)",
          (long)p.degree, (long)p.step, g_cm->monitor() ? "on" : "off");
  return ncclSuccess;
}

ncclResult_t fl_devices(int* ndev) {
  *ndev = g_ndev;
  return ncclSuccess;
}

template <class P>
void fill_props_common(int dev, P* props) {
  props->name = g_names[dev];
  props->pciPath = g_pci[dev];
  props->guid = g_guid[dev];
  // the TCP transport reads/writes host memory; GPU buffers are accepted (and staged by the plugin) only on request
  props->ptrSupport = NCCL_PTR_HOST | (g_ngpus > 0 ? NCCL_PTR_CUDA : 0);
  props->speed = g_speed[dev];            // Mbps
  props->port = 0;
  props->latency = 0;
  props->maxComms = g_max_comms[dev];
  props->maxRecvs = 1;                    // grouped receives are not supported (as in the reference)
}
ncclResult_t fl_props_v6(int dev, ncclNetProperties_v6_t* props) {
  if (dev < 0 || dev >= g_ndev) return ncclInvalidArgument;
  fill_props_common(dev, props);
  return ncclSuccess;
}
ncclResult_t fl_props_v7(int dev, ncclNetProperties_v7_t* props) {
  if (dev < 0 || dev >= g_ndev) return ncclInvalidArgument;
  fill_props_common(dev, props);
  props->netDeviceType = NCCL_NET_DEVICE_HOST;
  props->netDeviceVersion = 0;
  return ncclSuccess;
}
ncclResult_t fl_props_v8(int dev, ncclNetProperties_v8_t* props) {
  if (dev < 0 || dev >= g_ndev) return ncclInvalidArgument;
  fill_props_common(dev, props);
  props->regIsGlobal = 0;
  props->netDeviceType = NCCL_NET_DEVICE_HOST;
  props->netDeviceVersion = 0;
  return ncclSuccess;
}

// ---------------------------------------------------------------------------------------------------
ncclResult_t fl_listen(int dev, void* opaque, void** listen_comm) {
  if (dev < 0 || dev >= g_ndev) return ncclInvalidArgument;
  Handle* h = reinterpret_cast<Handle*>(opaque);
  if (g_rdma) {
    RdmaListenComm* rl = nullptr;
    ncclResult_t rc = rdma_listen(dev, g_channel_counter.fetch_add(1), h, &rl);
    *listen_comm = rl;
    return rc;
  }
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
  lc->channel_id = g_channel_counter.fetch_add(1);   // global channel id, carried in the handle (src/plugin.cc:690-698)
  h->magic = kHandleMagic;
  h->addr = addr;
  h->channel_id = lc->channel_id;
  h->ndev = g_ndev;
  h->listen_dev = dev;
  if (g_ngpus > 0 && params().nvl) {
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
  *listen_comm = lc;
  return ncclSuccess;
}

// connect(): re-entered until *send_comm != NULL.  Stage 0 starts one control and ndev data connections,
// stage 1 finishes the TCP handshakes and sends the hellos.  All data sockets are set up eagerly (the
// reference builds its per-NIC side comms eagerly too, src/plugin.cc:727-753) so switching device later costs
// nothing.
ncclResult_t fl_connect_impl(int dev, void* opaque, void** send_comm) {
  *send_comm = nullptr;
  Handle* h = reinterpret_cast<Handle*>(opaque);
  if (h->magic != kHandleMagic) return ncclInvalidArgument;
  if (dev < 0 || dev >= g_ndev) return ncclInvalidArgument;
  if (g_rdma) {
    RdmaComm* rc = nullptr;
    ncclResult_t e = rdma_connect(dev, h, &rc);
    *send_comm = rc;
    return e;
  }
  Comm* c = reinterpret_cast<Comm*>(h->connect_state);
  if (!c) {
    c = new Comm();
    c->is_send = true;
    c->own_dev = dev;
    c->peer_dev = h->listen_dev;
    c->ndev = h->ndev < g_ndev ? h->ndev : g_ndev;
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
    if (h->nvl_token && g_ngpus > 0 && params().nvl) {
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
  *send_comm = c;
  return ncclSuccess;
}

ncclResult_t fl_accept_impl(void* listen_comm, void** recv_comm) {
  *recv_comm = nullptr;
  if (g_rdma) {
    RdmaComm* rc = nullptr;
    ncclResult_t e = rdma_accept(reinterpret_cast<RdmaListenComm*>(listen_comm), &rc);
    *recv_comm = rc;
    return e;
  }
  ListenComm* lc = reinterpret_cast<ListenComm*>(listen_comm);
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
      *recv_comm = c;
      return ncclSuccess;
    }
  }
  return ncclSuccess;
}

ncclResult_t fl_connect_v6(int dev, void* handle, void** send_comm) { return fl_connect_impl(dev, handle, send_comm); }
ncclResult_t fl_accept_v6(void* listen_comm, void** recv_comm) { return fl_accept_impl(listen_comm, recv_comm); }
ncclResult_t fl_connect_v7(int dev, void* handle, void** send_comm, ncclNetDeviceHandle_v7_t** dev_comm) {
  if (dev_comm) *dev_comm = nullptr;    // no device offload
  return fl_connect_impl(dev, handle, send_comm);
}
ncclResult_t fl_accept_v7(void* listen_comm, void** recv_comm, ncclNetDeviceHandle_v7_t** dev_comm) {
  if (dev_comm) *dev_comm = nullptr;
  return fl_accept_impl(listen_comm, recv_comm);
}

// ---------------------------------------------------------------------------------------------------
// Registration.  Host memory needs nothing.  A CUDA pointer is accepted when the cuMem layer can adopt it
// (a VMM allocation, NCCL_CUMEM_ENABLE=1): the region handle is kept so the buffer can be re-homed onto a
// relay GPU, which is what the reference's regMr does (src/plugin.cc:1168-1330).  The TCP data path itself
// only touches host memory, so a CUDA registration is refused unless the device transport is active.
void fl_dereg_region(MemHandle* m) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_adopted.find(m->base ? m->base : m->data);
  if (it != g_adopted.end() && it->second.region == m->region) {
    if (--it->second.refs == 0) {
      fl_vmm_destroy(m->region);
      g_adopted.erase(it);
    }
  } else {
    fl_vmm_destroy(m->region);
  }
  m->region = nullptr;
}

ncclResult_t fl_reg_mr_sz(void* comm, void* data, size_t size, int type, void** mhandle) {
  auto finish = [&](MemHandle* m) -> ncclResult_t {
    if (g_rdma) {
      m->rdma = rdma_reg(data, size);
      if (!m->rdma) {
        if (m->region) fl_dereg_region(m);
        delete m;
        return ncclSystemError;
      }
    }
    *mhandle = m;
    return ncclSuccess;
  };
  if (type == NCCL_PTR_HOST) return finish(new MemHandle{data, size, type, nullptr, 0, nullptr, nullptr});
  if (type != NCCL_PTR_CUDA || g_ngpus <= 0) {
    FL_WARN("regMr: pointer type %d is not supported (set FUSELINK_CUDA_PTRS=1 for device buffers)", type);
    return ncclInvalidUsage;
  }
  // Device buffer: adopt the cuMem allocation behind it and re-home it onto the relay GPU of this channel,
  // relay = (owner + channelId) % nGPUs (src/plugin.cc:1201), keeping the address and the contents and leaving the
  // owner GPU with read/write access (src/fuselink.cc:43-56).  A buffer that is not a cuMem allocation (or that is
  // registered again) is used where it is.
  const int channel = !comm ? 0 : g_rdma ? reinterpret_cast<RdmaComm*>(comm)->channel_id : reinterpret_cast<Comm*>(comm)->channel_id;
  MemHandle* m = new MemHandle{data, size, type, nullptr, 0, nullptr, nullptr};
  if (params().remap || params().nvl) {
    // NCCL registers sub-ranges of larger allocations: the unit that can be taken over is the whole mapping
    void* base = data;
    size_t span = size;
    if (fl_vmm_address_range(data, &base, &span) != 0) { base = data; span = size; }
    m->base = base;
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_adopted.find(base);
    if (it != g_adopted.end()) {
      // NCCL registers one buffer once per channel: the allocation is adopted (and re-homed) by the first
      // registration only, the others share it, so that an exported descriptor always names what the address maps
      it->second.refs++;
      m->region = it->second.region;
      m->mr_id = it->second.mr_id;
    } else {
      int dev = fl_vmm_pointer_device(data);
      if (dev < 0) dev = 0;
      FlVmmRegion* r = fl_vmm_adopt(base, span, dev);
      if (r) {
        const int relay = (dev + channel) % g_ngpus;
        long usec = 0;
        const int access[2] = {dev, relay};
        if (params().remap && relay != dev && fl_vmm_remap_slab(r, 0, relay, 1, access, 2, &usec) == 0)
          FL_INFO("regMr: %zu bytes at %p re-homed GPU %d -> GPU %d in %ld us", span, base, dev, relay, usec);   // "Remap time"
        m->region = r;
        m->mr_id = g_mr_counter.fetch_add(1);
        g_adopted[base] = Adopted{r, m->mr_id, 1};
      } else {
        FL_INFO("regMr: %p is not a cuMem allocation (%s): registered in place", data, fl_vmm_last_error());
      }
    }
  }
  return finish(m);
}
ncclResult_t fl_reg_mr(void* comm, void* data, int size, int type, void** mhandle) {
  return fl_reg_mr_sz(comm, data, (size_t)size, type, mhandle);
}
ncclResult_t fl_reg_mr_dmabuf(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle) {
  (void)offset; (void)fd;
  return fl_reg_mr_sz(comm, data, size, type, mhandle);
}
ncclResult_t fl_dereg_mr(void* comm, void* mhandle) {
  MemHandle* m = reinterpret_cast<MemHandle*>(mhandle);
  if (m && m->mr_id && comm && !g_rdma) {
    // a sender of this connection may hold a mapping of the region: tell it to let go
    Comm* c = reinterpret_cast<Comm*>(comm);
    for (auto it = c->exported.begin(); it != c->exported.end(); ++it) {
      if (*it != m->mr_id) continue;
      c->exported.erase(it);
      if (c->nvl_fd >= 0) {
        NvlExportMsg bye;
        memset(&bye, 0, sizeof bye);
        bye.magic = kNvlMagic;
        bye.mr_id = m->mr_id;
        nvl_send_fds(c->nvl_fd, bye, nullptr, 0);
      }
      break;
    }
  }
  if (m && m->rdma) rdma_dereg(m->rdma);
  if (m && m->region) fl_dereg_region(m);
  delete m;
  return ncclSuccess;
}

// ---------------------------------------------------------------------------------------------------
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

ncclResult_t fl_isend(void* send_comm, void* data, int size, int tag, void* mhandle, void** request) {
  if (g_rdma) {
    RdmaRequest* rr = nullptr;
    MemHandle* m = reinterpret_cast<MemHandle*>(mhandle);
    ncclResult_t e = rdma_isend(reinterpret_cast<RdmaComm*>(send_comm), g_cm, data, size, tag, m ? m->rdma : nullptr, &rr);
    *request = rr;
    return e;
  }
  Comm* c = reinterpret_cast<Comm*>(send_comm);
  *request = nullptr;
  ScopedTimer tm(&c->timers, T_ISEND, params().timers != 0);
  if (c->error) return (ncclResult_t)c->error;
  if (size < 0) return ncclInvalidArgument;
  comm_progress(c, g_cm);
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
  MemHandle* mh = reinterpret_cast<MemHandle*>(mhandle);
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
    int dev0 = next_alive_dev(c, g_cm->bid_tx(c->channel_id, c->own_dev, d.proposed_dev) % c->ndev);
    if (dev0 < 0) dev0 = 0;
    Stripe st;
    st.dev = dev0;
    st.hdr.magic = kFrameDirectMagic;
    st.hdr.slot = d.slot;
    st.hdr.total = (uint64_t)size;
    st.hdr.offset = 0;
    st.hdr.len = 0;
    st.hdr.tx_mask = g_cm->tx_mask(c->own_dev);
    r->stripes.push_back(st);
    c->data[dev0].txq.emplace_back(r, 0);
    r->moved = (uint64_t)size;
    g_direct_bytes.fetch_add((uint64_t)size, std::memory_order_relaxed);
    g_direct_msgs.fetch_add(1, std::memory_order_relaxed);
    c->msg_index++;
    comm_progress(c, g_cm);
    *request = r;
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
  const int first = g_cm->bid_tx(c->channel_id, c->own_dev, d.proposed_dev) % c->ndev;
  int nstripes = (int)p.degree;
  if (nstripes > c->ndev) nstripes = c->ndev;
  while (nstripes > 1 && (uint64_t)size / (uint64_t)nstripes < (uint64_t)p.min_stripe_bytes) --nstripes;
  const uint64_t mask = g_cm->tx_mask(c->own_dev);
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
        g_cm->release_tx(held);
        held = -1;
      }
      if (held < 0) {
        const int b = g_cm->borrow_tx(c->own_dev, used, dev);
        if (b >= 0 && c->data[b].fd >= 0) held = b;
        else if (b >= 0) g_cm->release_tx(b);
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
    g_cm->mark_tx(r->stripes[s].dev, r->stripes[s].hdr.len);
  }
  c->msg_index++;
  comm_progress(c, g_cm);
  *request = r;
  return ncclSuccess;
}

ncclResult_t fl_irecv(void* recv_comm, int n, void** data, int* sizes, int* tags, void** mhandles, void** request) {
  if (g_rdma) {
    *request = nullptr;
    if (n != 1) {
      FL_WARN("irecv: grouped receives (n=%d) are not supported", n);
      return ncclInternalError;
    }
    RdmaRequest* rr = nullptr;
    MemHandle* m = reinterpret_cast<MemHandle*>(mhandles[0]);
    ncclResult_t e = rdma_irecv(reinterpret_cast<RdmaComm*>(recv_comm), g_cm, data[0], sizes[0], tags[0], m ? m->rdma : nullptr, &rr);
    *request = rr;
    return e;
  }
  Comm* c = reinterpret_cast<Comm*>(recv_comm);
  *request = nullptr;
  ScopedTimer tm(&c->timers, T_IRECV, params().timers != 0);
  if (c->error) return (ncclResult_t)c->error;
  if (n != 1) {
    FL_WARN("irecv: grouped receives (n=%d) are not supported", n);
    return ncclInternalError;
  }
  if (sizes[0] < 0) return ncclInvalidArgument;
  Request* r = get_request(c);
  if (!r) return ncclSuccess;                      // everything in flight: NCCL retries
  r->is_send = false;
  r->data = reinterpret_cast<uint8_t*>(data[0]);
  r->size = (uint64_t)sizes[0];
  r->tag = tags[0];
  MemHandle* mh = reinterpret_cast<MemHandle*>(mhandles[0]);
  if (mh && mh->type == NCCL_PTR_CUDA && sizes[0] > 0) {
    r->stage.resize((size_t)sizes[0]);
    r->user = r->data;                       // bytes land in the bounce buffer and are copied up when complete
    r->data = r->stage.data();
  }
  // choose the device for this message: re-evaluated every kFinishedBatch completions and only when the
  // connection is quiescent, so a path switch never races with data in flight (src/plugin.cc:1700-1716)
  {
    ScopedTimer ts(&c->timers, T_SELECT, params().timers != 0);
    const bool quiescent = c->posted == c->completed;
    if (c->cur_dev < 0 || (c->n_finished >= kFinishedBatch && quiescent)) {
      c->cur_dev = g_cm->refresh_rx(c->channel_id, c->own_dev, c->cur_dev, c->peer_tx_mask, quiescent);
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
  if (mh && mh->mr_id && mh->region && c->nvl_fd >= 0 && sizes[0] > 0) {
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
      d.mr_off = (uint64_t)(reinterpret_cast<uint8_t*>(data[0]) - reinterpret_cast<uint8_t*>(fl_vmm_ptr(mh->region)));
    }
  }
  {
    ScopedTimer tp(&c->timers, T_POST_DESC, params().timers != 0);
    const uint8_t* p = reinterpret_cast<const uint8_t*>(&d);
    c->ctrl_tx.insert(c->ctrl_tx.end(), p, p + sizeof d);
    g_cm->touch_rx(c->cur_dev);                 // bytes are accounted on the device their stripes really arrive on
    c->posted++;
    comm_progress(c, g_cm);
  }
  *request = r;
  return ncclSuccess;
}

// TCP: data lands in host memory through the kernel's socket stack, nothing to flush.  RDMA into device memory:
// a one-byte read through the NIC when NCCL_GDR_FLUSH_DISABLE=0 (the reference ships with it set to 1,
// src/plugin.cc:887,1768-1799, and so does this plugin).
ncclResult_t fl_iflush(void* recv_comm, int n, void** data, int* sizes, void** mhandles, void** request) {
  *request = nullptr;
  if (!g_rdma || n < 1) return ncclSuccess;
  MemHandle* m = reinterpret_cast<MemHandle*>(mhandles[0]);
  if (!m || m->type != NCCL_PTR_CUDA) return ncclSuccess;
  RdmaRequest* rr = nullptr;
  ncclResult_t e = rdma_iflush(reinterpret_cast<RdmaComm*>(recv_comm), g_cm, data[0], sizes[0], m->rdma, &rr);
  *request = rr;
  return e;
}

ncclResult_t fl_test(void* request, int* done, int* sizes) {
  if (g_rdma) return rdma_test(reinterpret_cast<RdmaRequest*>(request), g_cm, done, sizes);
  Request* r = reinterpret_cast<Request*>(request);
  Comm* c = r->comm;
  *done = 0;
  {
    ScopedTimer tm(&c->timers, T_PROGRESS, params().timers != 0);
    comm_progress(c, g_cm);
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

ncclResult_t fl_close_send(void* send_comm) {
  if (g_rdma) {
    RdmaComm* rc = reinterpret_cast<RdmaComm*>(send_comm);
    if (rc && g_cm) for (int d : rc->extra_dev) if (d >= 0) g_cm->release_tx(d);
    rdma_close(rc);
    return ncclSuccess;
  }
  if (send_comm && g_cm) for (int d : reinterpret_cast<Comm*>(send_comm)->extra_dev) if (d >= 0) g_cm->release_tx(d);
  comm_close(reinterpret_cast<Comm*>(send_comm));
  return ncclSuccess;
}
ncclResult_t fl_close_recv(void* recv_comm) {
  if (g_rdma) {
    RdmaComm* rc = reinterpret_cast<RdmaComm*>(recv_comm);
    if (rc && g_cm && g_cm->monitor() && rc->cur_dev >= 0 && rc->cur_dev != rc->own_dev) fl_monitor_release(g_cm->monitor(), FL_DIR_RX, rc->cur_dev);
    rdma_close(rc);
    return ncclSuccess;
  }
  Comm* c = reinterpret_cast<Comm*>(recv_comm);
  if (c && g_cm && g_cm->monitor() && c->cur_dev >= 0 && c->cur_dev != c->own_dev)
    fl_monitor_release(g_cm->monitor(), FL_DIR_RX, c->cur_dev);
  comm_close(c);
  return ncclSuccess;
}
ncclResult_t fl_close_listen(void* listen_comm) {
  if (g_rdma) {
    rdma_close_listen(reinterpret_cast<RdmaListenComm*>(listen_comm));
    return ncclSuccess;
  }
  ListenComm* lc = reinterpret_cast<ListenComm*>(listen_comm);
  if (!lc) return ncclSuccess;
  for (auto& ps : lc->pending) close(ps.fd);
  for (auto& p : lc->partials) comm_close(p.comm);
  for (auto& np : lc->nvl_pending) close(np.fd);
  if (lc->uds_fd >= 0) close(lc->uds_fd);
  if (lc->fd >= 0) close(lc->fd);
  delete lc;
  return ncclSuccess;
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) ncclNet_v8_t ncclNetPlugin_v8 = {
    "FuseLink", fl_init, fl_devices, fl_props_v8, fl_listen, fl_connect_v7, fl_accept_v7, fl_reg_mr_sz, fl_reg_mr_dmabuf,
    fl_dereg_mr, fl_isend, fl_irecv, fl_iflush, fl_test, fl_close_send, fl_close_recv, fl_close_listen, nullptr, nullptr};

__attribute__((visibility("default"))) ncclNet_v7_t ncclNetPlugin_v7 = {
    "FuseLink", fl_init, fl_devices, fl_props_v7, fl_listen, fl_connect_v7, fl_accept_v7, fl_reg_mr, fl_reg_mr_dmabuf,
    fl_dereg_mr, fl_isend, fl_irecv, fl_iflush, fl_test, fl_close_send, fl_close_recv, fl_close_listen, nullptr, nullptr};

__attribute__((visibility("default"))) ncclNet_v6_t ncclNetPlugin_v6 = {
    "FuseLink", fl_init, fl_devices, fl_props_v6, fl_listen, fl_connect_v6, fl_accept_v6, fl_reg_mr, fl_reg_mr_dmabuf,
    fl_dereg_mr, fl_isend, fl_irecv, fl_iflush, fl_test, fl_close_send, fl_close_recv, fl_close_listen};

// Introspection for tests and tools (not part of the NCCL ABI).
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_decisions(void) { return g_cm ? g_cm->decisions() : 0; }
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_fallbacks(void) { return g_cm ? g_cm->fallbacks() : 0; }
__attribute__((visibility("default"))) void* fuselink_plugin_monitor(void) { return g_cm ? g_cm->monitor() : nullptr; }
// Stripes that were re-sent on another device after a data socket broke.
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_failovers(void) { return flnet::failover_count(); }
// Payload bytes / messages this process stored straight into a same-host peer's exported receive buffer.
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_direct_bytes(void) { return g_direct_bytes.load(); }
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_direct_msgs(void) { return g_direct_msgs.load(); }
// Peer regions a send connection currently has mapped (direct path).
__attribute__((visibility("default"))) int fuselink_comm_peer_regions(void* send_comm) {
  return g_rdma || !send_comm ? 0 : (int)reinterpret_cast<Comm*>(send_comm)->peer_mrs.size();
}
// Device carrying the stripes of a send request (stripe index s); -1 when out of range.
__attribute__((visibility("default"))) int fuselink_request_stripe_dev(void* request, int s) {
  if (g_rdma) {
    RdmaRequest* rr = reinterpret_cast<RdmaRequest*>(request);
    return (!rr || s < 0 || s >= (int)rr->pieces.size()) ? -1 : rr->pieces[s].dev;
  }
  Request* r = reinterpret_cast<Request*>(request);
  if (!r || s < 0 || s >= (int)r->stripes.size()) return -1;
  return r->stripes[s].dev;
}

}  // extern "C"
