// ncclNet plugin entry points: `libnccl-net-fuselink.so`, loaded by NCCL with NCCL_NET_PLUGIN=fuselink.
//
// Surface kept from the reference (src/plugin.cc:1997-2018): the table is named "FuseLink" and is exported
// as ncclNetPlugin_v7 with a v6 alias; getDeviceMr / irecvConsumed are NULL; multi-receive (n > 1) is
// rejected (src/plugin.cc:1449-1450,1879-1880).  A v8 table (size_t registration sizes) is exported too so
// that current NCCL releases find a version they probe for.
//
// What differs: this file is the table, the registration of buffers and the dispatch to one of two transports.  The
// TCP transport (tcp_endpoints.cc, tcp_transport.*) works on any machine; the RDMA transport (rdma_transport.*) drives
// libibverbs devices where they exist (verbs_provider.cc) or a software NIC in tests (soft_provider.cc).  Path
// selection goes through ConnManager and the lock-free monitor instead of peeking into NCCL's private proxy
// structures (src/fuselink.h:18-37): each transport counts its own posted / completed requests to know when a
// connection is quiescent.
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <mutex>

#include "conn_manager.h"
#include "ib_transport.h"
#include "logging.h"
#include "nccl_net_abi.h"
#include "nvl_channel.h"
#include "params.h"
#include "rdma_transport.h"
#include "tcp_transport.h"
#include "../mem/vmm.h"

using namespace flnet;

namespace {

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
  // on the RDMA transport a NIC must be able to reach device memory: by address (peer-memory module) or through a dma-buf
  // (the reference's ncclIbGdrSupport / ncclIbDmaBufSupport, src/plugin.cc:321-356, 367-372)
  const bool dmabuf = g_rdma && g_ngpus > 0 && rdma_dmabuf_supported();
  const bool cuda = g_ngpus > 0 && (!g_rdma || dmabuf || rdma_peer_memory_supported());
  props->ptrSupport = NCCL_PTR_HOST | (cuda ? NCCL_PTR_CUDA : 0) | (dmabuf ? NCCL_PTR_DMABUF : 0);
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
  ListenComm* lc = nullptr;
  ncclResult_t rc = tcp_listen(dev, g_ndev, g_channel_counter.fetch_add(1), g_ngpus > 0 && params().nvl != 0, h, &lc);
  *listen_comm = lc;
  return rc;
}

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
  Comm* tc = nullptr;
  ncclResult_t e = tcp_connect(dev, g_ndev, g_ngpus > 0 && params().nvl != 0, h, &tc);
  *send_comm = tc;
  return e;
}

ncclResult_t fl_accept_impl(void* listen_comm, void** recv_comm) {
  *recv_comm = nullptr;
  if (g_rdma) {
    RdmaComm* rc = nullptr;
    ncclResult_t e = rdma_accept(reinterpret_cast<RdmaListenComm*>(listen_comm), &rc);
    *recv_comm = rc;
    return e;
  }
  Comm* tc = nullptr;
  ncclResult_t e = tcp_accept(reinterpret_cast<ListenComm*>(listen_comm), &tc);
  *recv_comm = tc;
  return e;
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

// `given_fd` / `given_offset`: the dma-buf NCCL hands to regMrDmaBuf (-1: none).
ncclResult_t fl_reg_mr_impl(void* comm, void* data, size_t size, int type, int given_fd, uint64_t given_offset, void** mhandle) {
  auto finish = [&](MemHandle* m) -> ncclResult_t {
    if (g_rdma) {
      // How a NIC reaches device memory (src/plugin.cc:321-356, 1277-1289): by address when a peer-memory module is
      // loaded, else through a dma-buf.  A buffer this plugin has taken over may have been re-homed, and a descriptor
      // NCCL took before that names the old physical memory: such a buffer gets a descriptor of its own, taken now.
      int fd = -1, own_fd = -1;
      uint64_t off = 0;
      if (type == NCCL_PTR_CUDA) {
        if (given_fd >= 0 && !m->region) {
          fd = given_fd;
          off = given_offset;
        } else if ((given_fd >= 0 || !rdma_peer_memory_supported()) && rdma_dmabuf_supported() &&
                   fl_vmm_dmabuf_fd(data, size ? size : 1, &own_fd, &off) == 0) {
          fd = own_fd;
        } else if (!rdma_peer_memory_supported()) {
          FL_WARN("regMr: the NICs cannot reach device memory at %p: no peer-memory module and no dma-buf (%s)", data, fl_vmm_last_error());
          if (m->region) fl_dereg_region(m);
          delete m;
          return ncclInvalidUsage;
        } else {
          FL_INFO("regMr: no dma-buf for %p (%s); registering by address", data, fl_vmm_last_error());
        }
      }
      m->rdma = rdma_reg(data, size, fd, off);
      if (own_fd >= 0) close(own_fd);
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
ncclResult_t fl_reg_mr_sz(void* comm, void* data, size_t size, int type, void** mhandle) {
  return fl_reg_mr_impl(comm, data, size, type, -1, 0, mhandle);
}
ncclResult_t fl_reg_mr(void* comm, void* data, int size, int type, void** mhandle) {
  return fl_reg_mr_impl(comm, data, (size_t)size, type, -1, 0, mhandle);
}
ncclResult_t fl_reg_mr_dmabuf(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle) {
  return fl_reg_mr_impl(comm, data, size, type, fd, offset, mhandle);
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
ncclResult_t fl_isend(void* send_comm, void* data, int size, int tag, void* mhandle, void** request) {
  if (g_rdma) {
    RdmaRequest* rr = nullptr;
    MemHandle* m = reinterpret_cast<MemHandle*>(mhandle);
    ncclResult_t e = rdma_isend(reinterpret_cast<RdmaComm*>(send_comm), g_cm, data, size, tag, m ? m->rdma : nullptr, &rr);
    *request = rr;
    return e;
  }
  MemHandle* m = reinterpret_cast<MemHandle*>(mhandle);
  TcpMem mem{m ? m->type : NCCL_PTR_HOST, m ? m->region : nullptr, m ? m->mr_id : 0u};
  Request* tr = nullptr;
  ncclResult_t e = tcp_isend(reinterpret_cast<Comm*>(send_comm), g_cm, data, size, tag, &mem, &tr);
  *request = tr;
  return e;
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
  *request = nullptr;
  if (n != 1) {
    FL_WARN("irecv: grouped receives (n=%d) are not supported", n);
    return ncclInternalError;
  }
  MemHandle* m = reinterpret_cast<MemHandle*>(mhandles[0]);
  TcpMem mem{m ? m->type : NCCL_PTR_HOST, m ? m->region : nullptr, m ? m->mr_id : 0u};
  Request* tr = nullptr;
  ncclResult_t e = tcp_irecv(reinterpret_cast<Comm*>(recv_comm), g_cm, data[0], sizes[0], tags[0], &mem, &tr);
  if (m && mem.mr_id == 0) m->mr_id = 0;          // the region turned out not to be exportable: do not try again
  *request = tr;
  return e;
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
  return tcp_test(reinterpret_cast<Request*>(request), g_cm, done, sizes);
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
  tcp_close_listen(reinterpret_cast<ListenComm*>(listen_comm));
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
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_direct_bytes(void) { return flnet::tcp_direct_bytes(); }
__attribute__((visibility("default"))) unsigned long long fuselink_plugin_direct_msgs(void) { return flnet::tcp_direct_msgs(); }
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
