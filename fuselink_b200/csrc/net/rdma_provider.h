// What the RDMA transport needs from a NIC, as an interface with two implementations:
//
//   * VerbsProvider (verbs_provider.cc): libibverbs opened with dlopen, the way the reference reaches it
//     through NCCL's wrappers (src/extern/ibvwrap.h:30-90) -- protection domains, memory regions, completion
//     queues, reliable-connected queue pairs, RDMA write / write-with-immediate, zero-length receives.
//   * SoftProvider (soft_provider.cc): the same semantics between processes of one machine over Unix
//     sockets (a software NIC).  It exists so the transport's protocol -- descriptor FIFO, striping over
//     devices and queue pairs, immediate-data completion, remote-key checks -- runs and is tested on machines
//     without RDMA hardware.
//
// The surface is the subset of verbs the reference's data path uses (src/plugin.cc:626-688 queue pairs,
// :1168-1330 registration, :1394-1500 posting, :1816-1955 completion handling), with plain structs instead of
// the verbs ABI so that nothing above this file depends on rdma-core headers.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace flnet {
namespace rdma {

enum LinkLayer : uint8_t { kLinkUnknown = 0, kLinkIB = 1, kLinkEthernet = 2 };

struct DeviceInfo {
  std::string name;
  int port = 1;
  uint64_t guid = 0;
  std::string pci_path;
  int speed_mbps = 0;           // width x per-lane rate, as the reference's tables give it (src/plugin.cc:140-161)
  int max_qp = 0;
  LinkLayer link = kLinkUnknown;
  bool relaxed_ordering = false; // the library knows IBV_ACCESS_RELAXED_ORDERING (src/plugin.cc:164-172)
};

// What the two ends exchange out of band before a queue pair can be connected (src/plugin.cc:432-446).
struct QpInfo {
  uint32_t qpn;
  uint16_t lid;
  uint8_t link;                 // LinkLayer
  uint8_t port;
  uint8_t mtu;                  // verbs enum value (1..5)
  uint8_t pad[7];
  uint8_t gid[16];
  uint64_t cookie;              // provider-private (the software NIC puts its process id here)
  // enhanced connection establishment: vendor options the two ends agree on before the queue pair is connected
  // (src/plugin.cc:393-395, 801-802, 856-857, 986-994)
  uint32_t ece_vendor_id, ece_options, ece_comp_mask, ece_supported;
};

struct Ece {
  uint32_t vendor_id = 0, options = 0, comp_mask = 0;
};

struct Pd;
struct Cq;
struct Qp;
struct Mr {
  uint32_t lkey = 0, rkey = 0;
  void* addr = nullptr;
  size_t len = 0;
  void* impl = nullptr;
};

enum Opcode : uint8_t { kWrite = 0, kWriteImm = 1, kRead = 2 };   // kRead: laddr receives len bytes from raddr

struct SendWr {
  uint64_t wr_id = 0;
  Opcode op = kWrite;
  const void* laddr = nullptr;  // may be null when len == 0
  uint32_t len = 0;
  uint32_t lkey = 0;
  uint64_t raddr = 0;
  uint32_t rkey = 0;
  uint32_t imm = 0;
  bool signaled = false;
  bool inline_data = false;     // the payload is copied at post time (small control writes)
};

enum WcStatus : int { kWcOk = 0, kWcRemoteAccess = 10, kWcRetryExceeded = 12, kWcFlushed = 5, kWcGeneral = 21 };

struct Completion {
  uint64_t wr_id = 0;
  int status = kWcOk;
  bool is_recv = false;         // a receive consumed by a write-with-immediate
  uint32_t imm = 0;
  uint32_t byte_len = 0;
  uint32_t qpn = 0;
};

struct QpCaps {
  int max_send_wr = 512;
  int max_recv_wr = 512;
  int max_inline = 0;
};

struct QpConnectParams {        // NCCL_IB_* knobs of the reference (src/plugin.cc:87-93)
  int gid_index = 0, timeout = 18, retry_cnt = 7, pkey = 0, sl = 0, tc = 0;
};

enum AccessFlags : int { kAccessLocalWrite = 1, kAccessRemoteWrite = 2, kAccessRemoteRead = 4, kAccessRelaxedOrdering = 1 << 20 };

class Provider {
 public:
  virtual ~Provider() {}
  virtual const char* name() const = 0;
  virtual int device_count() = 0;
  virtual DeviceInfo device(int dev) = 0;

  virtual Pd* alloc_pd(int dev) = 0;                 // one per device, shared by every connection (reference: up-front, :290-297)
  virtual void dealloc_pd(Pd* pd) = 0;
  virtual Mr* reg_mr(Pd* pd, void* addr, size_t len, int access) = 0;
  // Registration of device memory through a dma-buf file descriptor: `len` bytes starting `offset` bytes into the
  // buffer behind `fd`, addressed by the peer (and by local work requests) as [iova, iova + len).  The descriptor may be
  // closed once the call returns.  Null when the provider cannot (src/plugin.cc:1277-1280 is the reference's use).
  virtual Mr* reg_dmabuf_mr(Pd* pd, int fd, uint64_t offset, size_t len, uint64_t iova, int access) {
    (void)pd; (void)fd; (void)offset; (void)len; (void)iova; (void)access;
    return nullptr;
  }
  // Can device `dev` register dma-bufs (the reference probes ibv_reg_dmabuf_mr with a dummy descriptor,
  // src/plugin.cc:337-356), and can it register device pointers by address (a peer-memory kernel module, :321-331)?
  virtual bool dmabuf_supported(int dev) { (void)dev; return false; }
  virtual bool peer_memory_supported() { return false; }
  virtual void dereg_mr(Mr* mr) = 0;
  virtual Cq* create_cq(int dev, int depth) = 0;
  virtual void destroy_cq(Cq* cq) = 0;
  virtual Qp* create_qp(Pd* pd, Cq* cq, const QpCaps& caps) = 0;
  virtual void destroy_qp(Qp* qp) = 0;
  virtual int query_qp_info(Qp* qp, int gid_index, QpInfo* out) = 0;           // local side of the exchange
  virtual int connect_qp(Qp* qp, const QpInfo& remote, const QpConnectParams& p) = 0;   // INIT -> RTR -> RTS
  // Enhanced connection establishment, both before connect_qp.  query: the options this queue pair offers (after a
  // set: what is left of them).  set: take the peer's options.  False when the device or the library has none.
  virtual bool query_ece(Qp* qp, Ece* out) { (void)qp; (void)out; return false; }
  virtual bool set_ece(Qp* qp, const Ece& ece) { (void)qp; (void)ece; return false; }
  virtual int post_send(Qp* qp, const SendWr* wrs, int n) = 0;                 // a chain, executed in order
  virtual int post_recv(Qp* qp, uint64_t wr_id) = 0;                           // zero-length receive
  virtual int poll_cq(Cq* cq, int max, Completion* out) = 0;
  // Software NICs move bytes here; hardware ones do nothing.
  virtual void progress() {}
  // Blocks up to timeout_ms for an asynchronous event of `dev` (port down, fatal ...); returns 1 and a
  // description when one arrived, 0 on timeout, -1 when the device is gone / unsupported.
  virtual int wait_async_event(int dev, int timeout_ms, std::string* what) { (void)dev; (void)timeout_ms; (void)what; return -1; }
};

// FUSELINK_RDMA_PROVIDER = verbs | soft | none (default: verbs, which reports 0 devices without libibverbs).
// The object lives for the whole process.
Provider* get_provider();
Provider* make_soft_provider();
Provider* make_verbs_provider();

}  // namespace rdma
}  // namespace flnet
