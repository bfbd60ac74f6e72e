// RDMA data transport of the plugin: the receiver-driven write protocol of the reference's verbs path
// (src/plugin.cc:1394-1677, 1816-1955) on top of the provider interface, so the same code drives libibverbs
// and the software NIC.
//
//   irecv   keeps zero-length receives posted on every queue pair and RDMA-writes a descriptor {address, size,
//           tag, slot, proposed device, the buffer's remote key on every device} into the sender's FIFO
//           (256 slots; the reference's ncclIbSendFifo, src/plugin.cc:487-503).
//   isend   takes the FIFO entry at its head, checks tag and size, cuts the message into pieces -- one stripe per
//           selected device (NCCL_FUSELINK_DEGREE / _STEP), each stripe over the queue pairs of that device when
//           NCCL_IB_SPLIT_DATA_ON_QPS is set, in multiples of 128 bytes (src/plugin.cc:1467-1472) -- and posts for
//           every piece an RDMA write followed by a zero-length write-with-immediate, or a single
//           write-with-immediate below NCCL_IB_AR_THRESHOLD (src/plugin.cc:1454-1462).  The first piece also
//           writes {actual size, sender's device mask} into the receiver's record for the slot.
//   test    polls the completion queues: a send is done when all its pieces completed, a receive when it has
//           seen every piece the immediate data announces (slot in bits 0-7, piece count in 8-15, piece index in 16-23).
//   A device whose queue pair fails (retry exceeded, flushed) is marked dead for the connection: the sender posts the
//   affected pieces again on another device, the receiver moves its descriptor writes to another device and writes the
//   descriptors of its unfinished receives again (both are idempotent).  A remote-access error is not a link failure
//   and fails the connection.
//
// Connections are bootstrapped over TCP like the reference's (src/plugin.cc:700-880): the two ends exchange
// queue-pair addresses, FIFO address and keys, then a "ready" byte.
#pragma once
#include <stdint.h>

#include <deque>
#include <vector>

#include "conn_manager.h"
#include "nccl_net_abi.h"
#include "rdma_provider.h"
#include "tcp_transport.h"

namespace flnet {

constexpr int kRdmaMaxQps = 4;            // per device and connection (NCCL_IB_QPS_PER_CONNECTION, capped)
constexpr int kFifoSignalEvery = 64;      // descriptor writes are unsignalled except one in this many

struct RdmaMrSet {                        // one registration per device
  rdma::Mr* mr[kMaxDev];
  void* data;
  size_t size;
};

struct RdmaDesc {                         // 128 bytes, receiver -> sender FIFO
  uint64_t addr;
  uint64_t size;
  int32_t tag;
  uint32_t slot;
  int32_t proposed_dev;
  uint32_t pad0;
  uint32_t rkey[kMaxDev];
  uint64_t pad1[3];
  uint64_t seq;                           // index of the post + 1; written last, polled by the sender
};
static_assert(sizeof(RdmaDesc) == 128, "descriptor layout");

struct RdmaDoneRec {                      // sender -> receiver, per slot
  uint64_t size;
  uint64_t tx_mask;
};

struct RdmaConnInfo {                     // exchanged over the bootstrap socket
  uint32_t magic;
  int32_t ndev;
  int32_t nqps;
  int32_t own_dev;
  rdma::QpInfo qp[kMaxDev][kRdmaMaxQps];
  uint64_t fifo_addr;                     // sender only
  uint32_t fifo_rkey[kMaxDev];
  uint64_t done_addr;                     // receiver only
  uint32_t done_rkey[kMaxDev];
};

struct RdmaPiece {
  int dev;
  int q;                                  // queue pair index on that device
  uint64_t off;
  uint64_t len;
  uint8_t gen = 0;                        // bumped when the piece is posted again after a device failure
  bool done = false;
};

struct RdmaComm;
struct RdmaRequest {
  bool used = false, is_send = false, is_flush = false;
  RdmaComm* comm = nullptr;
  uint32_t slot = 0;
  uint64_t size = 0;
  uint64_t total = UINT64_MAX;
  int tag = 0;
  int pieces_total = -1;                  // recv: unknown until the first immediate arrives
  int pieces_done = 0;
  uint64_t piece_mask = 0;                // recv: pieces whose immediate arrived (a piece sent twice counts once)
  int rx_dev = 0;
  uint64_t fifo_idx = 0;                  // recv: position of the descriptor in the sender's FIFO
  uint64_t last_progress_ns = 0;
  std::vector<RdmaPiece> pieces;          // send only
  const uint8_t* data = nullptr;          // send: what is needed to post a piece again
  RdmaMrSet* mr = nullptr;
  RdmaDesc desc;
  bool bad_key = false;                   // test hook
};

struct RdmaDevEnd {
  rdma::Cq* cq = nullptr;
  rdma::Qp* qp[kRdmaMaxQps] = {nullptr, nullptr, nullptr, nullptr};
};

struct RdmaComm {
  bool is_send = false;
  int own_dev = 0, peer_dev = 0, ndev = 1, nqps = 1, channel_id = 0;
  int ctrl_fd = -1;
  int error = 0;
  RdmaDevEnd dev[kMaxDev];
  RdmaRequest reqs[kMaxRequests];
  // sender
  RdmaDesc* fifo = nullptr;               // written by the peer
  RdmaMrSet* fifo_mr = nullptr;
  uint64_t fifo_head = 0;
  RdmaDoneRec* done_src = nullptr;        // staging for the per-slot records
  RdmaMrSet* done_src_mr = nullptr;
  uint64_t remote_done_addr = 0;
  uint32_t remote_done_rkey[kMaxDev];
  // receiver
  RdmaDoneRec* done = nullptr;            // written by the peer
  RdmaMrSet* done_mr = nullptr;
  RdmaDesc* fifo_src = nullptr;           // staging for descriptors
  RdmaMrSet* fifo_src_mr = nullptr;
  uint64_t remote_fifo_addr = 0;
  uint32_t remote_fifo_rkey[kMaxDev];
  uint64_t fifo_tail = 0;
  int ctrl_dev = 0;                       // device whose queue pair carries the descriptor writes
  bool dead[kMaxDev] = {};                // devices given up after a queue-pair failure
  // flush of device memory after a receive (NCCL_GDR_FLUSH_DISABLE=0): a queue pair connected to itself reads one
  // byte of the buffer back through the NIC, which orders the NIC's earlier writes before it (src/plugin.cc:1768-1799)
  rdma::Qp* flush_qp = nullptr;
  uint8_t* flush_buf = nullptr;
  RdmaMrSet* flush_mr = nullptr;
  // selection state (same meaning as in the TCP transport)
  int cur_dev = -1, n_finished = 0, posted = 0, completed = 0;
  uint64_t peer_tx_mask = ~0ull, msg_index = 0;
  int extra_dev[kMaxDev];                 // sender: device borrowed for stripe k > 0, kept for the life of the connection
  RdmaComm() { for (int& d : extra_dev) d = -1; }
  // bootstrap
  int stage = 0;
  size_t io_done = 0;
  uint64_t since_ns = 0;                  // accepted at (receiver): a bootstrap that stalls is dropped
  RdmaConnInfo mine, theirs;
  Timers timers;                          // FUSELINK_TIMERS=1: isend / irecv / descriptor post / completion polling / flush
};

struct RdmaListenComm {
  int fd = -1;
  int dev = 0;
  int channel_id = 0;
  std::vector<RdmaComm*> pending;         // accepted, bootstrap in progress
};

// Device table / lifetime
int rdma_init(ConnManager* cm);                           // number of devices (0: transport unavailable)
rdma::DeviceInfo rdma_device(int dev);

ncclResult_t rdma_listen(int dev, int channel_id, Handle* h, RdmaListenComm** out);
ncclResult_t rdma_connect(int dev, Handle* h, RdmaComm** out);      // re-entrant, *out stays null until connected
ncclResult_t rdma_accept(RdmaListenComm* lc, RdmaComm** out);       // re-entrant
// Registers [data, data + size) on every device, through the registration cache.  With dmabuf_fd >= 0 the memory is
// reached through that dma-buf (`data` lies dmabuf_offset bytes into it) instead of by address.
RdmaMrSet* rdma_reg(void* data, size_t size, int dmabuf_fd = -1, uint64_t dmabuf_offset = 0);
void rdma_dereg(RdmaMrSet* m);
bool rdma_dmabuf_supported();                             // every device can register a dma-buf
bool rdma_peer_memory_supported();                        // device pointers can be registered by address
void rdma_mr_counters(unsigned long long* registrations, unsigned long long* cache_hits, unsigned long long* dmabuf);
ncclResult_t rdma_isend(RdmaComm* c, ConnManager* cm, void* data, int size, int tag, RdmaMrSet* mr, RdmaRequest** out);
ncclResult_t rdma_irecv(RdmaComm* c, ConnManager* cm, void* data, int size, int tag, RdmaMrSet* mr, RdmaRequest** out);
ncclResult_t rdma_iflush(RdmaComm* c, ConnManager* cm, void* data, int size, RdmaMrSet* mr, RdmaRequest** out);   // *out null: nothing to do
ncclResult_t rdma_test(RdmaRequest* r, ConnManager* cm, int* done, int* size);
void rdma_close(RdmaComm* c);
void rdma_close_listen(RdmaListenComm* lc);

}  // namespace flnet
