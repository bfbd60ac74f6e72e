// TCP data transport of the plugin: every "device" is a virtual NIC (one data socket per device and
// connection) and one control socket carries the receiver's descriptors.
//
// The reference has sockets for out-of-band control only (src/extern/socket.{h,cc}) and moves data with
// RDMA writes; its wire protocol is receiver-driven: irecv publishes {address, size, tag, slot, chosen
// NIC} into the sender's FIFO and isend consumes FIFO slots in order (src/plugin.cc:1616-1677,
// 1500-1614).  The same protocol runs here over byte streams: a descriptor travels on the control socket,
// data travels as framed stripes on the data socket of the device the receiver chose (or of several
// devices when NCCL_FUSELINK_DEGREE > 1), and both ends progress from test() without blocking.
#pragma once
#include <netinet/in.h>
#include <stdint.h>

#include <deque>
#include <vector>

#include "conn_manager.h"
#include "logging.h"
#include "nccl_net_abi.h"

struct FlVmmRegion;   // csrc/mem/vmm.h

namespace flnet {

constexpr uint64_t kHandleMagic = 0x464c4e4b48444c31ull;  // "FLNKHDL1"
constexpr int kMaxDev = 16;
constexpr int kMaxRequests = 256;       // MAX_REQUESTS of the reference (src/plugin.cc:382-383)
constexpr int kFinishedBatch = 8;       // N_FINISHED_BATCH (src/plugin.cc:38)

struct Handle {                          // what listen() publishes; <= NCCL_NET_HANDLE_MAXSIZE bytes
  uint64_t magic;
  sockaddr_in6 addr;                     // v4 addresses are stored v4-mapped
  int32_t channel_id;
  int32_t ndev;
  int32_t listen_dev;
  int32_t pad;
  uint64_t nvl_token;                    // non-zero: the listener also accepts a same-host side channel for cuMem handles
  void* connect_state;                   // in-progress SendComm between re-entrant connect() calls
};
static_assert(sizeof(Handle) <= NCCL_NET_HANDLE_MAXSIZE, "handle too large");

struct Hello {                           // first bytes on every new socket
  uint64_t magic;
  uint64_t comm_uid;
  int32_t kind;                          // 0 control, 1 data
  int32_t dev;                           // virtual NIC index of a data socket
  int32_t sender_dev;                    // the sender's own (affine) device
  int32_t ndev;
};

struct RecvDesc {                        // receiver -> sender, control socket
  uint32_t magic;
  uint32_t slot;                         // receiver's request slot; echoed in every frame
  int32_t tag;
  int32_t proposed_dev;                  // the reference's fuselink_offset
  uint64_t size;                         // posted receive size (upper bound)
  uint64_t seq;                          // order of posting
  uint32_t mr_id;                        // direct path: id of the exported receive region (0 = none)
  uint32_t flags;                        // bit 0: the receive buffer was exported, the sender may write it directly
  uint64_t mr_off;                       // byte offset of the receive buffer inside that region
};
constexpr uint32_t kDescDirectOk = 1u;

struct NvlExportMsg {                    // receiver -> sender on the Unix side channel, with the slab fds as SCM_RIGHTS
  uint64_t magic;
  uint32_t mr_id;
  int32_t nslabs;
  uint64_t size;
  uint64_t slab_bytes;
};
constexpr uint64_t kNvlMagic = 0x464c4e564c313030ull;   // "FLNVL100"

struct FrameHdr {                        // sender -> receiver, in front of every stripe on a data socket
  uint32_t magic;
  uint32_t slot;
  uint64_t total;                        // full message size (may be smaller than the posted size)
  uint64_t offset;
  uint64_t len;
  uint64_t tx_mask;                      // sender's device availability (the reference's immediate data)
};

struct Stripe {
  int dev;
  FrameHdr hdr;
  size_t hdr_sent = 0;
  size_t sent = 0;
};

struct Comm;

struct Request {
  bool used = false;
  bool is_send = false;
  bool done = false;
  Comm* comm = nullptr;
  uint32_t slot = 0;
  uint8_t* data = nullptr;
  uint64_t size = 0;                     // send: message size; recv: posted size
  uint64_t total = UINT64_MAX;           // recv: actual size once the first frame arrived
  uint64_t moved = 0;                    // bytes sent / received so far
  int tag = 0;
  uint64_t last_progress_ns = 0;
  std::vector<Stripe> stripes;           // send only
  std::vector<uint8_t> stage;            // host bounce buffer when the user buffer is device memory
  uint8_t* user = nullptr;               // device address the staged bytes belong to (null: no staging)
  bool direct = false;                   // recv: the sender wrote the bytes straight into the exported buffer
  std::vector<uint64_t> got_offsets;     // recv: offsets of the stripes that arrived completely (a re-sent stripe counts once)
  size_t stripes_done = 0;
};

struct DataSock {
  int fd = -1;
  // send side: stripes queued on this socket, in order
  std::deque<std::pair<Request*, int>> txq;   // (request, stripe index)
  uint64_t tx_bytes = 0;
  // recv side: frame parser
  FrameHdr rx_hdr;
  size_t rx_hdr_got = 0;
  uint64_t rx_payload_got = 0;
  bool rx_in_payload = false;
};

struct Comm {
  bool is_send = false;
  int own_dev = 0;                       // device NCCL bound this comm to
  int peer_dev = 0;
  int ndev = 1;
  int channel_id = 0;
  uint64_t uid = 0;
  int ctrl_fd = -1;
  DataSock data[kMaxDev];
  Request reqs[kMaxRequests];
  int error = 0;                         // sticky ncclResult_t
  bool fault_fired = false;              // test hook: the injected link failure happens once per connection
  // control stream
  std::vector<uint8_t> ctrl_tx;          // receiver: descriptors not yet written
  uint8_t ctrl_rx[sizeof(RecvDesc)];
  size_t ctrl_rx_got = 0;
  std::deque<RecvDesc> fifo;             // sender: descriptors received, in posting order
  // selection state
  int cur_dev = -1;                      // receiver: device proposed for new messages
  int n_finished = 0;
  int posted = 0, completed = 0;
  uint64_t post_seq = 0;
  uint64_t peer_tx_mask = ~0ull;         // receiver: last mask advertised by the sender (txAvailable)
  uint64_t msg_index = 0;
  int extra_dev[kMaxDev];                // sender: device borrowed for stripe k > 0, kept for the life of the connection (-1: none yet)
  Comm() { for (int& d : extra_dev) d = -1; }
  // connect progress
  int connect_stage = 0;
  std::vector<int> pending_fds;
  std::vector<size_t> hello_sent;
  int connect_retries = 0;               // refused connection attempts so far (all sockets of this connect)
  Timers timers;
  // same-host direct path (cuMem export/import)
  int nvl_fd = -1;                       // Unix side channel, -1 when the peer is on another host or the path is off
  std::vector<uint32_t> exported;        // receiver: region ids already sent to this peer
  struct PeerMr { uint32_t id; void* base; uint64_t size; void* region; };
  std::vector<PeerMr> peer_mrs;          // sender: the peer's regions as mapped here
};

struct PendingSock {
  int fd;
  Hello hello;
  size_t got;
  uint64_t since_ns = 0;                 // accepted at; a socket that does not finish its hello in time is dropped
};
constexpr uint64_t kHelloTimeoutNs = 10ull * 1000000000ull;       // silent accepted sockets
constexpr uint64_t kPartialTimeoutNs = 120ull * 1000000000ull;    // a connection whose sockets never all arrive

struct ListenComm {
  int fd = -1;
  int dev = 0;
  int channel_id = 0;
  std::vector<PendingSock> pending;      // accepted, hello not complete yet
  struct Partial { uint64_t uid; Comm* comm; int have; uint64_t since_ns; };
  std::vector<Partial> partials;         // sockets grouped by connection uid
  int uds_fd = -1;                       // listener of the same-host side channel
  uint64_t nvl_token = 0;
  struct NvlPending { int fd; uint64_t uid; };
  std::vector<NvlPending> nvl_pending;   // side channels accepted, not yet matched to a connection
};

// What the transport needs to know about a registered buffer (plugin.cc owns the registration itself).
struct TcpMem {
  int type;                              // NCCL_PTR_HOST / NCCL_PTR_CUDA
  ::FlVmmRegion* region;                 // buffer taken over by the cuMem layer, else null
  uint32_t mr_id;                        // export id of that region; irecv sets it to 0 when the region turns out not to be exportable
};

// entry points (tcp_endpoints.cc)
ncclResult_t tcp_listen(int dev, int ndev, int channel_id, bool offer_nvl, Handle* h, ListenComm** out);
ncclResult_t tcp_connect(int dev, int ndev, bool want_nvl, Handle* h, Comm** out);     // re-entrant, *out null until connected
ncclResult_t tcp_accept(ListenComm* lc, Comm** out);                                   // re-entrant
ncclResult_t tcp_isend(Comm* c, ConnManager* cm, void* data, int size, int tag, const TcpMem* mem, Request** out);
ncclResult_t tcp_irecv(Comm* c, ConnManager* cm, void* data, int size, int tag, TcpMem* mem, Request** out);
ncclResult_t tcp_test(Request* r, ConnManager* cm, int* done, int* sizes);
void tcp_close_listen(ListenComm* lc);
uint64_t tcp_direct_bytes();                        // payload bytes / messages stored straight into a same-host peer's buffer
uint64_t tcp_direct_msgs();
uint64_t random_u64();

// helpers shared with plugin.cc
int set_nonblock_nodelay(int fd);
int pick_listen_addr(sockaddr_in6* out);           // honours NCCL_SOCKET_IFNAME / NCCL_SOCKET_FAMILY
ncclResult_t comm_progress(Comm* c, ConnManager* cm);
int next_alive_dev(const Comm* c, int from);       // first device >= from (cyclic) whose data socket is open, -1 if none
uint64_t failover_count();                          // stripes moved to another device after a socket failure (process-wide)
void comm_close(Comm* c);

}  // namespace flnet
