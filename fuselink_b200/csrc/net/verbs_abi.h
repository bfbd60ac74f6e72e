// The part of the libibverbs ABI (libibverbs.so.1, rdma-core) that the verbs provider touches, declared here so
// that the plugin builds without rdma-core headers and loads without the library.  The reference vendors NCCL's
// copy of these declarations for the same reason (src/extern/ibvcore.h:19-1058, src/extern/ibvwrap.h:30-90).
//
// Field order and enum values were checked against that copy (context function table slots 11 / 25 / 26, work request,
// completion, queue-pair attribute, port and device attribute layouts).  Only the leading fields that are read or
// written are spelled out; the fast-path calls (poll, post send, post
// receive) are inline in the public header and go through the function table inside the context, whose slots
// are addressed by index below.
#pragma once
#include <stdint.h>

namespace flnet {
namespace verbs_abi {

union ibv_gid {
  uint8_t raw[16];
  struct { uint64_t subnet_prefix, interface_id; } global;
};

struct ibv_context;
struct ibv_pd { ibv_context* context; uint32_t handle; };
struct ibv_mr { ibv_context* context; ibv_pd* pd; void* addr; size_t length; uint32_t handle, lkey, rkey; };
struct ibv_cq { ibv_context* context; /* more follows */ };
struct ibv_qp {
  ibv_context* context;
  void* qp_context;
  ibv_pd* pd;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  void* srq;
  uint32_t handle;
  uint32_t qp_num;
  /* more follows */
};

struct ibv_sge { uint64_t addr; uint32_t length; uint32_t lkey; };

enum { IBV_WR_RDMA_WRITE = 0, IBV_WR_RDMA_WRITE_WITH_IMM = 1, IBV_WR_RDMA_READ = 4 };
enum { IBV_SEND_SIGNALED = 2, IBV_SEND_INLINE = 8 };

struct ibv_send_wr {
  uint64_t wr_id;
  ibv_send_wr* next;
  ibv_sge* sg_list;
  int num_sge;
  int opcode;
  unsigned int send_flags;
  uint32_t imm_data;              // big-endian on the wire; opaque to both ends here
  union {
    struct { uint64_t remote_addr; uint32_t rkey; } rdma;
    struct { uint64_t remote_addr, compare_add, swap; uint32_t rkey; } atomic;
    struct { void* ah; uint32_t remote_qpn, remote_qkey; } ud;
  } wr;
  union { struct { uint32_t remote_srqn; } xrc; } qp_type;
  union {
    struct { void* mw; uint32_t rkey; struct { void* mr; uint64_t addr, length; unsigned int mw_access_flags; } bind_info; } bind_mw;
    struct { void* hdr; uint16_t hdr_sz, mss; } tso;
  };
};
struct ibv_recv_wr { uint64_t wr_id; ibv_recv_wr* next; ibv_sge* sg_list; int num_sge; };

enum { IBV_WC_SUCCESS = 0, IBV_WC_RECV_RDMA_WITH_IMM = 129 };
struct ibv_wc {
  uint64_t wr_id;
  int status;
  int opcode;
  uint32_t vendor_err;
  uint32_t byte_len;
  uint32_t imm_data;
  uint32_t qp_num;
  uint32_t src_qp;
  unsigned int wc_flags;
  uint16_t pkey_index, slid;
  uint8_t sl, dlid_path_bits;
};

// Function table inside ibv_context: 32 slots; the three that the inline fast-path wrappers use.
enum { kOpsSlots = 32, kOpPollCq = 11, kOpPostSend = 25, kOpPostRecv = 26 };
struct ibv_context {
  void* device;
  void* ops[kOpsSlots];
  int cmd_fd;
  int async_fd;
  int num_comp_vectors;
  /* more follows */
};
typedef int (*poll_cq_fn)(ibv_cq*, int, ibv_wc*);
typedef int (*post_send_fn)(ibv_qp*, ibv_send_wr*, ibv_send_wr**);
typedef int (*post_recv_fn)(ibv_qp*, ibv_recv_wr*, ibv_recv_wr**);

struct ibv_qp_cap { uint32_t max_send_wr, max_recv_wr, max_send_sge, max_recv_sge, max_inline_data; };
enum { IBV_QPT_RC = 2 };
struct ibv_qp_init_attr {
  void* qp_context;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  void* srq;
  ibv_qp_cap cap;
  int qp_type;
  int sq_sig_all;
  void* reserved;                 // older vendor stacks read one more pointer here (XRC domain): keep it zero
};

struct ibv_global_route { ibv_gid dgid; uint32_t flow_label; uint8_t sgid_index, hop_limit, traffic_class; };
struct ibv_ah_attr { ibv_global_route grh; uint16_t dlid; uint8_t sl, src_path_bits, static_rate, is_global, port_num; };

enum { IBV_QPS_RESET = 0, IBV_QPS_INIT = 1, IBV_QPS_RTR = 2, IBV_QPS_RTS = 3 };
enum {
  IBV_QP_STATE = 1 << 0, IBV_QP_ACCESS_FLAGS = 1 << 3, IBV_QP_PKEY_INDEX = 1 << 4, IBV_QP_PORT = 1 << 5, IBV_QP_AV = 1 << 7,
  IBV_QP_PATH_MTU = 1 << 8, IBV_QP_TIMEOUT = 1 << 9, IBV_QP_RETRY_CNT = 1 << 10, IBV_QP_RNR_RETRY = 1 << 11, IBV_QP_RQ_PSN = 1 << 12,
  IBV_QP_MAX_QP_RD_ATOMIC = 1 << 13, IBV_QP_MIN_RNR_TIMER = 1 << 15, IBV_QP_SQ_PSN = 1 << 16, IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17,
  IBV_QP_DEST_QPN = 1 << 20
};
struct ibv_qp_attr {
  int qp_state, cur_qp_state, path_mtu, path_mig_state;
  uint32_t qkey, rq_psn, sq_psn, dest_qp_num;
  unsigned int qp_access_flags;
  ibv_qp_cap cap;
  ibv_ah_attr ah_attr, alt_ah_attr;
  uint16_t pkey_index, alt_pkey_index;
  uint8_t en_sqd_async_notify, sq_draining, max_rd_atomic, max_dest_rd_atomic, min_rnr_timer, port_num, timeout, retry_cnt, rnr_retry,
      alt_port_num, alt_timeout;
  uint32_t rate_limit;
};

enum { IBV_ACCESS_LOCAL_WRITE = 1, IBV_ACCESS_REMOTE_WRITE = 2, IBV_ACCESS_REMOTE_READ = 4, IBV_ACCESS_RELAXED_ORDERING = 1 << 20 };

enum { IBV_PORT_ACTIVE = 4, IBV_LINK_LAYER_INFINIBAND = 1, IBV_LINK_LAYER_ETHERNET = 2 };
struct ibv_port_attr {
  int state, max_mtu, active_mtu, gid_tbl_len;
  uint32_t port_cap_flags, max_msg_sz, bad_pkey_cntr, qkey_viol_cntr;
  uint16_t pkey_tbl_len, lid, sm_lid;
  uint8_t lmc, max_vl_num, sm_sl, subnet_timeout, init_type_reply, active_width, active_speed, phys_state, link_layer, flags;
  uint16_t port_cap_flags2;
  uint32_t active_speed_ex;
  uint8_t reserve[64];            // room for fields newer libraries append
};

struct ibv_device_attr {
  char fw_ver[64];
  uint64_t node_guid, sys_image_guid, max_mr_size, page_size_cap;
  uint32_t vendor_id, vendor_part_id, hw_ver;
  int max_qp, max_qp_wr;
  unsigned int device_cap_flags;
  int max_sge, max_sge_rd, max_cq, max_cqe, max_mr, max_pd, max_qp_rd_atom, max_ee_rd_atom, max_res_rd_atom, max_qp_init_rd_atom,
      max_ee_init_rd_atom, atomic_cap, max_ee, max_rdd, max_mw, max_raw_ipv6_qp, max_raw_ethy_qp, max_mcast_grp, max_mcast_qp_attach,
      max_total_mcast_qp_attach, max_ah, max_fmr, max_map_per_fmr, max_srq, max_srq_wr, max_srq_sge;
  uint16_t max_pkeys;
  uint8_t local_ca_ack_delay, phys_port_cnt;
  uint8_t reserve[64];
};

struct ibv_ece { uint32_t vendor_id, options, comp_mask; };

struct ibv_async_event {
  union { void* cq; void* qp; void* srq; void* wq; int port_num; } element;
  int event_type;
};

}  // namespace verbs_abi
}  // namespace flnet
