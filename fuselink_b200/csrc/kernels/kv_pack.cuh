// Prefill -> decode paged KV-cache hand-off: page gather through the block table, optional layout
// change, and the NVLink transfer, in one kernel (see kv_pack.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum FlKvLayout : int {
  FL_KV_BLHSD = 0,  // [block][layer][head][slot][dim]   (prefill-side pool, the order the reference's
                    //  element count blocks*layers*heads*block_size*head_dim implies)
  FL_KV_LBSHD = 1,  // [layer][block][slot][head][dim]   (decode-side pool, attention-kernel friendly)
};

struct FlKvSendArgs {
  const void* src_k; const void* src_v;   // local pools (bf16)
  void* dst_k; void* dst_v;               // pools on the decode GPU (peer-mapped addresses)
  int src_layout, dst_layout;
  int src_num_blocks, dst_num_blocks;     // pool sizes in pages (bounds checks)
  int layers, heads, block_size, head_dim;
  int layer_begin, layer_end;             // layers moved by this launch (per-layer pipelining)
  const int* src_block_table;             // [batch, max_blocks] page ids in the source pool
  const int* dst_block_table;             // [batch, max_blocks] page ids in the destination pool
  const int* num_blocks;                  // [batch] pages in use per request
  int batch, max_blocks;
  // control message folded into the transfer: copied by the last CTA before the flag is published
  const void* hdr_src; void* hdr_dst; int hdr_bytes;
  uint32_t* done_flag;                    // word in the decode GPU's signal pad; set to `seq` when done
  unsigned int seq;
  unsigned int* cta_counter;              // local scratch word, zero before first use (self-resetting)
  int* status;
};

#ifdef __cplusplus
extern "C" {
#endif
int fl_kv_pack_send(const FlKvSendArgs* a, int num_ctas, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
