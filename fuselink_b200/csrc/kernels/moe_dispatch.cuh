// MoE expert-parallel token movement: top-k permute/scatter fused with the dispatch all-to-all
// (rows are stored straight into the owning expert's buffer on the peer GPU), tail zeroing, and the
// home-side weighted combine.  See moe_dispatch.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "grouped_gemm.cuh"  // FlPeerPtrs

struct FlMoeDispatchArgs {
  const void* x;              // [tokens, hidden] bf16, this rank's tokens
  const int* topk_idx;        // [tokens, topk] global expert ids
  const float* row_scale;     // optional [tokens, topk]: row is multiplied by it (backward: gate weight)
  int tokens, topk, hidden;
  int num_experts;            // global
  int experts_per_rank;
  int cap;                    // rows reserved per expert in the destination buffers
  int rank, world;
  int* local_count;           // [num_experts] scratch, zero before the first call (the kernels leave it zero)
  int* ticket;                // optional: one more zeroed int of scratch.  With it counting and reservation are ONE launch
                              // (the last CTA to finish counting reserves the rows); without it they are two
  int* base;                  // [num_experts] scratch: first row this rank owns in each expert buffer
  int* pos;                   // [tokens, topk] scratch: position inside (rank, expert)
  int* slot;                  // [tokens, topk] out (forward) / in (backward): row inside the owner's buffer
  FlPeerPtrs count_peers;     // every rank's int32 counts[2][experts_per_rank] (double-buffered by step parity)
  int parity;
  FlPeerPtrs x_peers;         // every rank's expert input buffer [experts_per_rank * cap, hidden] bf16
  FlPeerPtrs info_peers;      // every rank's int32 row_info[experts_per_rank * cap]
  int reuse_slots;            // 1: skip counting/reservation, place rows at `slot` (backward dispatch)
  int* status;
};

#ifdef __cplusplus
extern "C" {
#endif
// forward: count + reserve (one system-scope atomic per expert; one launch with `ticket`, else two) -> scatter.
// backward: scatter only.
int fl_moe_dispatch(const FlMoeDispatchArgs* a, cudaStream_t stream);
// load the dispatch kernels on the current device now rather than at their first launch; returns a cudaError
int fl_moe_dispatch_preload(void);
// zero rows [counts[e], roundup(counts[e], 128)) of a grouped [E_local * cap, width] bf16 buffer
int fl_moe_zero_tail(void* buf, const int* counts, int experts_local, int cap, int width, cudaStream_t stream);
// out[t] = sum_k w[t,k] * slots[t*topk + k]   (w == nullptr => plain sum)
int fl_moe_combine(const void* slots, const float* w, void* out, int tokens, int topk, int hidden, cudaStream_t stream);
// dw[t,k] = <dout[t], slots[t*topk + k]>
int fl_moe_combine_dw(const void* dout, const void* slots, float* dw, int tokens, int topk, int hidden,
                      cudaStream_t stream);
#ifdef __cplusplus
}
#endif
