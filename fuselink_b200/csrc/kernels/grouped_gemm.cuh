// Host-visible description of one grouped-GEMM launch (tcgen05 / TMEM / TMA, sm_100a).
//
// The kernel computes, for every group g (an expert of a MoE layer):
//   group_mode 0 ("M-grouped", forward / dgrad):   C_g[rows_g, N] = A_g[rows_g, K] * B_g[N, K]^T
//        A_g is rows [g*cap, g*cap + counts[g]) of one token buffer, B_g is expert g's weight.
//   group_mode 1 ("K-grouped", wgrad):             C_g[M, N]      = A_g[rows_g, M]^T * B_g[rows_g, N]
//        the contraction runs over the rows (tokens) that were routed to expert g.
// Operands may be K-major (contraction dimension contiguous) or MN-major (row/col dimension
// contiguous); the MN-major forms are what the backward pass needs so no transposed copy of a weight
// or an activation is ever materialised.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define FL_MAX_PEERS 8
#define FL_GEMM_MAX_GROUPS 64

struct FlPeerPtrs {
  void* p[FL_MAX_PEERS];
};

enum FlGemmEpilogue : int {
  FL_EPI_STORE = 0,    // C (bf16) row-major, leading dimension ldc; rows past counts[g] optionally zeroed
  FL_EPI_SWIGLU = 1,   // B rows interleaved [128 gate | 128 up] per 256; writes act = silu(gate)*up and gate/up
  FL_EPI_SCATTER = 2,  // each output row goes to peers.p[rank(row)] + slot(row)*ldc   (combine / dX return)
  FL_EPI_DSWIGLU = 3,  // accumulator is dAct; reads saved gate/up, writes dgate/dup in the interleaved layout
  FL_EPI_WGRAD = 4,    // K-grouped: store dW_g (bf16), or apply W_g -= lr * dW_g in place when sgd_lr != 0; with push_world
                       // the rows of dW_g go to the ranks that sum them (see push_world below)
};

struct FlGemmDesc {
  // problem
  int group_mode;   // 0 M-grouped, 1 K-grouped
  int num_groups;   // <= FL_GEMM_MAX_GROUPS
  int cap;          // rows reserved per group in the grouped buffers
  int M, N, K;      // M-grouped: N,K dense (M unused); K-grouped: M,N dense (K unused)
  const int* counts;  // device int32[num_groups]; nullptr => every group has `cap` rows
  int elem_bytes;   // 2 = bf16 operands, 1 = fp8 e4m3 operands (K-major only)
  // operands: 3-D views {inner, outer, group}; ld* in elements, gs* = elements between groups
  const void* A; int a_mn_major; long long lda; long long gsa;
  const void* B; int b_mn_major; long long ldb; long long gsb;
  // epilogue
  int epilogue;
  void* C; long long ldc; long long gsc;          // STORE / WGRAD / SWIGLU(act, ld = N/2)
  void* gu; long long ldgu;                       // SWIGLU: saved gate/up (may be null); DSWIGLU: input
  void* dgu;                                      // DSWIGLU output (same ld as gu)
  const int* row_info;                            // SCATTER: per grouped row  (rank << 28) | slot
  FlPeerPtrs peers;                               // SCATTER: base of each rank's receive buffer
  int num_peers;                                  // SCATTER: entries of `peers` in use; a row naming another rank is skipped
  long long peer_rows;                            // SCATTER: rows of every receive buffer (0 = not checked); a slot beyond it is skipped
  float sgd_lr;                                   // WGRAD: 0 => store dW
  // WGRAD, first half of a sum over ranks done by the GEMM itself: with push_world > 0 the rows of dW_g are dealt out in
  // blocks of 2^push_block_log2 rows, block b to rank b % push_world, and stored (bf16) into that rank's buffer
  // peers.p[b % push_world], laid out [num_groups][push_world sources][M / push_world rows][ldc], at source push_rank and
  // row (b / push_world) * 2^push_block_log2 + (row inside the block).  M must be a multiple of push_world blocks; sgd_lr
  // must be 0 and C is not written.  fl_shadow_update (shadow_reduce.cuh) sums the sources and applies the result.
  int push_world, push_rank, push_block_log2;
  int zero_tail;                                  // STORE/SWIGLU/DSWIGLU: write zeros to rows in [count, roundup(count,128))
  // fp8 block scaling (elem_bytes == 1): fp32 scales, A: [rows, K/128] per-row-per-128, B: [N/128, K/128]
  const float* a_scale; long long lda_scale;
  const float* b_scale; long long ldb_scale; long long gsb_scale;
  // scheduling
  int group_m;      // rasterisation: m-tiles per super-column (default 16)
  int max_ctas;     // 0 => one CTA per SM
  int* status;      // device int32[8], zero on success
};

#ifdef __cplusplus
extern "C" {
#endif
// Returns 0 on success, a negative value for a rejected description, a positive cudaError otherwise.
int fl_grouped_gemm(const FlGemmDesc* desc, cudaStream_t stream);
const char* fl_gemm_last_error(void);
// 0: one CTA per 128 x 256 tile; 1: CTA pairs on 256 x 256 tiles (tcgen05 cta_group::2, two accumulators); 2: CTA pairs on
// 256 x 512 tiles (one accumulator handed back in halves); 3: chosen per launch from the shape and the epilogue.
// Default: FUSELINK_GEMM_PAIR or 3.
void fl_gemm_set_variant(int pair);
int fl_gemm_get_variant(void);
#ifdef __cplusplus
}
#endif
