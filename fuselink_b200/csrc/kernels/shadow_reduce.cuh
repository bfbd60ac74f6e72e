// Second half of the sum of replicated ("shadow") experts' weight gradients over the ranks.
//
// The first half is done by the weight-gradient GEMM itself (FlGemmDesc::push_world in grouped_gemm.cuh): every rank
// stores each block of rows of its partial dW_g straight into the staging buffer of the one rank that sums that block,
// over NVLink, from the GEMM's epilogue.  Once every rank has signalled that its GEMMs are complete, this kernel runs on
// every rank: for the blocks it is responsible for it adds up the world partial rows in fp32, applies the SGD update to
// its own copy of the weights (all copies are equal before the step), and stores the new bf16 rows into every rank's
// copy -- or, with lr == 0, stores the summed gradient rows into every rank's gradient buffer.  Each row of each copy is
// written by exactly one rank, so the copies stay bit-identical without an all-reduce: a rank sends (world - 1) / world of
// the gradient in the GEMM and the same amount of new weights here, and the first of the two is hidden behind the MMAs.
//
// The reference has no counterpart: it leaves expert exchange inside one box to NCCL (README.md, "experiments/ep").
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "grouped_gemm.cuh"

typedef struct {
  const void* part;        // this rank's staging: [groups][world][M / world][N] bf16, filled by the ranks' GEMMs
  const void* w;           // lr != 0: this rank's copy of the replicated weights, group g at w + g * group_stride elements
  FlPeerPtrs out_peers;    // every rank's destination (weights when lr != 0, summed gradients when lr == 0), same layout as w
  int groups, world, rank;
  int M, N;                // rows and columns of one group's matrix; N a multiple of 8
  int block_log2;          // rows are dealt out to the ranks in blocks of 2^block_log2 (the GEMM's push_block_log2)
  long long group_stride;  // elements between groups in w and in every destination
  float lr;
  int max_ctas;            // 0 => two CTAs per SM
} FlShadowUpdateArgs;

#ifdef __cplusplus
extern "C" {
#endif
// Returns 0, a negative value for rejected arguments, or a positive cudaError.
int fl_shadow_update(const FlShadowUpdateArgs* args, cudaStream_t stream);
const char* fl_shadow_update_error(void);
#ifdef __cplusplus
}
#endif
