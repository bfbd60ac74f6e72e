// Arguments of the fused embedding-bag + pooled-embedding all-to-all kernels (see embbag.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "grouped_gemm.cuh"  // FlPeerPtrs

struct FlEmbBagArgs {
  const float* weights;       // forward : [t_local, rows, dim] fp32, this rank's tables
  float* weights_rw;          // backward: same buffer, updated in place
  const long long* indices;   // [t_local, b_global, pooling] int64 row ids (fixed pooling factor)
  int t_local;                // tables owned by this rank
  int t_first;                // global index of this rank's first table
  int t_total;                // tables over all ranks (26 for the Criteo-shaped DLRM)
  long long rows;             // rows per table
  int dim;                    // embedding dimension, multiple of 128
  int pooling;                // indices per bag (<= 32)
  int b_global;               // samples in the global batch
  int b_local;                // samples per rank; sample b lives on rank b / b_local
  FlPeerPtrs out_peers;       // forward: every rank's pooled buffer [b_local, t_total, dim];
                              // backward: every rank's gradient buffer of the same shape
  float lr;                   // backward: SGD learning rate
  int* status;                // device int32[8]
  int hot_rows;               // backward: updates of rows [0, hot_rows) of a table are summed in shared memory per CTA and applied
                              // once at the end (tables whose ids are ordered by frequency, as Zipf-distributed ids are, have
                              // their hot rows there); 0 = the library's default (FUSELINK_EMBBAG_HOT_ROWS or 64), < 0 = off
};

#ifdef __cplusplus
extern "C" {
#endif
int fl_embbag_a2a_fwd(const FlEmbBagArgs* a, int num_ctas, cudaStream_t stream);
int fl_embbag_a2a_bwd_sgd(const FlEmbBagArgs* a, int num_ctas, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
