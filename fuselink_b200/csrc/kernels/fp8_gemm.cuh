// Block-scaled fp8 (e4m3) grouped GEMM and the quantisation kernels that feed it.
//
// Scaling scheme ("1 x 128"): activations carry one fp32 scale per row per 128 contraction elements,
// weights one fp32 scale per 128 x 128 block.  tcgen05.mma kind::f8f6f4 accumulates one 128-deep block in
// TMEM; the 8 promotion warps read that partial, multiply it by the two scales and add it to fp32 register
// accumulators while the tensor core already works on the next block (two TMEM partial buffers).  The final
// tile never exists in TMEM: the fused epilogue runs from registers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "grouped_gemm.cuh"

struct FlFp8GemmDesc {
  int num_groups, cap, N, K;       // M-grouped only: C_g[rows_g, N] = A_g[rows_g, K] * B_g^T
  const int* counts;
  const void* A;                    // [G*cap, K] e4m3, K-major
  const float* a_scale;             // [G*cap, K/128]
  const void* B;                    // K-major: [G, N, K] e4m3;  MN-major: [G, K, N] e4m3
  int b_mn_major;
  const float* b_scale;             // K-major: [G, N/128, K/128];  MN-major: [G, K/128, N/128]
  int epilogue;                     // FL_EPI_STORE, FL_EPI_SWIGLU, FL_EPI_SCATTER, FL_EPI_DSWIGLU
  void* C; long long ldc;           // bf16 output (STORE, SWIGLU act with ldc = N/2)
  void* gu; long long ldgu;         // SWIGLU: saved gate/up (bf16, may be null); DSWIGLU: input
  void* dgu;                        // DSWIGLU output
  const int* row_info;              // SCATTER
  FlPeerPtrs peers;
  int num_peers;                    // SCATTER: entries of `peers` in use
  long long peer_rows;              // SCATTER: rows of every receive buffer (0 = not checked)
  int zero_tail;
  int group_m;
  int max_ctas;
  int* status;
};

#ifdef __cplusplus
extern "C" {
#endif
int fl_fp8_grouped_gemm(const FlFp8GemmDesc* d, cudaStream_t stream);
const char* fl_fp8_last_error(void);
// x: [rows, K] bf16 -> q: [rows, K] e4m3, scale: [rows, K/128] fp32 (scale = amax / 448, 0 rows give scale 1)
// counts/cap (optional): x is a grouped buffer of `cap` rows per group and only the first roundup(counts[g], 128) rows of
// each group are quantised.
int fl_fp8_quantize_rows(const void* x, void* q, float* scale, long long rows, int K, const int* counts, int cap,
                         cudaStream_t stream);
// w: [G, R, C] bf16 -> q e4m3 same shape, scale: [G, R/128, C/128] fp32
int fl_fp8_quantize_blocks(const void* w, void* q, float* scale, int G, int R, int C, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
