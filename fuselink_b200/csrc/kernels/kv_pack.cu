// kv_pack_send: the KV hand-off of disaggregated serving as one kernel.
//
// Reference behaviour being replaced (experiments/serving/model.hh:253-337): after the whole prefill,
// five ncclSend calls in one group ship the first tokens, the entire K pool, the entire V pool, the
// block table and the block counts to rank + world/2; the decoder mirrors them with ncclRecv
// (model.hh:420-426).  Here only the pages a request owns are moved, they are re-laid-out on the fly for
// the decode side, the metadata rides along as a header, and completion is one release-store per launch,
// so layer l can be in flight while layer l+1 is still being computed.
#include "kv_pack.cuh"
#include "../common/fl_ptx.cuh"

namespace fl {

__device__ __forceinline__ long long page_base(int layout, int nblocks, int layers, long long page_elems, int blk,
                                               int layer) {
  return layout == FL_KV_BLHSD ? ((long long)blk * layers + layer) * page_elems
                               : ((long long)layer * nblocks + blk) * page_elems;
}

__global__ void __launch_bounds__(256) kv_pack_send_kernel(const FlKvSendArgs a) {
  const int H = a.heads, S = a.block_size, D = a.head_dim;
  const int vec_per_row = D / 8;                       // 16-byte vectors per (head, slot) row
  const int vec_per_page = H * S * vec_per_row;
  const long long page_elems = (long long)H * S * D;
  const int nl = a.layer_end - a.layer_begin;

  // total pages over the batch (batch is small: scan)
  __shared__ int s_total;
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int b = 0; b < a.batch; ++b) tot += min(a.num_blocks[b], a.max_blocks);
    s_total = tot;
  }
  __syncthreads();
  const long long units = (long long)s_total * nl * 2;

  for (long long u = blockIdx.x; u < units; u += gridDim.x) {
    const int kv = (int)(u & 1);
    long long r = u >> 1;
    const int layer = a.layer_begin + (int)(r % nl);
    int pg = (int)(r / nl);
    int b = 0;
    for (; b < a.batch; ++b) {
      const int nb = min(a.num_blocks[b], a.max_blocks);
      if (pg < nb) break;
      pg -= nb;
    }
    const int sblk = a.src_block_table[(long long)b * a.max_blocks + pg];
    const int dblk = a.dst_block_table[(long long)b * a.max_blocks + pg];
    if (sblk < 0 || sblk >= a.src_num_blocks || dblk < 0 || dblk >= a.dst_num_blocks) {
      if (threadIdx.x == 0) report(a.status, kBadIndex, 1000);
      continue;  // skip the access, keep going
    }
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(kv ? a.src_v : a.src_k) +
                               page_base(a.src_layout, a.src_num_blocks, a.layers, page_elems, sblk, layer);
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(kv ? a.dst_v : a.dst_k) +
                         page_base(a.dst_layout, a.dst_num_blocks, a.layers, page_elems, dblk, layer);
    if (a.src_layout == a.dst_layout) {
      for (int v = threadIdx.x; v < vec_per_page; v += blockDim.x)
        st_v4(reinterpret_cast<uint4*>(dst) + v, ld_nc_v4(reinterpret_cast<const uint4*>(src) + v));
    } else {
      // page-internal order differs: [head][slot][dim] <-> [slot][head][dim]; iterate in destination order
      const bool dst_shd = a.dst_layout == FL_KV_LBSHD;
      for (int v = threadIdx.x; v < vec_per_page; v += blockDim.x) {
        const int d8 = v % vec_per_row;
        const int rw = v / vec_per_row;
        int h, s;
        if (dst_shd) { s = rw / H; h = rw % H; } else { h = rw / S; s = rw % S; }
        const int src_v = dst_shd ? ((h * S + s) * vec_per_row + d8) : ((s * H + h) * vec_per_row + d8);
        st_v4(reinterpret_cast<uint4*>(dst) + v, ld_nc_v4(reinterpret_cast<const uint4*>(src) + src_v));
      }
    }
  }

  // completion: the last CTA to finish copies the header and publishes the flag
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    fence_sys();
    const unsigned int prev = atomicAdd(a.cta_counter, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (a.hdr_bytes > 0 && a.hdr_src && a.hdr_dst) {
      for (int i = threadIdx.x; i < a.hdr_bytes; i += blockDim.x)
        reinterpret_cast<uint8_t*>(a.hdr_dst)[i] = reinterpret_cast<const uint8_t*>(a.hdr_src)[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *a.cta_counter = 0;
      fence_sys();
      if (a.done_flag) st_release_sys(a.done_flag, a.seq);
    }
  }
}

}  // namespace fl

extern "C" int fl_kv_pack_send(const FlKvSendArgs* a, int num_ctas, cudaStream_t stream) {
  if (a->head_dim % 8) return -1;
  if (a->layer_begin < 0 || a->layer_end > a->layers || a->layer_begin >= a->layer_end) return -2;
  if (a->batch < 1 || a->max_blocks < 1) return -3;
  if (!a->cta_counter) return -4;
  if (num_ctas <= 0) num_ctas = 148 * 4;
  fl::kv_pack_send_kernel<<<num_ctas, 256, 0, stream>>>(*a);
  return (int)cudaGetLastError();
}
