// MoE dispatch / combine data movement.
//
// Dispatch is push-based: the rank that owns a token computes where the row goes and stores it into the
// expert owner's buffer over NVLink.  Row placement needs one system-scope atomic per (rank, expert) --
// a contiguous range is reserved on the owner -- not one per token.  Alongside each row the sender
// writes where the result must return to (rank, token*topk + k); the second expert GEMM's epilogue uses
// that to store its output row straight back into the home rank's combine slots, so neither direction
// has a stand-alone all-to-all.
//
// Reference parity: the reference's MoE experiment is an external Megatron-DeepSpeed checkout
// (.gitmodules:11-13): framework permute + NCCL all_to_all_single, twice per layer.
#include "moe_dispatch.cuh"
#include "../common/fl_ptx.cuh"

namespace fl {

__global__ void moe_count_kernel(const FlMoeDispatchArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.tokens * a.topk) return;
  const int e = a.topk_idx[i];
  if (e < 0 || e >= a.num_experts) {
    report(a.status, kBadIndex, 1100);
    a.pos[i] = -1;
    return;
  }
  a.pos[i] = atomicAdd(&a.local_count[e], 1);
}

// One contiguous range of rows per (rank, expert) on the expert's owner: one system-scope atomic each.
__device__ __forceinline__ void reserve_rows(const FlMoeDispatchArgs& a) {
  for (int e = threadIdx.x; e < a.num_experts; e += blockDim.x) {
    const int owner = e / a.experts_per_rank, le = e % a.experts_per_rank;
    int* cnt = reinterpret_cast<int*>(a.count_peers.p[owner]) + a.parity * a.experts_per_rank + le;
    const int n = __ldcg(a.local_count + e);      // other CTAs' atomics: read at L2
    a.base[e] = n > 0 ? atomicAdd_system(cnt, n) : 0;
    a.local_count[e] = 0;  // ready for the next step
  }
  // clear the other parity's counters of THIS rank; peers touch them only after the next inter-rank barrier
  for (int i = threadIdx.x; i < a.experts_per_rank; i += blockDim.x)
    reinterpret_cast<int*>(a.count_peers.p[a.rank])[(a.parity ^ 1) * a.experts_per_rank + i] = 0;
}

__global__ void moe_reserve_kernel(const FlMoeDispatchArgs a) { reserve_rows(a); }

// Counting and reservation in one launch: every CTA counts its share, takes a ticket, and the CTA that draws the last
// ticket -- by then every count is in -- reserves the rows and rearms the ticket.
__global__ void __launch_bounds__(256) moe_count_reserve_kernel(const FlMoeDispatchArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < a.tokens * a.topk) {
    const int e = a.topk_idx[i];
    if (e < 0 || e >= a.num_experts) {
      report(a.status, kBadIndex, 1100);
      a.pos[i] = -1;
    } else {
      a.pos[i] = atomicAdd(&a.local_count[e], 1);
    }
  }
  __shared__ int last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(a.ticket, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  reserve_rows(a);
  if (threadIdx.x == 0) *a.ticket = 0;
}

// one warp per token: the row is read once and stored to each of its top-k destinations
__global__ void __launch_bounds__(256) moe_scatter_kernel(const FlMoeDispatchArgs a) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int vecs = a.hidden / 8;  // 16-byte vectors per row
  for (int t = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); t < a.tokens; t += gridDim.x * warps_per_cta) {
    const uint4* src = reinterpret_cast<const uint4*>(a.x) + (long long)t * vecs;
    for (int k = 0; k < a.topk; ++k) {
      const int i = t * a.topk + k;
      const int e = a.topk_idx[i];
      if (e < 0 || e >= a.num_experts) continue;
      const int owner = e / a.experts_per_rank, le = e % a.experts_per_rank;
      int row;
      if (a.reuse_slots) {
        row = a.slot[i];
      } else {
        const int r = a.base[e] + a.pos[i];
        row = (r >= 0 && r < a.cap && a.pos[i] >= 0) ? le * a.cap + r : -1;
        if (lane == 0) a.slot[i] = row;
      }
      if (row < 0 || row >= a.experts_per_rank * a.cap) {
        if (lane == 0) report(a.status, kBadIndex, 1101);
        continue;
      }
      uint4* dst = reinterpret_cast<uint4*>(a.x_peers.p[owner]) + (long long)row * vecs;
      if (a.row_scale) {
        const float s = a.row_scale[i];
        for (int v = lane; v < vecs; v += 32) {
          uint4 d = ld_nc_v4(src + v);
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&d);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(h[j]);
            h[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
          }
          st_v4(dst + v, d);
        }
      } else {
        for (int v = lane; v < vecs; v += 32) st_v4(dst + v, ld_nc_v4(src + v));
      }
      if (!a.reuse_slots && lane == 0)
        reinterpret_cast<int*>(a.info_peers.p[owner])[row] = (a.rank << 28) | i;
    }
  }
}

__global__ void moe_zero_tail_kernel(__nv_bfloat16* buf, const int* counts, int cap, int width) {
  const int e = blockIdx.y;
  const int cnt = min(counts[e], cap);
  const int end = min((cnt + 127) / 128 * 128, cap);
  const int vecs = width / 8;
  const long long n = (long long)(end - cnt) * vecs;
  uint4* base = reinterpret_cast<uint4*>(buf + ((long long)e * cap + cnt) * width);
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    st_v4(base + i, z);
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* slots, const float* w,
                                                          __nv_bfloat16* out, int tokens, int topk, int hidden) {
  const int vecs = hidden / 8;
  const long long total = (long long)tokens * vecs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vecs), v = (int)(i % vecs);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < topk; ++k) {
      const float wk = w ? w[t * topk + k] : 1.f;
      uint4 d = ld_v4(reinterpret_cast<const uint4*>(slots) + ((long long)t * topk + k) * vecs + v);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += wk * f.x;
        acc[2 * j + 1] += wk * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    st_v4(reinterpret_cast<uint4*>(out) + i, o);
  }
}

// one warp per (token, k)
__global__ void __launch_bounds__(256) moe_combine_dw_kernel(const __nv_bfloat16* dout, const __nv_bfloat16* slots,
                                                             float* dw, int tokens, int topk, int hidden) {
  const int lane = threadIdx.x & 31;
  const int vecs = hidden / 8;
  const long long n = (long long)tokens * topk;
  for (long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n;
       i += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long t = i / topk;
    const uint4* a = reinterpret_cast<const uint4*>(dout) + t * vecs;
    const uint4* b = reinterpret_cast<const uint4*>(slots) + i * vecs;
    float acc = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      uint4 x = ld_v4(a + v), y = ld_v4(b + v);
      const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&x);
      const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(xh[j]), g = __bfloat1622float2(yh[j]);
        acc += f.x * g.x + f.y * g.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) dw[i] = acc;
  }
}

}  // namespace fl

extern "C" int fl_moe_dispatch(const FlMoeDispatchArgs* a, cudaStream_t stream) {
  if (a->hidden % 8) return -1;
  if (a->num_experts < 1 || a->num_experts > 1024) return -2;
  if (a->world < 1 || a->world > 8 || a->experts_per_rank * a->world != a->num_experts) return -3;
  if (a->rank < 0 || a->rank >= a->world || (long long)a->tokens * a->topk >= (1ll << 28)) return -4;
  if (a->cap <= 0 || a->topk < 1 || a->tokens < 0) return -5;
  const int n = a->tokens * a->topk;
  if (n == 0) return 0;
  if (!a->reuse_slots) {
    if (a->ticket != nullptr) {
      fl::moe_count_reserve_kernel<<<(n + 255) / 256, 256, 0, stream>>>(*a);
    } else {
      fl::moe_count_kernel<<<(n + 255) / 256, 256, 0, stream>>>(*a);
      fl::moe_reserve_kernel<<<1, 1024, 0, stream>>>(*a);
    }
  }
  int ctas = (a->tokens + 7) / 8;
  if (ctas > 148 * 8) ctas = 148 * 8;
  fl::moe_scatter_kernel<<<ctas, 256, 0, stream>>>(*a);
  return (int)cudaGetLastError();
}

extern "C" int fl_moe_dispatch_preload(void) {
  // makes the runtime load the three dispatch kernels on the current device now (module loading may allocate and
  // synchronise) instead of at their first launch
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, fl::moe_count_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, fl::moe_reserve_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, fl::moe_count_reserve_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, fl::moe_scatter_kernel);
  return (int)e;
}

extern "C" int fl_moe_zero_tail(void* buf, const int* counts, int experts_local, int cap, int width,
                                cudaStream_t stream) {
  if (width % 8 || experts_local < 1) return -1;
  dim3 grid(8, experts_local);
  fl::moe_zero_tail_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)buf, counts, cap, width);
  return (int)cudaGetLastError();
}

extern "C" int fl_moe_combine(const void* slots, const float* w, void* out, int tokens, int topk, int hidden,
                              cudaStream_t stream) {
  if (hidden % 8) return -1;
  if (tokens == 0) return 0;
  long long total = (long long)tokens * (hidden / 8);
  int ctas = (int)((total + 255) / 256);
  if (ctas > 148 * 16) ctas = 148 * 16;
  fl::moe_combine_kernel<<<ctas, 256, 0, stream>>>((const __nv_bfloat16*)slots, w, (__nv_bfloat16*)out, tokens, topk, hidden);
  return (int)cudaGetLastError();
}

extern "C" int fl_moe_combine_dw(const void* dout, const void* slots, float* dw, int tokens, int topk, int hidden,
                                 cudaStream_t stream) {
  if (hidden % 8) return -1;
  if (tokens == 0) return 0;
  long long n = (long long)tokens * topk;
  int ctas = (int)((n + 7) / 8);
  if (ctas > 148 * 8) ctas = 148 * 8;
  fl::moe_combine_dw_kernel<<<ctas, 256, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)slots, dw, tokens, topk, hidden);
  return (int)cudaGetLastError();
}
