// See shadow_reduce.cuh.
#include "shadow_reduce.cuh"
#include "../common/fl_ptx.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace {

thread_local char g_err[200] = "";

struct Params {
  const uint4* part;
  const uint4* w;
  FlPeerPtrs out;
  int groups, world, rank, M, N, shift;
  long long gs;
  float lr;
};

__device__ __forceinline__ void add8(float* acc, const uint4& q) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(u[i] << 16);
    acc[2 * i + 1] += __uint_as_float(u[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// One thread per 8 consecutive columns (16 bytes) of one row this rank sums; a warp covers 512 contiguous bytes of the
// row in every source and in every destination.
template <int WORLD>
__global__ void __launch_bounds__(512) shadow_update_kernel(const Params p) {
  const int world = WORLD > 0 ? WORLD : p.world;
  const long long vec_per_row = p.N / 8;
  const long long rows_own = p.M / world;
  const long long per_group = rows_own * vec_per_row;
  const long long total = per_group * p.groups;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int mask = (1 << p.shift) - 1;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += stride) {
    const int g = (int)(v / per_group);
    const long long rem = v - g * per_group;
    const long long lrow = rem / vec_per_row;
    const long long c8 = rem - lrow * vec_per_row;
    uint4 q[WORLD > 0 ? WORLD : 8];
#pragma unroll
    for (int s = 0; s < (WORLD > 0 ? WORLD : 8); ++s)
      if (s < world) q[s] = __ldg(p.part + (((long long)g * world + s) * rows_own + lrow) * vec_per_row + c8);
    const long long row = ((((lrow >> p.shift) * world + p.rank)) << p.shift) + (lrow & mask);
    const long long off = (g * p.gs + row * p.N) / 8 + c8;      // in 16-byte units; gs and N are multiples of 8
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < (WORLD > 0 ? WORLD : 8); ++s)
      if (s < world) add8(acc, q[s]);
    if (p.lr != 0.f) {
      float wv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8(wv, p.w[off]);      // a plain load: this thread rewrites the same 16 bytes of the own copy below
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(-p.lr, acc[i], wv[i]);
    }
    uint4 o;
    o.x = pack2(acc[0], acc[1]); o.y = pack2(acc[2], acc[3]); o.z = pack2(acc[4], acc[5]); o.w = pack2(acc[6], acc[7]);
#pragma unroll
    for (int d = 0; d < (WORLD > 0 ? WORLD : 8); ++d) {
      const int dd = (d + p.rank) % world;                       // every rank starts with a different destination
      if (d < world) reinterpret_cast<uint4*>(p.out.p[dd])[off] = o;
    }
  }
  fl::fence_sys();   // the stores to the peers are visible before this kernel's completion is signalled to them
}

}  // namespace

extern "C" const char* fl_shadow_update_error(void) { return g_err; }

extern "C" int fl_shadow_update(const FlShadowUpdateArgs* a, cudaStream_t stream) {
  g_err[0] = 0;
  auto bad = [](const char* why) {
    snprintf(g_err, sizeof g_err, "%s", why);
    return -1;
  };
  if (!a) return bad("null argument block");
  if (a->groups < 1 || a->world < 1 || a->world > FL_MAX_PEERS || a->rank < 0 || a->rank >= a->world) return bad("groups / world / rank out of range");
  if (a->N <= 0 || a->N % 8 || a->group_stride % 8) return bad("N and group_stride must be multiples of 8 elements (16 bytes)");
  if (a->block_log2 < 0 || a->block_log2 > 16 || a->M <= 0 || a->M % (a->world << a->block_log2)) return bad("M must be a whole number of blocks per rank");
  if (!a->part || (a->lr != 0.f && !a->w)) return bad("null staging or weight pointer");
  if ((reinterpret_cast<uintptr_t>(a->part) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return bad("pointers must be 16-byte aligned");
  for (int i = 0; i < a->world; ++i)
    if (!a->out_peers.p[i] || (reinterpret_cast<uintptr_t>(a->out_peers.p[i]) & 15)) return bad("a destination is null or not 16-byte aligned");
  Params p;
  p.part = reinterpret_cast<const uint4*>(a->part); p.w = reinterpret_cast<const uint4*>(a->w); p.out = a->out_peers;
  p.groups = a->groups; p.world = a->world; p.rank = a->rank; p.M = a->M; p.N = a->N; p.shift = a->block_log2;
  p.gs = a->group_stride; p.lr = a->lr;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a->groups * (a->M / a->world) * (a->N / 8);
  long long ctas = (total + 511) / 512;
  const long long cap = a->max_ctas > 0 ? a->max_ctas : 2LL * sms;
  if (ctas > cap) ctas = cap;
  switch (a->world) {
    case 2: shadow_update_kernel<2><<<(int)ctas, 512, 0, stream>>>(p); break;
    case 4: shadow_update_kernel<4><<<(int)ctas, 512, 0, stream>>>(p); break;
    case 8: shadow_update_kernel<8><<<(int)ctas, 512, 0, stream>>>(p); break;
    default: shadow_update_kernel<0><<<(int)ctas, 512, 0, stream>>>(p); break;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) snprintf(g_err, sizeof g_err, "launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}
