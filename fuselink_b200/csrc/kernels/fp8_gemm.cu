// Block-scaled fp8 grouped GEMM (see fp8_gemm.cuh for the scheme).
//
//   warp 0      : TMA producer (e4m3 tiles, 128-byte swizzle, never multicast)
//   warp 1      : MMA issuer   (tcgen05.mma kind::f8f6f4; one 128-deep block per TMEM partial buffer)
//   warps 2..9  : promotion + epilogue (tcgen05.ld partial -> scale -> fp32 registers -> fused epilogue)
//
// Reference parity: none in the reference (it has no kernels); this is the fp8 arm of the MoE expert GEMMs.
#include "fp8_gemm.cuh"
#include "../common/fl_ptx.cuh"
#include <cuda.h>
#include <cuda_fp8.h>
#include <stdio.h>
#include <string.h>

namespace fl8 {
using namespace fl;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BKB = 128;                      // bytes (= e4m3 elements) of contraction per stage = one scale block
constexpr int STAGES = 4;
constexpr int A_STAGE = BM * BKB;             // 16 KiB
constexpr int B_STAGE = BN * BKB;             // 32 KiB
constexpr int STAGE = A_STAGE + B_STAGE;
constexpr int NUM_THREADS = 320;
constexpr int TMEM_COLS = 512;                // two partial buffers of 256 columns
constexpr int SMEM_BYTES = STAGES * STAGE + 1024 + 1024;

struct KParams {
  int num_groups, cap, N, K;
  const int* counts;
  const float* a_scale;
  const float* b_scale;
  int b_mn;
  int epilogue;
  __nv_bfloat16* C; long long ldc;
  __nv_bfloat16* gu; long long ldgu;
  __nv_bfloat16* dgu;
  const int* row_info;
  FlPeerPtrs peers;
  int num_peers; long long peer_rows;
  int zero_tail;
  int group_m;
  int* status;
};

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t pfull[2];
  uint64_t pempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int counts[FL_GEMM_MAX_GROUPS];
};

struct Tile {
  int g, m0, n0, rows, cnt;
};

__device__ __forceinline__ bool map_tile(const KParams& p, const int* counts, int id, Tile& t) {
  const int NT = (p.N + BN - 1) / BN;
  int acc = 0;
  for (int g = 0; g < p.num_groups; ++g) {
    const int cnt = counts[g];
    const int mt = (cnt + BM - 1) / BM;
    const int tiles = mt * NT;
    if (id < acc + tiles) {
      const int l = id - acc;
      const int per_sg = p.group_m * NT;
      const int sg = l / per_sg;
      const int first_m = sg * p.group_m;
      const int gsz = min(p.group_m, mt - first_m);
      const int r = l - sg * per_sg;
      t.g = g; t.m0 = (first_m + r % gsz) * BM; t.n0 = (r / gsz) * BN;
      t.rows = min(BM, cnt - t.m0);
      t.cnt = cnt;
      return true;
    }
    acc += tiles;
  }
  return false;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void store32_bf16(__nv_bfloat16* dst, const float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 o;
    o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
    o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
    o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
    o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
    st_v4(dst + 8 * i, o);
  }
}
// 16-column variants: the epilogues that need the saved gate/up beside the 128 accumulators of a thread work on 16
// columns at a time, which keeps their temporaries (and with them the register spills) small
__device__ __forceinline__ void store16_bf16(__nv_bfloat16* dst, const float* v) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 o;
    o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
    o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
    o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
    o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
    st_v4(dst + 8 * i, o);
  }
}
__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* src, float* v) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 o = ld_v4(src + 8 * i);
    const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
      v[8 * i + 2 * j] = __bfloat162float(h.x);
      v[8 * i + 2 * j + 1] = __bfloat162float(h.y);
    }
  }
}
__device__ __forceinline__ void load32_bf16(const __nv_bfloat16* src, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 o = ld_v4(src + 8 * i);
    const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
      v[8 * i + 2 * j] = __bfloat162float(h.x);
      v[8 * i + 2 * j + 1] = __bfloat162float(h.y);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// quantisation
// ------------------------------------------------------------------------------------------------
// one warp per (row, 128-element block): 4 elements per lane
// With `counts` (grouped buffer, `cap` rows per group) only rows below roundup(counts[g], 128) are processed.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const __nv_bfloat16* x, __nv_fp8_storage_t* q, float* scale,
                                                            long long rows, int K, const int* counts, int cap) {
  const int lane = threadIdx.x & 31;
  const int kblocks = K / 128;
  const long long total = rows * kblocks;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
       w += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long row = w / kblocks;
    const int kb = (int)(w - row * kblocks);
    if (counts != nullptr) {
      const int g = (int)(row / cap);
      if ((int)(row - (long long)g * cap) >= (min(counts[g], cap) + 127) / 128 * 128) continue;
    }
    const __nv_bfloat16* src = x + row * K + kb * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float v[4] = {__bfloat162float(h0.x), __bfloat162float(h0.y), __bfloat162float(h1.x), __bfloat162float(h1.y)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / s;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      packed |= (uint32_t)__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * i);
    *reinterpret_cast<uint32_t*>(q + row * K + kb * 128 + lane * 4) = packed;
    if (lane == 0) scale[w] = s;
  }
}

// one CTA (256 threads) per 128 x 128 block of a [G, R, C] weight
__global__ void __launch_bounds__(256) quantize_blocks_kernel(const __nv_bfloat16* w, __nv_fp8_storage_t* q, float* scale,
                                                              int R, int C) {
  const int cb = blockIdx.x, rb = blockIdx.y, g = blockIdx.z;
  const long long base = (long long)g * R * C;
  __shared__ float red[8];
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 32; i += 256) {      // 32 x (4 elements) per row
    const int r = i >> 5, c4 = i & 31;
    const uint2 raw = *reinterpret_cast<const uint2*>(w + base + (long long)(rb * 128 + r) * C + cb * 128 + c4 * 4);
    const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(__bfloat162float(h0.x)), fabsf(__bfloat162float(h0.y))),
                             fmaxf(fabsf(__bfloat162float(h1.x)), fabsf(__bfloat162float(h1.y)))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / s;
  if (threadIdx.x == 0) scale[((long long)g * (R / 128) + rb) * (C / 128) + cb] = s;
  for (int i = threadIdx.x; i < 128 * 32; i += 256) {
    const int r = i >> 5, c4 = i & 31;
    const long long off = base + (long long)(rb * 128 + r) * C + cb * 128 + c4 * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(w + off);
    const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float v[4] = {__bfloat162float(h0.x), __bfloat162float(h0.y), __bfloat162float(h1.x), __bfloat162float(h1.y)};
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      packed |= (uint32_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
    *reinterpret_cast<uint32_t*>(q + off) = packed;
  }
}

// ------------------------------------------------------------------------------------------------
// GEMM
// ------------------------------------------------------------------------------------------------
// Columns a promotion thread owns inside the 256-wide tile: chunks 0,1 in the first 128-column block, chunks 2,3 in
// the second, 64 columns per warp-half in each.  With the gate|up interleaved weight this gives every thread the gate
// and the up value of the same 64 activation columns, and every chunk pair exactly one weight scale block.
__device__ __forceinline__ int chunk_col(int half, int c) { return (c < 2 ? 0 : 128) + 64 * half + 32 * (c & 1); }

__global__ void __launch_bounds__(NUM_THREADS, 1)
fp8_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int KB = p.K / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->pfull[b], 1);
      mbar_init(&sh->pempty[b], 8);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  for (int g = threadIdx.x; g < p.num_groups; g += NUM_THREADS)
    sh->counts[g] = p.counts ? min(p.counts[g], p.cap) : p.cap;
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  const int* counts = sh->counts;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      Tile t;
      for (int id = blockIdx.x; ok && map_tile(p, counts, id, t); id += gridDim.x) {
        for (int kb = 0; kb < KB && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&sh->empty[s], ph ^ 1, abort_flag, p.status, kTimeoutMbarEmpty, 2100 + s);
          if (!ok) break;
          uint8_t* a_dst = smem + s * STAGE;
          uint8_t* b_dst = a_dst + A_STAGE;
          mbar_arrive_expect_tx(&sh->full[s], STAGE);
          const int k0 = kb * 128;
          tma_load_3d(a_dst, &tmA, &sh->full[s], k0, t.m0, t.g);
          if (!p.b_mn) {
            tma_load_3d(b_dst, &tmB, &sh->full[s], k0, t.n0, t.g);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tma_load_3d(b_dst + j * (128 * BKB), &tmB, &sh->full[s], t.n0 + 128 * j, k0, t.g);
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(0, 0, 0u, p.b_mn ? 1u : 0u, BM, BN);   // e4m3 x e4m3 -> fp32
      uint32_t it = 0;
      bool ok = true;
      Tile t;
      for (int id = blockIdx.x; ok && map_tile(p, counts, id, t); id += gridDim.x) {
        for (int kb = 0; kb < KB && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const int b = it & 1;
          const uint32_t bph = (it >> 1) & 1;
          ok = mbar_wait(&sh->pempty[b], bph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, 2200 + b);
          if (!ok) break;
          ok = mbar_wait(&sh->full[s], ph, abort_flag, p.status, kTimeoutMbarFull, 2300 + s);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * STAGE);
          const uint32_t b_base = a_base + A_STAGE;
          const uint32_t d_tmem = tmem_base + b * BN;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {   // 4 x (K = 32) per 128-deep block
            const uint64_t da = make_smem_desc(a_base + kk * 32, 16, 1024);
            const uint64_t db = p.b_mn ? make_smem_desc(b_base + kk * 4096, 128 * BKB, 1024)
                                       : make_smem_desc(b_base + kk * 32, 16, 1024);
            umma_f8(d_tmem, da, db, idesc, kk != 0 ? 1u : 0u);
          }
          umma_commit(&sh->empty[s]);
          umma_commit(&sh->pfull[b]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t it = 0;
    bool ok = true;
    Tile t;
    for (int id = blockIdx.x; ok && map_tile(p, counts, id, t); id += gridDim.x) {
      const int r_in_tile = q * 32 + lane;
      const int row = t.m0 + r_in_tile;
      const long long grow = (long long)t.g * p.cap + row;
      const bool valid = r_in_tile < t.rows;
      const int NB = p.N / 128;
      const int nb0 = t.n0 / 128;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      const float* sa_row = p.a_scale + grow * KB;
      for (int kb = 0; kb < KB && ok; ++kb, ++it) {
        const int b = it & 1;
        const uint32_t bph = (it >> 1) & 1;
        // scales of this block (loaded before the wait so their latency overlaps it)
        const float sa = valid ? sa_row[kb] : 0.f;
        float sb0, sb1;
        if (!p.b_mn) {
          sb0 = p.b_scale[((long long)t.g * NB + nb0) * KB + kb];
          sb1 = p.b_scale[((long long)t.g * NB + nb0 + 1) * KB + kb];
        } else {
          sb0 = p.b_scale[((long long)t.g * KB + kb) * NB + nb0];
          sb1 = p.b_scale[((long long)t.g * KB + kb) * NB + nb0 + 1];
        }
        const float s0 = sa * sb0, s1 = sa * sb1;
        ok = mbar_wait(&sh->pfull[b], bph, abort_flag, p.status, kTimeoutTmemFull, 2400 + b);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + b * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + chunk_col(half, c), r);
          tmem_ld_wait();
          const float sc = c < 2 ? s0 : s1;
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), sc, acc[c * 32 + i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->pempty[b]);
      }
      if (!ok) break;
      // ---- fused epilogue from registers ----------------------------------------------------------
      const bool zero_row = !valid && p.zero_tail && row < min(p.cap, (t.cnt + 127) / 128 * 128);
      if (p.epilogue == FL_EPI_STORE || p.epilogue == FL_EPI_SCATTER) {
        __nv_bfloat16* dst = nullptr;
        if (p.epilogue == FL_EPI_STORE) {
          dst = p.C + grow * p.ldc;
        } else if (valid) {
          const int info = p.row_info[grow];
          const int rk = (info >> 28) & 0xF;
          const long long slot = info & 0x0FFFFFFF;
          if (rk < p.num_peers && (p.peer_rows <= 0 || slot < p.peer_rows))
            dst = reinterpret_cast<__nv_bfloat16*>(p.peers.p[rk]) + slot * p.ldc;
          else
            report(p.status, kBadIndex, 2500);   // names no rank / no slot of the receive buffer: not stored
        }
        if ((valid && dst != nullptr) || (zero_row && p.epilogue == FL_EPI_STORE)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = valid ? acc[c * 32 + i] : 0.f;
            store32_bf16(dst + t.n0 + chunk_col(half, c), v);
          }
        }
      } else if (p.epilogue == FL_EPI_SWIGLU) {
        if (valid || zero_row) {
          __nv_bfloat16* act = p.C + grow * p.ldc + t.n0 / 2 + 64 * half;
          __nv_bfloat16* gu = p.gu ? p.gu + grow * p.ldgu + t.n0 + 64 * half : nullptr;
#pragma unroll
          for (int c = 0; c < 4; ++c) {                        // 16 columns at a time: gate in acc[0, 64), up in acc[64, 128)
            float g[16], u[16], a[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              g[i] = valid ? acc[c * 16 + i] : 0.f;
              u[i] = valid ? acc[64 + c * 16 + i] : 0.f;
              a[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
            }
            store16_bf16(act + 16 * c, a);
            if (gu) {
              store16_bf16(gu + 16 * c, g);
              store16_bf16(gu + 128 + 16 * c, u);
            }
          }
        }
      } else {  // FL_EPI_DSWIGLU: acc = dAct over 256 activation columns
        if (valid || zero_row) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {                        // 16 columns at a time: acc[16 c, 16 c + 16)
            const int a_col = t.n0 + chunk_col(half, c >> 1) + 16 * (c & 1);
            const long long gcol = (long long)(a_col >> 7) * 256 + (a_col & 127);
            float dg[16], du[16];
            if (valid) {
              float g[16], u[16];
              load16_bf16(p.gu + grow * p.ldgu + gcol, g);
              load16_bf16(p.gu + grow * p.ldgu + gcol + 128, u);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float da = acc[c * 16 + i];
                const float sg = 1.f / (1.f + __expf(-g[i]));
                dg[i] = da * u[i] * (sg * (1.f + g[i] * (1.f - sg)));
                du[i] = da * g[i] * sg;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) dg[i] = du[i] = 0.f;
            }
            store16_bf16(p.dgu + grow * p.ldgu + gcol, dg);
            store16_bf16(p.dgu + grow * p.ldgu + gcol + 128, du);
          }
        }
      }
    }
    if (p.epilogue == FL_EPI_SCATTER) fence_sys();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static thread_local char g_err[256] = "";

static int make_map(CUtensorMap* m, const void* base, long long inner, long long outer, long long groups, int box_inner,
                    int box_outer) {
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      enc = reinterpret_cast<EncodeTiledFn>(sym);
  }
  if (!enc) { snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not available"); return -10; }
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)groups};
  cuuint64_t strides[2] = {(cuuint64_t)inner, (cuuint64_t)inner * (cuuint64_t)outer};   // bytes: 1 per element
  cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (strides[0] & 15)) {
    snprintf(g_err, sizeof g_err, "fp8 operand base and row pitch must be 16-byte aligned");
    return -11;
  }
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return -12; }
  return 0;
}

}  // namespace fl8

extern "C" const char* fl_fp8_last_error(void) { return fl8::g_err; }

extern "C" int fl_fp8_grouped_gemm(const FlFp8GemmDesc* d, cudaStream_t stream) {
  using namespace fl8;
  g_err[0] = 0;
  auto bad = [](const char* why) { snprintf(g_err, sizeof g_err, "%s", why); return -1; };
  if (d->num_groups < 1 || d->num_groups > FL_GEMM_MAX_GROUPS) return bad("num_groups out of range");
  if (d->cap <= 0 || d->cap % 128) return bad("cap must be a positive multiple of 128");
  if (d->N % 256) return bad("N must be a multiple of 256");
  if (d->K % 128) return bad("K must be a multiple of 128 (one scale block per stage)");
  if (d->epilogue != FL_EPI_STORE && d->epilogue != FL_EPI_SWIGLU && d->epilogue != FL_EPI_SCATTER && d->epilogue != FL_EPI_DSWIGLU)
    return bad("unsupported epilogue for the fp8 kernel");
  KParams p;
  memset(&p, 0, sizeof p);
  p.num_groups = d->num_groups; p.cap = d->cap; p.N = d->N; p.K = d->K; p.counts = d->counts;
  p.a_scale = d->a_scale; p.b_scale = d->b_scale; p.b_mn = d->b_mn_major; p.epilogue = d->epilogue;
  p.C = (__nv_bfloat16*)d->C; p.ldc = d->ldc; p.gu = (__nv_bfloat16*)d->gu; p.ldgu = d->ldgu; p.dgu = (__nv_bfloat16*)d->dgu;
  p.row_info = d->row_info; p.peers = d->peers; p.zero_tail = d->zero_tail;
  p.num_peers = d->num_peers; p.peer_rows = d->peer_rows;
  if (d->epilogue == FL_EPI_SCATTER) {
    if (d->num_peers < 1 || d->num_peers > FL_MAX_PEERS) return bad("SCATTER needs 1..8 receive buffers (num_peers)");
    if (d->row_info == nullptr) return bad("SCATTER needs row_info");
    for (int i = 0; i < d->num_peers; ++i)
      if (d->peers.p[i] == nullptr) return bad("SCATTER: a receive buffer is null");
  }
  p.group_m = d->group_m > 0 ? d->group_m : 16; p.status = d->status;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, d->A, d->K, d->cap, d->num_groups, 128, BM);
  if (rc) return rc;
  rc = d->b_mn_major ? make_map(&tmB, d->B, d->N, d->K, d->num_groups, 128, 128)
                     : make_map(&tmB, d->B, d->K, d->N, d->num_groups, 128, BN);
  if (rc) return rc;
  static int sms_of[64];                       // per device: the shared-memory attribute belongs to the device's copy of the kernel
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return bad("device ordinal out of range");
  int& num_sms = sms_of[dev];
  if (!num_sms) {
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(fp8_grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) { num_sms = 0; return (int)e; }
  }
  int grid = num_sms;
  if (d->max_ctas > 0 && d->max_ctas < grid) grid = d->max_ctas;
  fp8_grouped_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

extern "C" int fl_fp8_quantize_rows(const void* x, void* q, float* scale, long long rows, int K, const int* counts, int cap,
                                    cudaStream_t stream) {
  if (K % 128 || rows <= 0) return -1;
  long long warps = rows * (K / 128);
  int ctas = (int)((warps + 7) / 8 < 148 * 16 ? (warps + 7) / 8 : 148 * 16);
  fl8::quantize_rows_kernel<<<ctas, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_fp8_storage_t*)q, scale, rows, K, counts, cap);
  return (int)cudaGetLastError();
}

extern "C" int fl_fp8_quantize_blocks(const void* w, void* q, float* scale, int G, int R, int C, cudaStream_t stream) {
  if (R % 128 || C % 128 || G < 1) return -1;
  dim3 grid(C / 128, R / 128, G);
  fl8::quantize_blocks_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)w, (__nv_fp8_storage_t*)q, scale, R, C);
  return (int)cudaGetLastError();
}
