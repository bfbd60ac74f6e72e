// Persistent, warp-specialised grouped GEMM for sm_100a.
//
//   warp 0      : TMA producer  (tiled TMA loads, one per CTA; operands are always local memory)
//   warp 1      : MMA issuer    (tcgen05.mma kind::f16, one elected thread), owns the TMEM allocation
//   warps 2..9  : epilogue      (tcgen05.ld -> registers -> fused epilogue -> global / peer stores); two warps
//                 share each TMEM lane quadrant and split the tile's columns
//
// One CTA per SM walks a tile list that is derived on the device from the per-expert row counts, so the
// host never has to read the routing result back.  Tile = 128 x 256 fp32 accumulator in TMEM, two
// accumulators (512 columns) so the epilogue of tile i overlaps the main loop of tile i+1.  Operand
// tiles are 128-byte-swizzled, 4 stages of (16 KiB A + 32 KiB B).
//
// The fused epilogues are what make this the MoE hot path rather than a library GEMM:
//   SWIGLU  : gate/up interleaved weight -> act = silu(g)*u written once, g/u saved for backward
//   SCATTER : every output row is stored straight into the home GPU's combine buffer over NVLink
//   DSWIGLU : backward of the activation applied on the dAct accumulator
//   WGRAD   : contraction over the routed tokens (both operands MN-major), optional in-place SGD
//
// Reference parity: the reference ships no GPU kernels; its MoE workload is an external
// Megatron-DeepSpeed checkout (.gitmodules:11-13) whose expert FFN is a framework GEMM between two NCCL
// all-to-alls.  This file is the replacement for that GEMM + the second all-to-all.
#include "grouped_gemm.cuh"
#include "../common/fl_ptx.cuh"
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace fl {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int ROW_BYTES = 128;            // one swizzle row: 64 bf16 along the contiguous dimension
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * ROW_BYTES;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * ROW_BYTES;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 320;           // 1 TMA warp + 1 MMA warp + 8 epilogue warps
constexpr int TMEM_COLS = 512;
constexpr int EPI_STAGE_BYTES = 32 * 64;   // per epilogue warp: 32 rows x 32 bf16, the transposition buffer of its stores
constexpr int EPI_SMEM_BYTES = 8 * EPI_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 1024 /*barriers, counts*/ + EPI_SMEM_BYTES;

struct KParams {
  int group_mode, num_groups, cap, M, N, K;
  const int* counts;
  int a_mn, b_mn;
  int epilogue;
  __nv_bfloat16* C; long long ldc, gsc;
  __nv_bfloat16* gu; long long ldgu;
  __nv_bfloat16* dgu;
  const int* row_info;
  FlPeerPtrs peers;
  int num_peers; long long peer_rows;
  int push_world, push_rank, push_shift;   // WGRAD: rows dealt out to the ranks that sum them (FlGemmDesc::push_world)
  float sgd_lr;
  int zero_tail;
  int group_m;
  int* status;
  int stagger_ns;   // wide kernel: CTA pair i starts its first tile i / num_pairs of this long after the others (0 = off)
};

struct Tile {
  int g, m0, n0, kblocks, rows;  // rows: valid rows of this tile (M-grouped), BM otherwise
  int cnt;                       // rows routed to group g
};

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int counts[FL_GEMM_MAX_GROUPS];
};

// Map a linear tile id to a tile.  Every role of the CTA calls this with the same id and gets the same
// answer; the list ends at the first id that maps to nothing.
__device__ __forceinline__ bool map_tile(const KParams& p, const int* counts, int id, Tile& t, const int TM = BM,
                                         const int TN = BN) {
  const int NT = (p.N + TN - 1) / TN;
  if (p.group_mode == 0) {
    const int kblocks = (p.K * 2 /*bytes*/ + ROW_BYTES - 1) / ROW_BYTES;
    int acc = 0;
    for (int g = 0; g < p.num_groups; ++g) {
      const int cnt = counts[g];
      const int mt = (cnt + TM - 1) / TM;
      const int tiles = mt * NT;
      if (id < acc + tiles) {
        const int l = id - acc;
        const int per_sg = p.group_m * NT;
        const int sg = l / per_sg;
        const int first_m = sg * p.group_m;
        const int gsz = min(p.group_m, mt - first_m);
        const int r = l - sg * per_sg;
        const int m = first_m + r % gsz;
        const int n = r / gsz;
        t.g = g; t.m0 = m * TM; t.n0 = n * TN; t.kblocks = kblocks;
        t.rows = min(TM, cnt - t.m0);
        t.cnt = cnt;
        return true;
      }
      acc += tiles;
    }
    return false;
  } else {
    const int MT = (p.M + TM - 1) / TM;
    const int per_group = MT * NT;
    const int g = id / per_group;
    if (g >= p.num_groups) return false;
    const int l = id - g * per_group;
    const int per_sg = p.group_m * NT;
    const int sg = l / per_sg;
    const int first_m = sg * p.group_m;
    const int gsz = min(p.group_m, MT - first_m);
    const int r = l - sg * per_sg;
    t.g = g; t.m0 = (first_m + r % gsz) * TM; t.n0 = (r / gsz) * TN;
    t.kblocks = (counts[g] + 63) / 64;
    t.rows = TM;
    t.cnt = counts[g];
    return true;
  }
}

// sigmoid(x) = 0.5 tanh(0.5 x) + 0.5 with the hardware tanh (one special-function instruction; its error is far below
// the bf16 rounding of the results).  The epilogues that use it cost energy in proportion to their instruction count, and
// an exponential followed by an IEEE division is about fifteen instructions per element.
__device__ __forceinline__ float sigmoid_f(float x) { return fmaf(tanh_approx(0.5f * x), 0.5f, 0.5f); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack_bf16(uint32_t u, float& a, float& b) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  a = __bfloat162float(v.x);
  b = __bfloat162float(v.y);
}
// store 32 fp32 values as 32 bf16 (64 B) to a 16-byte aligned address
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
__device__ __forceinline__ void load32_bf16(const __nv_bfloat16* src, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 o = ld_v4(src + 8 * i);
    unpack_bf16(o.x, v[8 * i + 0], v[8 * i + 1]);
    unpack_bf16(o.y, v[8 * i + 2], v[8 * i + 3]);
    unpack_bf16(o.z, v[8 * i + 4], v[8 * i + 5]);
    unpack_bf16(o.w, v[8 * i + 6], v[8 * i + 7]);
  }
}

// Coalesced store of a 32-row x 32-column bf16 block that the warp holds row-per-thread (thread t = row t, as TMEM hands
// it out).  Written straight from the registers, every store instruction would touch 32 rows x 16 bytes: 32 half-used
// sectors.  Instead every thread parks its row (64 bytes) in the warp's shared-memory buffer and the warp writes the block
// back out with four lanes per row: one instruction covers 8 rows x 64 contiguous bytes, whole sectors only.
//   pk       the thread's 32 values as 16 packed bf16 pairs
//   row_dst  global address of the first of these 32 columns in the thread's OWN row, 0 if the row is not to be stored
// The 16-byte pieces of a row are XOR-swizzled by the row number so that neither the row-wise writes nor the
// four-lanes-per-row reads conflict on shared-memory banks.
__device__ __forceinline__ void staged_store_packed(uint8_t* stg, int lane, const uint32_t* pk, unsigned long long row_dst) {
  const uint32_t base = smem_u32(stg);
  const uint32_t wsw = (uint32_t)((lane >> 1) & 3);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t a = base + lane * 64 + (((uint32_t)j ^ wsw) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(pk[4 * j + 0]), "r"(pk[4 * j + 1]), "r"(pk[4 * j + 2]),
                 "r"(pk[4 * j + 3])
                 : "memory");
  }
  __syncwarp();
  const int piece = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = (lane >> 2) + 8 * i;
    const unsigned long long d = __shfl_sync(0xffffffffu, row_dst, r);
    const uint32_t a = base + r * 64 + (((uint32_t)piece ^ (uint32_t)((r >> 1) & 3)) << 4);
    uint4 x;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "r"(a) : "memory");
    if (d != 0) st_v4(reinterpret_cast<void*>(d + 16ull * piece), x);
  }
  __syncwarp();
}
__device__ __forceinline__ void staged_store32(uint8_t* stg, int lane, const float* v, unsigned long long row_dst) {
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
  staged_store_packed(stg, lane, pk, row_dst);
}

// What one CTA drains from its accumulator: a slab of 128 rows x BN columns.
struct EpiSlab {
  int g;           // group (expert)
  int row0;        // first row of the slab inside the group (M-grouped) or first output row (K-grouped)
  int n0;          // first column
  int valid_rows;  // M-grouped: rows of the slab that hold routed tokens (may be <= 0); K-grouped: 128
  int zero_limit;  // rows in [valid, zero_limit) are written as zeros when zero_tail is set
  bool have_acc;   // false when the contraction was empty (an expert that received no token)
};

// DSWIGLU reads the saved gate/up of its slab: `cols` accumulator columns starting at n0 correspond to 2 * cols contiguous
// columns of the interleaved gate/up row.  Asked for before the wait on the accumulator, the rows are in L2 by the time the
// epilogue's loads want them (they were written by the forward pass and have long left the cache).  One request per row.
__device__ __forceinline__ void prefetch_saved_gate_up(const KParams& p, int g, int row0, int valid_rows, int n0, int cols,
                                                       int r_in_tile) {
  if (r_in_tile < valid_rows) {
    const __nv_bfloat16* src = p.gu + ((long long)g * p.cap + row0 + r_in_tile) * p.ldgu + 2ll * n0;
    bulk_prefetch_l2(src, (uint32_t)(cols * 2 * 2));
  }
}

// WGRAD with the fused SGD update reads the weights it rewrites: one L2 request per weight row of the slab, made before the
// wait on the accumulator, so that the epilogue's row-per-thread loads find them in L2.
__device__ __forceinline__ void prefetch_weights(const KParams& p, int g, int row0, int n0, int cols, int r_in_tile) {
  const int row = row0 + r_in_tile;
  if (row < p.M && cols > 0)
    bulk_prefetch_l2(p.C + (long long)g * p.gsc + (long long)row * p.ldc + n0, (uint32_t)(cols * 2));
}

// Fused epilogues, run by the 8 epilogue warps of a CTA: warp (q, half) owns TMEM lanes [32q, 32q+32) and half of
// the columns; thread = one output row.
__device__ __forceinline__ void epilogue_slab(const KParams& p, const EpiSlab& e, uint32_t acc_addr, int q, int half,
                                              int lane, uint8_t* stg) {
  const int r_in_tile = q * 32 + lane;
  const int row = e.row0 + r_in_tile;            // row inside the group (M-grouped) / output row (K-grouped)
  const uint32_t t_addr = acc_addr + ((uint32_t)(q * 32) << 16);
  const bool have_acc = e.have_acc;
  if (p.epilogue == FL_EPI_STORE || p.epilogue == FL_EPI_SCATTER || p.epilogue == FL_EPI_WGRAD) {
    bool valid, zero_row = false;
    __nv_bfloat16* dst = nullptr;
    if (p.epilogue == FL_EPI_STORE) {
      valid = r_in_tile < e.valid_rows;
      zero_row = !valid && p.zero_tail && row < e.zero_limit;
      dst = p.C + (long long)e.g * p.gsc + (long long)row * p.ldc;
    } else if (p.epilogue == FL_EPI_SCATTER) {
      valid = r_in_tile < e.valid_rows;
      if (valid) {
        const int info = p.row_info[(long long)e.g * p.cap + row];
        const int rk = (info >> 28) & 0xF;
        const long long slot = info & 0x0FFFFFFF;
        if (rk >= p.num_peers || (p.peer_rows > 0 && slot >= p.peer_rows)) {
          report(p.status, kBadIndex, 500);      // a row that names no rank / no slot of the receive buffer: not stored
          valid = false;
        } else {
          dst = reinterpret_cast<__nv_bfloat16*>(p.peers.p[rk]) + slot * p.ldc;
        }
      }
    } else if (p.push_world > 0) {
      // the row goes to the rank that sums its block, into the part of that rank's buffer kept for this source
      valid = row < p.M;
      const int blk = row >> p.push_shift;
      const long long lrow = ((long long)(blk / p.push_world) << p.push_shift) + (row & ((1 << p.push_shift) - 1));
      const long long rows_own = p.M / p.push_world;
      dst = reinterpret_cast<__nv_bfloat16*>(p.peers.p[blk % p.push_world]) +
            (((long long)e.g * p.push_world + p.push_rank) * rows_own + lrow) * p.ldc;
    } else {
      valid = row < p.M;
      dst = p.C + (long long)e.g * p.gsc + (long long)row * p.ldc;
    }
#pragma unroll 1
    for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
      uint32_t r[32];
      float v[32];
      if (have_acc) {
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      const int col = e.n0 + c * 32;
      if (col >= p.N) continue;
      if (valid) {
        if (p.epilogue == FL_EPI_WGRAD && p.sgd_lr != 0.f) {
          float w[32];
          load32_bf16(dst + col, w);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = w[i] - p.sgd_lr * v[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      staged_store32(stg, lane, v, (valid || zero_row) ? reinterpret_cast<unsigned long long>(dst + col) : 0ull);
    }
  } else if (p.epilogue == FL_EPI_SWIGLU) {
    const bool valid = r_in_tile < e.valid_rows;
    const bool zero_row = !valid && p.zero_tail && row < e.zero_limit;
    const long long grow = (long long)e.g * p.cap + row;
    __nv_bfloat16* act = p.C + grow * p.ldc + e.n0 / 2;
    __nv_bfloat16* gu = p.gu ? p.gu + grow * p.ldgu + e.n0 : nullptr;
#pragma unroll 1
    for (int c = half * 2; c < half * 2 + 2; ++c) {
      uint32_t rg[32], ru[32];
      tmem_ld_32x32(t_addr + c * 32, rg);
      tmem_ld_32x32(t_addr + 128 + c * 32, ru);
      tmem_ld_wait();
      uint32_t pa[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float g0 = valid ? __uint_as_float(rg[2 * i]) : 0.f, g1 = valid ? __uint_as_float(rg[2 * i + 1]) : 0.f;
        const float u0 = valid ? __uint_as_float(ru[2 * i]) : 0.f, u1 = valid ? __uint_as_float(ru[2 * i + 1]) : 0.f;
        pa[i] = pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
        rg[i] = pack_bf16(g0, g1);      // the packed gate / up reuse the front half of their registers
        ru[i] = pack_bf16(u0, u1);
      }
      const bool st = valid || zero_row;
      staged_store_packed(stg, lane, pa, st ? reinterpret_cast<unsigned long long>(act + c * 32) : 0ull);
      if (gu) {
        staged_store_packed(stg, lane, rg, st ? reinterpret_cast<unsigned long long>(gu + c * 32) : 0ull);
        staged_store_packed(stg, lane, ru, st ? reinterpret_cast<unsigned long long>(gu + 128 + c * 32) : 0ull);
      }
    }
  } else {  // FL_EPI_DSWIGLU
    const bool valid = r_in_tile < e.valid_rows;
    const bool zero_row = !valid && p.zero_tail && row < e.zero_limit;
    const long long grow = (long long)e.g * p.cap + row;
    // Saved gate/up of the next 32-column chunk are fetched (packed bf16, 2 x 64 B) while the current chunk's
    // accumulator read and math are in flight, so the global-load latency is paid once per tile, not per chunk.
    const int c0 = half * (BN / 64), c1 = c0 + BN / 64;
    auto gate_col = [&](int c) {
      const int a_col = e.n0 + c * 32;                          // column of dAct
      return (long long)(a_col >> 7) * 256 + (a_col & 127);     // gate position in the interleaved row; up is +128
    };
    const __nv_bfloat16* gu_row = p.gu + grow * p.ldgu;
    __nv_bfloat16* dgu_row = p.dgu + grow * p.ldgu;
    uint4 gq[4], uq[4];
    if (valid) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        gq[i] = ld_v4(gu_row + gate_col(c0) + 8 * i);
        uq[i] = ld_v4(gu_row + gate_col(c0) + 128 + 8 * i);
      }
    }
#pragma unroll
    for (int c = c0; c < c1; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(t_addr + c * 32, r);
      uint4 gn[4], un[4];
      if (valid && c + 1 < c1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          gn[i] = ld_v4(gu_row + gate_col(c + 1) + 8 * i);
          un[i] = ld_v4(gu_row + gate_col(c + 1) + 128 + 8 * i);
        }
      }
      tmem_ld_wait();
      const long long gcol = gate_col(c);
      uint32_t pdg[16], pdu[16];
      if (valid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t gw[4] = {gq[i].x, gq[i].y, gq[i].z, gq[i].w};
          const uint32_t uw[4] = {uq[i].x, uq[i].y, uq[i].z, uq[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float g0, g1, u0, u1;
            unpack_bf16(gw[j], g0, g1);
            unpack_bf16(uw[j], u0, u1);
            const int e = 8 * i + 2 * j;
            const float da0 = __uint_as_float(r[e]), da1 = __uint_as_float(r[e + 1]);
            // with s = sigmoid(g) and t = g s = silu(g):  d/dg silu(g) = s + t (1 - s),  so  dG = dA u (s + t - t s),  dU = dA t
            const float s0 = sigmoid_f(g0), s1 = sigmoid_f(g1);
            const float t0 = g0 * s0, t1 = g1 * s1;
            pdg[e >> 1] = pack_bf16((da0 * u0) * (fmaf(-t0, s0, t0) + s0), (da1 * u1) * (fmaf(-t1, s1, t1) + s1));
            pdu[e >> 1] = pack_bf16(da0 * t0, da1 * t1);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) pdg[i] = pdu[i] = 0u;
      }
      {
        const bool st = valid || zero_row;
        staged_store_packed(stg, lane, pdg, st ? reinterpret_cast<unsigned long long>(dgu_row + gcol) : 0ull);
        staged_store_packed(stg, lane, pdu, st ? reinterpret_cast<unsigned long long>(dgu_row + gcol + 128) : 0ull);
      }
      if (c + 1 < c1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) { gq[i] = gn[i]; uq[i] = un[i]; }
      }
    }
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  // operand stages need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tmem_full[a], 1);
      mbar_init(&sh->tmem_empty[a], 8);  // one arrival per epilogue warp
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;  // global k-block counter -> stage and phase
      bool ok = true;
      Tile t;
      for (int id = blockIdx.x; ok && map_tile(p, counts, id, t); id += gridDim.x) {
        for (int kb = 0; kb < t.kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&sh->empty[s], ph ^ 1, abort_flag, p.status, kTimeoutMbarEmpty, 100 + s);
          if (!ok) break;
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&sh->full[s], STAGE_BYTES);
          const int k0 = kb * 64;
          if (p.group_mode == 0) {
            // A rows of group g, K-major: box {64 k, 128 rows}
            tma_load_3d(a_dst, &tmA, &sh->full[s], k0, t.m0, t.g);
            if (!p.b_mn) {
              tma_load_3d(b_dst, &tmB, &sh->full[s], k0, t.n0, t.g);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(b_dst + j * (64 * ROW_BYTES), &tmB, &sh->full[s], t.n0 + 64 * j, k0, t.g);
            }
          } else {
            // both operands MN-major, contraction over the rows of group g: boxes {64 mn, 64 rows}
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(a_dst + j * (64 * ROW_BYTES), &tmA, &sh->full[s], t.m0 + 64 * j, k0, t.g);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * (64 * ROW_BYTES), &tmB, &sh->full[s], t.n0 + 64 * j, k0, t.g);
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight time to land before the CTA (and its shared memory) goes away
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 1, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u, BM, BN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      Tile t;
      for (int id = blockIdx.x; ok && map_tile(p, counts, id, t); id += gridDim.x, ++tile_i) {
        const int acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        ok = mbar_wait(&sh->tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, 200 + acc);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&sh->full[s], ph, abort_flag, p.status, kTimeoutMbarFull, 300 + s);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_base = a_base + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // 4 x (K = 16) per 64-wide k-block
            const uint64_t da = p.a_mn ? make_smem_desc(a_base + kk * 2048, 64 * ROW_BYTES, 1024)
                                       : make_smem_desc(a_base + kk * 32, 16, 1024);
            const uint64_t db = p.b_mn ? make_smem_desc(b_base + kk * 2048, 64 * ROW_BYTES, 1024)
                                       : make_smem_desc(b_base + kk * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&sh->empty[s]);  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        if (t.kblocks > 0) umma_commit(&sh->tmem_full[acc]);
        else mbar_arrive(&sh->tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps, 128 rows x 2 column halves)
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    uint32_t tile_i = 0;
    bool ok = true;
    Tile t;
    for (int id = blockIdx.x; ok && map_tile(p, counts, id, t); id += gridDim.x, ++tile_i) {
      const int acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (p.epilogue == FL_EPI_DSWIGLU && half == 0)
        prefetch_saved_gate_up(p, t.g, t.m0, t.rows, t.n0, min(BN, p.N - t.n0), q * 32 + lane);
      if (p.epilogue == FL_EPI_WGRAD && p.sgd_lr != 0.f && half == 0)
        prefetch_weights(p, t.g, t.m0, t.n0, min(BN, p.N - t.n0), q * 32 + lane);
      ok = mbar_wait(&sh->tmem_full[acc], acc_ph, abort_flag, p.status, kTimeoutTmemFull, 400 + acc);
      if (!ok) break;
      tc_fence_after_sync();
      EpiSlab e;
      e.g = t.g; e.row0 = t.m0; e.n0 = t.n0; e.valid_rows = t.rows; e.have_acc = t.kblocks > 0;
      e.zero_limit = p.group_mode == 0 ? min(p.cap, (t.cnt + 127) / 128 * 128) : 0;
      epilogue_slab(p, e, tmem_base + acc * BN, q, half, lane, smem + STAGES * STAGE_BYTES + 1024 + (warp - 2) * EPI_STAGE_BYTES);
      // accumulator drained: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
    }
    if (p.epilogue == FL_EPI_SCATTER || p.push_world > 0) fence_sys();  // peer stores visible before the kernel's completion is signalled
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ==================================================================================================
// CTA-pair variant: two CTAs (a cluster of 2, one per SM of a pair) work on one 256 x 256 tile with
// tcgen05 cta_group::2.  Each CTA loads its own 128 rows of A and its own 128 columns' worth of B (so a pair
// moves 64 KiB per k-block for twice the math of a single CTA's 48 KiB: a third less L2 -> SM traffic),
// the leader CTA issues the MMAs for both, and each CTA drains the 128 accumulator rows that live in its own
// TMEM.  No load is multicast: the second CTA fetches its halves itself.
// ==================================================================================================
constexpr int STAGES2 = 6;
constexpr int HALF_BYTES = 128 * ROW_BYTES;            // 16 KiB: 128 rows (or 2 x 64-wide MN atoms) x 128 B
constexpr int STAGE2_BYTES = 2 * HALF_BYTES;           // A half + B half per CTA
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 1024 + 1024 + EPI_SMEM_BYTES;

struct SharedPair {
  uint64_t full[STAGES2];
  uint64_t empty[STAGES2];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int counts[FL_GEMM_MAX_GROUPS];
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedPair* sh = reinterpret_cast<SharedPair*>(smem + STAGES2 * STAGE2_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();       // 0 = leader (issues the MMAs), 1 = peer
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  constexpr int TM = 2 * BM;                      // rows of a pair's tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&sh->full[s], 1);                 // used in the leader: one arrive.expect_tx covering both CTAs' bytes
      mbar_init(&sh->empty[s], 1);                // one multicast commit from the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tmem_full[a], 1);
      mbar_init(&sh->tmem_empty[a], 16);          // used in the leader: 8 epilogue warps of each CTA
    }
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  for (int g = threadIdx.x; g < p.num_groups; g += NUM_THREADS)
    sh->counts[g] = p.counts ? min(p.counts[g], p.cap) : p.cap;
  if (warp == 1) {
    tmem_alloc_2cta(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                              // both CTAs' barriers exist before either signals the other
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  const int* counts = sh->counts;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      Tile t;
      for (int id = pair_id; ok && map_tile(p, counts, id, t, TM); id += num_pairs) {
        for (int kb = 0; kb < t.kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          ok = mbar_wait(&sh->empty[s], ph ^ 1, abort_flag, p.status, kTimeoutMbarEmpty, 1100 + s);
          if (!ok) break;
          uint8_t* a_dst = smem + s * STAGE2_BYTES;
          uint8_t* b_dst = a_dst + HALF_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&sh->full[s], 2 * STAGE2_BYTES);   // bytes of both CTAs
          const uint32_t full_leader = map_to_cta(smem_u32(&sh->full[s]), 0);
          const int k0 = kb * 64;
          const int mh = t.m0 + 128 * (int)rank;   // this CTA's rows of the tile
          const int nh = t.n0 + 128 * (int)rank;   // this CTA's share of the tile's columns (B operand)
          if (p.group_mode == 0) {
            tma_load_3d_pair(a_dst, &tmA, full_leader, k0, mh, t.g);
            if (!p.b_mn) {
              tma_load_3d_pair(b_dst, &tmB, full_leader, k0, nh, t.g);
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j)
                tma_load_3d_pair(b_dst + j * (64 * ROW_BYTES), &tmB, full_leader, nh + 64 * j, k0, t.g);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(a_dst + j * (64 * ROW_BYTES), &tmA, full_leader, mh + 64 * j, k0, t.g);
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(b_dst + j * (64 * ROW_BYTES), &tmB, full_leader, nh + 64 * j, k0, t.g);
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(1, 1, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u, TM, BN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      Tile t;
      for (int id = pair_id; ok && map_tile(p, counts, id, t, TM); id += num_pairs, ++tile_i) {
        const int acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        ok = mbar_wait(&sh->tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, 1200 + acc);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          ok = mbar_wait(&sh->full[s], ph, abort_flag, p.status, kTimeoutMbarFull, 1300 + s);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * STAGE2_BYTES);
          const uint32_t b_base = a_base + HALF_BYTES;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t da = p.a_mn ? make_smem_desc(a_base + kk * 2048, 64 * ROW_BYTES, 1024)
                                       : make_smem_desc(a_base + kk * 32, 16, 1024);
            const uint64_t db = p.b_mn ? make_smem_desc(b_base + kk * 2048, 64 * ROW_BYTES, 1024)
                                       : make_smem_desc(b_base + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&sh->empty[s], 0x3);          // frees the stage in both CTAs
        }
        if (!ok) break;
        if (t.kblocks > 0) {
          umma_commit_pair(&sh->tmem_full[acc], 0x3);    // accumulator ready in both CTAs
        } else {
          mbar_arrive(&sh->tmem_full[acc]);
          mbar_arrive_cluster(map_to_cta(smem_u32(&sh->tmem_full[acc]), 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t tile_i = 0;
    bool ok = true;
    Tile t;
    for (int id = pair_id; ok && map_tile(p, counts, id, t, TM); id += num_pairs, ++tile_i) {
      const int acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (p.epilogue == FL_EPI_DSWIGLU && half == 0)
        prefetch_saved_gate_up(p, t.g, t.m0 + 128 * (int)rank, min(128, t.cnt - (t.m0 + 128 * (int)rank)), t.n0, min(BN, p.N - t.n0),
                               q * 32 + lane);
      if (p.epilogue == FL_EPI_WGRAD && p.sgd_lr != 0.f && half == 0)
        prefetch_weights(p, t.g, t.m0 + 128 * (int)rank, t.n0, min(BN, p.N - t.n0), q * 32 + lane);
      ok = mbar_wait(&sh->tmem_full[acc], acc_ph, abort_flag, p.status, kTimeoutTmemFull, 1400 + acc);
      if (!ok) break;
      tc_fence_after_sync();
      EpiSlab e;
      e.g = t.g; e.row0 = t.m0 + 128 * (int)rank; e.n0 = t.n0; e.have_acc = t.kblocks > 0;
      e.valid_rows = p.group_mode == 0 ? min(128, t.cnt - e.row0) : 128;
      e.zero_limit = p.group_mode == 0 ? min(p.cap, (t.cnt + 127) / 128 * 128) : 0;
      epilogue_slab(p, e, tmem_base + acc * BN, q, half, lane, smem + STAGES2 * STAGE2_BYTES + 1024 + (warp - 2) * EPI_STAGE_BYTES);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->tmem_empty[acc]), 0));
    }
    if (p.epilogue == FL_EPI_SCATTER || p.push_world > 0) fence_sys();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                              // neither CTA frees TMEM while the other may still use the pair's
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}


// ==================================================================================================
// Wide CTA-pair variant: one 256 x 512 tile per pair, the whole of TMEM (512 columns) as ONE accumulator.
//
// Why: without multicast loads every SM has to pull all the operand bytes its MMAs consume through its own
// L2 port.  With 256 x 256 tiles that is 32 KiB per CTA for every 512 tensor-core cycles, which is what the
// port delivers at best, so loads and MMAs cannot both run at full rate.  A 256 x 512 tile reuses the A rows
// for twice as many columns: 48 KiB per CTA for every 1024 cycles, a quarter less traffic per FLOP.
//
// Price: there is no second accumulator to fill while the first is drained.  The accumulator is handed back
// in two column halves instead: the epilogue warps drain half 0, return it, then half 1, and the MMA thread
// starts the next tile on half 0 as soon as that half is back -- the first WIDE_LEAD k-blocks are issued for
// half 0 alone (their stages were loaded while the previous tile drained), then half 1 catches up and the
// two halves run in step, each k-block's stage being released after both have read it.
// ==================================================================================================
constexpr int STAGES3 = 4;
constexpr int WIDE_N = 512;
constexpr int WIDE_LEAD = 3;                            // k-blocks half 0 runs ahead of half 1 at the start of a tile (< STAGES3)
constexpr int STAGE3_BYTES = 3 * HALF_BYTES;           // A half (16 KiB) + B: this CTA's 128 columns of each 256-column half (2 x 16 KiB)
constexpr int SMEM3_BYTES = STAGES3 * STAGE3_BYTES + 1024 + 1024 + EPI_SMEM_BYTES;

struct SharedWide {
  uint64_t full[STAGES3];
  uint64_t empty[STAGES3];
  uint64_t half_full[2];     // accumulator columns [256 h, 256 h + 256) complete
  uint64_t half_empty[2];    // ... drained by the 8 epilogue warps of both CTAs
  uint32_t tmem_base;
  int abort_flag;
  int counts[FL_GEMM_MAX_GROUPS];
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedWide* sh = reinterpret_cast<SharedWide*>(smem + STAGES3 * STAGE3_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  constexpr int TM = 2 * BM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES3; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(&sh->half_full[h], 1);
      mbar_init(&sh->half_empty[h], 16);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  for (int g = threadIdx.x; g < p.num_groups; g += NUM_THREADS)
    sh->counts[g] = p.counts ? min(p.counts[g], p.cap) : p.cap;
  if (warp == 1) {
    tmem_alloc_2cta(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  const int* counts = sh->counts;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      Tile t;
      for (int id = pair_id; ok && map_tile(p, counts, id, t, TM, WIDE_N); id += num_pairs) {
        for (int kb = 0; kb < t.kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES3;
          const uint32_t ph = (it / STAGES3) & 1;
          ok = mbar_wait(&sh->empty[s], ph ^ 1, abort_flag, p.status, kTimeoutMbarEmpty, 2100 + s);
          if (!ok) break;
          uint8_t* a_dst = smem + s * STAGE3_BYTES;
          uint8_t* b_dst = a_dst + HALF_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&sh->full[s], 2 * STAGE3_BYTES);
          const uint32_t full_leader = map_to_cta(smem_u32(&sh->full[s]), 0);
          const int k0 = kb * 64;
          const int mh = t.m0 + 128 * (int)rank;
          if (p.group_mode == 0) {
            tma_load_3d_pair(a_dst, &tmA, full_leader, k0, mh, t.g);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(a_dst + j * (64 * ROW_BYTES), &tmA, full_leader, mh + 64 * j, k0, t.g);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int nh = t.n0 + 256 * h + 128 * (int)rank;   // this CTA's 128 columns of column half h
            uint8_t* bh = b_dst + h * HALF_BYTES;
            if (p.group_mode == 0 && !p.b_mn) {
              tma_load_3d_pair(bh, &tmB, full_leader, k0, nh, t.g);
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j)
                tma_load_3d_pair(bh + j * (64 * ROW_BYTES), &tmB, full_leader, nh + 64 * j, k0, t.g);
            }
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(1, 1, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u, TM, 256);
      uint32_t it0 = 0, tile_i = 0;               // it0: global index of the tile's first k-block
      bool ok = true;
      Tile t;
      // the MMAs of k-block `kb` of the tile for column half `h`
      auto issue = [&](int kb, int h) {
        const uint32_t it = it0 + kb;
        const int s = it % STAGES3;
        const uint32_t a_base = smem_u32(smem + s * STAGE3_BYTES);
        const uint32_t b_base = a_base + HALF_BYTES + h * HALF_BYTES;
        const uint32_t d_tmem = tmem_base + h * 256;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t da = p.a_mn ? make_smem_desc(a_base + kk * 2048, 64 * ROW_BYTES, 1024)
                                     : make_smem_desc(a_base + kk * 32, 16, 1024);
          const uint64_t db = p.b_mn ? make_smem_desc(b_base + kk * 2048, 64 * ROW_BYTES, 1024)
                                     : make_smem_desc(b_base + kk * 32, 16, 1024);
          umma_f16_pair(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
        }
      };
      auto wait_full = [&](int kb) {
        const uint32_t it = it0 + kb;
        const int s = it % STAGES3;
        const bool r = mbar_wait(&sh->full[s], (it / STAGES3) & 1, abort_flag, p.status, kTimeoutMbarFull, 2300 + s);
        tc_fence_after_sync();
        return r;
      };
      auto release = [&](int kb) { umma_commit_pair(&sh->empty[(it0 + kb) % STAGES3], 0x3); };
      if (p.stagger_ns > 0) {
        // Pairs that start together stay together: every pair would then reach its epilogue at the same moment and the
        // whole chip would write its output in one burst that the memory system cannot absorb, while nothing computes.
        // Spreading the starts over one tile's duration spreads the epilogues over the kernel.
        const uint64_t until = global_timer_ns() + (uint64_t)p.stagger_ns * (uint64_t)pair_id / (uint64_t)num_pairs;
        while (global_timer_ns() < until) __nanosleep(2000);
      }
      for (int id = pair_id; ok && map_tile(p, counts, id, t, TM, WIDE_N); id += num_pairs, ++tile_i) {
        const uint32_t ph = tile_i & 1;
        const int KB = t.kblocks;
        const int lead = min(WIDE_LEAD, KB);
        // half 0 may start as soon as it is drained: its first k-blocks are issued while half 1 is still being read out.
        // (The stages these k-blocks sit in were filled while the previous tile drained, so holding them costs nothing.)
        ok = mbar_wait(&sh->half_empty[0], ph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, 2200);
        if (!ok) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < lead && ok; ++kb) {
          ok = wait_full(kb);
          if (ok) issue(kb, 0);
        }
        if (!ok) break;
        ok = mbar_wait(&sh->half_empty[1], ph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, 2201);
        if (!ok) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < lead; ++kb) {       // half 1 catches up; from here on a k-block feeds both halves
          issue(kb, 1);
          release(kb);
        }
        for (int kb = lead; kb < KB && ok; ++kb) {
          ok = wait_full(kb);
          if (!ok) break;
          issue(kb, 0);
          issue(kb, 1);
          release(kb);
        }
        if (!ok) break;
        if (KB > 0) {
          umma_commit_pair(&sh->half_full[0], 0x3);
          umma_commit_pair(&sh->half_full[1], 0x3);
        } else {
          for (int h = 0; h < 2; ++h) {
            mbar_arrive(&sh->half_full[h]);
            mbar_arrive_cluster(map_to_cta(smem_u32(&sh->half_full[h]), 1));
          }
        }
        it0 += KB;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows, half by half)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t tile_i = 0;
    bool ok = true;
    Tile t;
    for (int id = pair_id; ok && map_tile(p, counts, id, t, TM, WIDE_N); id += num_pairs, ++tile_i) {
      const uint32_t ph = tile_i & 1;
      if (p.epilogue == FL_EPI_DSWIGLU && half == 0)
        prefetch_saved_gate_up(p, t.g, t.m0 + 128 * (int)rank, min(128, t.cnt - (t.m0 + 128 * (int)rank)), t.n0,
                               min(WIDE_N, p.N - t.n0), q * 32 + lane);
      if (p.epilogue == FL_EPI_WGRAD && p.sgd_lr != 0.f && half == 0)
        prefetch_weights(p, t.g, t.m0 + 128 * (int)rank, t.n0, min(WIDE_N, p.N - t.n0), q * 32 + lane);
      for (int h = 0; h < 2 && ok; ++h) {
        ok = mbar_wait(&sh->half_full[h], ph, abort_flag, p.status, kTimeoutTmemFull, 2400 + h);
        if (!ok) break;
        tc_fence_after_sync();
        EpiSlab e;
        e.g = t.g; e.row0 = t.m0 + 128 * (int)rank; e.n0 = t.n0 + 256 * h; e.have_acc = t.kblocks > 0;
        e.valid_rows = p.group_mode == 0 ? min(128, t.cnt - e.row0) : 128;
        e.zero_limit = p.group_mode == 0 ? min(p.cap, (t.cnt + 127) / 128 * 128) : 0;
        if (e.n0 < p.N)
          epilogue_slab(p, e, tmem_base + h * 256, q, half, lane, smem + STAGES3 * STAGE3_BYTES + 1024 + (warp - 2) * EPI_STAGE_BYTES);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->half_empty[h]), 0));
      }
    }
    if (p.epilogue == FL_EPI_SCATTER || p.push_world > 0) fence_sys();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

// --------------------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static thread_local char g_err[256] = "";

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 3-D bf16 view {inner, outer, groups}; box {box_inner, box_outer, 1}; 128-byte swizzle; zero fill.
static int make_map(CUtensorMap* m, const void* base, long long inner, long long outer, long long groups,
                    long long ld_elems, long long gs_elems, int box_inner, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled entry point not available");
    return -10;
  }
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)groups};
  if (gs_elems <= 0) gs_elems = ld_elems * outer;
  cuuint64_t strides[2] = {(cuuint64_t)ld_elems * 2, (cuuint64_t)gs_elems * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (strides[0] & 15) || (strides[1] & 15)) {
    snprintf(g_err, sizeof g_err, "operand base/strides must be 16-byte aligned");
    return -11;
  }
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err, sizeof g_err, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return -12;
  }
  return 0;
}

}  // namespace fl

extern "C" const char* fl_gemm_last_error(void) { return fl::g_err; }

// 0 = one CTA per tile (128 x 256), 1 = CTA pairs (256 x 256 tiles, two accumulators), 2 = CTA pairs on 256 x 512 tiles
// (one accumulator, a quarter less operand traffic per FLOP), 3 = chosen per launch (the default): the wide tiles for the
// row-grouped GEMMs, except where the epilogue is long and the contraction short (DSWIGLU with K < 8192) or the output is
// narrower than one wide tile; the 256 x 256 tiles for the weight-gradient GEMMs, whose contraction is as short as the
// smallest expert's row count while every tile's epilogue reads and rewrites its weights -- the second accumulator hides
// that.  FUSELINK_GEMM_PAIR overrides.
static int g_variant = -1;
extern "C" void fl_gemm_set_variant(int v) { g_variant = v < 0 ? 0 : v > 3 ? 3 : v; }
extern "C" int fl_gemm_get_variant(void) {
  if (g_variant < 0) {
    const char* e = getenv("FUSELINK_GEMM_PAIR");
    g_variant = (e && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 3;
  }
  return g_variant;
}

extern "C" int fl_grouped_gemm(const FlGemmDesc* d, cudaStream_t stream) {
  using namespace fl;
  g_err[0] = 0;
  auto bad = [](const char* why) {
    snprintf(g_err, sizeof g_err, "%s", why);
    return -1;
  };
  if (d->elem_bytes != 2) return bad("only bf16 operands are handled by this kernel (fp8 has its own entry point)");
  if (d->num_groups < 1 || d->num_groups > FL_GEMM_MAX_GROUPS) return bad("num_groups out of range");
  if (d->cap <= 0 || d->cap % 128) return bad("cap must be a positive multiple of 128");
  if (d->N % 32) return bad("N must be a multiple of 32");
  KParams p;
  memset(&p, 0, sizeof p);
  p.group_mode = d->group_mode; p.num_groups = d->num_groups; p.cap = d->cap;
  p.M = d->M; p.N = d->N; p.K = d->K; p.counts = d->counts;
  p.a_mn = d->a_mn_major; p.b_mn = d->b_mn_major; p.epilogue = d->epilogue;
  p.C = (__nv_bfloat16*)d->C; p.ldc = d->ldc; p.gsc = d->gsc;
  p.gu = (__nv_bfloat16*)d->gu; p.ldgu = d->ldgu; p.dgu = (__nv_bfloat16*)d->dgu;
  p.row_info = d->row_info; p.peers = d->peers; p.sgd_lr = d->sgd_lr; p.zero_tail = d->zero_tail;
  p.num_peers = d->num_peers; p.peer_rows = d->peer_rows;
  if (d->epilogue == FL_EPI_SCATTER) {
    if (d->num_peers < 1 || d->num_peers > FL_MAX_PEERS) return bad("SCATTER needs 1..8 receive buffers (num_peers)");
    if (d->row_info == nullptr) return bad("SCATTER needs row_info");
    for (int i = 0; i < d->num_peers; ++i)
      if (d->peers.p[i] == nullptr) return bad("SCATTER: a receive buffer is null");
  }
  if (d->push_world > 0) {
    if (d->epilogue != FL_EPI_WGRAD || d->group_mode != 1) return bad("push_world belongs to the K-grouped WGRAD epilogue");
    if (d->sgd_lr != 0.f) return bad("push_world: the update is applied by the rank that sums the rows, sgd_lr must be 0");
    if (d->push_world > FL_MAX_PEERS || d->push_rank < 0 || d->push_rank >= d->push_world) return bad("push_world / push_rank out of range");
    if (d->push_block_log2 < 0 || d->push_block_log2 > 16 || d->M % (d->push_world << d->push_block_log2))
      return bad("push_world: M must be a whole number of blocks per rank");
    for (int i = 0; i < d->push_world; ++i)
      if (d->peers.p[i] == nullptr) return bad("push_world: a receive buffer is null");
    p.push_world = d->push_world; p.push_rank = d->push_rank; p.push_shift = d->push_block_log2;
  }
  p.group_m = d->group_m > 0 ? d->group_m : 16;
  p.status = d->status;
  {
    // one wide tile takes about K / 64 k-blocks x 1024 tensor-core cycles; worth it only for the epilogues that write (and
    // read) several times the tile's size and when every pair has a few tiles to work on
    static int forced = -2;
    if (forced == -2) { const char* e = getenv("FUSELINK_GEMM_STAGGER_NS"); forced = e ? atoi(e) : -1; }
    const bool heavy = d->epilogue == FL_EPI_SWIGLU || d->epilogue == FL_EPI_DSWIGLU;
    p.stagger_ns = forced >= 0 ? forced : (heavy && d->group_mode == 0 ? (d->K / 64) * 650 : 0);
  }

  int variant = fl_gemm_get_variant();
  if (variant == 3) {
    const bool short_k_long_epilogue = d->group_mode == 0 && d->epilogue == FL_EPI_DSWIGLU && d->K < 8192;
    variant = (d->N < 512 || short_k_long_epilogue || d->group_mode == 1) ? 1 : 2;
  }
  const bool pair = variant >= 1;
  CUtensorMap tmA, tmB;
  int rc;
  if (d->group_mode == 0) {
    if (d->a_mn_major) return bad("M-grouped GEMM takes a K-major A (token rows)");
    if (d->K % 8) return bad("K must be a multiple of 8");
    if (d->epilogue == FL_EPI_WGRAD) return bad("WGRAD epilogue needs group_mode 1");
    if ((d->epilogue == FL_EPI_SWIGLU) && (d->N % 256)) return bad("SWIGLU needs N % 256 == 0");
    if ((d->epilogue == FL_EPI_DSWIGLU) && (d->N % 128)) return bad("DSWIGLU needs N % 128 == 0");
    rc = make_map(&tmA, d->A, d->K, d->cap, d->num_groups, d->lda, d->gsa, 64, BM);
    if (rc) return rc;
    if (!d->b_mn_major) rc = make_map(&tmB, d->B, d->K, d->N, d->num_groups, d->ldb, d->gsb, 64, pair ? 128 : BN);
    else rc = make_map(&tmB, d->B, d->N, d->K, d->num_groups, d->ldb, d->gsb, 64, 64);
    if (rc) return rc;
  } else {
    if (!d->a_mn_major || !d->b_mn_major) return bad("K-grouped GEMM takes MN-major A and B (token-major buffers)");
    if (d->epilogue != FL_EPI_WGRAD) return bad("K-grouped GEMM supports the WGRAD epilogue only");
    if (d->M % 8) return bad("M must be a multiple of 8");
    rc = make_map(&tmA, d->A, d->M, d->cap, d->num_groups, d->lda, d->gsa, 64, 64);
    if (rc) return rc;
    rc = make_map(&tmB, d->B, d->N, d->cap, d->num_groups, d->ldb, d->gsb, 64, 64);
    if (rc) return rc;
  }

  // per device: a process may drive several GPUs, and the shared-memory attribute belongs to the device's copy of the kernel
  constexpr int kMaxDev = 64;
  static int sms_of[kMaxDev], pairs_of[kMaxDev];
  static bool attr_set_of[kMaxDev];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDev) return bad("device ordinal out of range");
  int& num_sms = sms_of[dev];
  int& max_pairs = pairs_of[dev];
  bool& attr_set = attr_set_of[dev];
  if (!attr_set) {
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(grouped_gemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM3_BYTES);
    if (e != cudaSuccess) return (int)e;
    // how many CTA pairs can be resident at once (SM pairs are not guaranteed for every SM of the chip)
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(num_sms & ~1, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM2_BYTES;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int nclusters = 0;
    if (cudaOccupancyMaxActiveClusters(&nclusters, grouped_gemm_pair_kernel, &cfg) == cudaSuccess && nclusters > 0)
      max_pairs = nclusters;
    else
      max_pairs = num_sms / 2;
    cudaGetLastError();
    attr_set = true;
  }
  if (pair) {
    int pairs = max_pairs;
    if (d->max_ctas > 0 && d->max_ctas / 2 < pairs) pairs = d->max_ctas / 2 > 0 ? d->max_ctas / 2 : 1;
    if (variant == 2) grouped_gemm_wide_kernel<<<2 * pairs, NUM_THREADS, SMEM3_BYTES, stream>>>(tmA, tmB, p);
    else grouped_gemm_pair_kernel<<<2 * pairs, NUM_THREADS, SMEM2_BYTES, stream>>>(tmA, tmB, p);
    return (int)cudaGetLastError();
  }
  int grid = num_sms;
  if (d->max_ctas > 0 && d->max_ctas < grid) grid = d->max_ctas;
  grouped_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}
