// Chunked multi-segment put, flag wait and flag barrier (see comm_kernels.cuh for the protocol).
//
// Reference parity: the reference moves bytes between GPUs only implicitly (NCCL's copy kernel writes
// through a remapped VA, src/fuselink.cc:43-56) and stripes one transfer over NCCL channels in 512 KiB
// chunks with 8 steps in flight (experiments/bw_test/run_bw_test.sbatch:34-46, src/fuselink.h:14).  Here
// the stripes are explicit: one launch copies any number of (src, dst) segments chunk by chunk and
// publishes a flag per chunk, so a relay GPU can forward chunk c while chunk c+1 is still in flight.
#include "comm_kernels.cuh"
#include "../common/fl_ptx.cuh"
#include <string.h>

namespace fl {

constexpr int BULK_SLOTS = 4;
constexpr int BULK_SLOT_BYTES = 16 * 1024;

__device__ __forceinline__ void copy_vec(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                         unsigned long long bytes) {
  const int tid = threadIdx.x, nt = blockDim.x;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    const unsigned long long n16 = bytes >> 4;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    unsigned long long i = tid;
    // 4 independent 16-byte loads in flight per thread before the first store
    for (; i + 3ull * nt < n16; i += 4ull * nt) {
      uint4 a = ld_nc_v4(s + i), b = ld_nc_v4(s + i + nt), c = ld_nc_v4(s + i + 2 * nt), e = ld_nc_v4(s + i + 3 * nt);
      st_v4(d + i, a); st_v4(d + i + nt, b); st_v4(d + i + 2 * nt, c); st_v4(d + i + 3 * nt, e);
    }
    for (; i < n16; i += nt) st_v4(d + i, ld_nc_v4(s + i));
    for (unsigned long long b = (n16 << 4) + tid; b < bytes; b += nt) dst[b] = src[b];
  } else {
    for (unsigned long long b = tid; b < bytes; b += nt) dst[b] = src[b];
  }
}

// One thread streams the chunk through a ring of shared-memory slots with the bulk-copy engine:
// global -> smem (mbarrier completion) then smem -> global (bulk group).  No multicast anywhere.
__device__ __forceinline__ bool copy_bulk(const uint8_t* src, uint8_t* dst, unsigned long long bytes,
                                          uint8_t* ring, uint64_t* bars, uint32_t& phase_bits, int* abort_flag,
                                          int* status) {
  const int n = (int)((bytes + BULK_SLOT_BYTES - 1) / BULK_SLOT_BYTES);
  auto slot_bytes = [&](int j) {
    unsigned long long off = (unsigned long long)j * BULK_SLOT_BYTES;
    unsigned long long left = bytes - off;
    return (uint32_t)(left < BULK_SLOT_BYTES ? left : BULK_SLOT_BYTES);
  };
  auto issue_load = [&](int j) {
    const int s = j % BULK_SLOTS;
    mbar_arrive_expect_tx(&bars[s], slot_bytes(j));
    bulk_load(ring + s * BULK_SLOT_BYTES, src + (unsigned long long)j * BULK_SLOT_BYTES, slot_bytes(j), &bars[s]);
  };
  for (int j = 0; j < n && j < BULK_SLOTS - 1; ++j) issue_load(j);
  bool ok = true;
  for (int j = 0; j < n; ++j) {
    const int s = j % BULK_SLOTS;
    ok = mbar_wait(&bars[s], (phase_bits >> s) & 1, abort_flag, status, kTimeoutMbarFull, 500 + s);
    if (!ok) break;
    phase_bits ^= 1u << s;
    fence_proxy_async_smem();
    bulk_store(dst + (unsigned long long)j * BULK_SLOT_BYTES, ring + s * BULK_SLOT_BYTES, slot_bytes(j));
    tma_store_commit();
    const int nj = j + BULK_SLOTS - 1;  // reuses the slot read by store j-1
    if (nj < n) {
      tma_store_wait_read<1>();
      issue_load(nj);
    }
  }
  tma_store_wait<0>();  // all writes of this chunk performed before the flag is published
  if (!ok) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // let a stray in-flight load land
  }
  return ok;
}

__global__ void __launch_bounds__(1024) put_chunks_kernel(const FlPutArgs a) {
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  __shared__ uint64_t bars[BULK_SLOTS];
  __shared__ int abort_flag;
  __shared__ int wait_ok;
  uint32_t phase_bits = 0;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    if (a.use_bulk) {
      for (int s = 0; s < BULK_SLOTS; ++s) mbar_init(&bars[s], 1);
      mbar_fence_init();
    }
  }
  __syncthreads();

  unsigned long long chunks_before = 0;
  bool live = true;
  for (int si = 0; si < a.nseg && live; ++si) {
    const FlSeg& sg = a.seg[si];
    const unsigned long long nch = (sg.bytes + a.chunk_bytes - 1) / a.chunk_bytes;
    unsigned long long done_here = 0;      // thread 0: bytes of this segment this CTA has finished
    // CTAs take chunks round-robin over the concatenation of all segments
    unsigned long long first = (blockIdx.x + gridDim.x - (chunks_before % gridDim.x)) % gridDim.x;
    for (unsigned long long c = first; c < nch && live; c += gridDim.x) {
      const unsigned long long off = c * a.chunk_bytes;
      const unsigned long long len = (sg.bytes - off) < a.chunk_bytes ? (sg.bytes - off) : a.chunk_bytes;
      if (sg.wait_flags) {
        if (threadIdx.x == 0) wait_ok = wait_flag_ge(sg.wait_flags + c, a.seq, a.status, 600 + si) ? 1 : 0;
        __syncthreads();
        const int okv = wait_ok;
        __syncthreads();
        if (!okv) { live = false; break; }
      }
      const uint8_t* s = reinterpret_cast<const uint8_t*>(sg.src) + off;
      uint8_t* d = reinterpret_cast<uint8_t*>(sg.dst) + off;
      const bool bulk_ok = a.use_bulk && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d) | len) & 15) == 0;
      if (bulk_ok) {
        if (threadIdx.x == 0) {
          if (!copy_bulk(s, d, len, dyn_smem, bars, phase_bits, &abort_flag, a.status)) abort_flag = 1;
          fence_proxy_async_all();
        }
      } else {
        copy_vec(s, d, len);
      }
      __syncthreads();
      if (abort_flag) { live = false; break; }
      // The flag update is itself a release at system scope: it orders this thread's bulk stores (complete, see
      // copy_bulk) and, through the barrier above, the other threads' stores before the flag becomes visible.
      if (threadIdx.x == 0 && sg.flag_mode != FL_FLAG_NONE) {
        if (sg.flag_mode == FL_FLAG_SEQ_PER_CHUNK) st_release_sys(sg.flags + c, a.seq);
        else red_release_sys_add(sg.flags, 1u);
      }
      // device-side completion counter: the host monitor folds it into the path's completed bytes
      if (threadIdx.x == 0 && sg.bytes_done != nullptr) {
        if (a.done_scratch != nullptr) done_here += len;
        else atomicAdd_system(sg.bytes_done, (unsigned long long)len);
      }
    }
    if (threadIdx.x == 0 && done_here != 0) atomicAdd(a.done_scratch + si, done_here);
    chunks_before += nch;
  }
  if (a.done_scratch != nullptr && threadIdx.x == 0) {
    // every CTA takes a ticket, also one that gave up a wait; the last one forwards the totals and rearms the words
    __threadfence();
    const unsigned long long ticket = atomicAdd(a.done_scratch + FL_MAX_SEGS, 1ull);
    if (ticket == (unsigned long long)gridDim.x - 1) {
      __threadfence();
      for (int si = 0; si < a.nseg; ++si) {
        const unsigned long long total = atomicExch(a.done_scratch + si, 0ull);
        if (total != 0 && a.seg[si].bytes_done != nullptr) atomicAdd_system(a.seg[si].bytes_done, total);
      }
      atomicExch(a.done_scratch + FL_MAX_SEGS, 0ull);
    }
  }
  if (!live) return;
  if (blockIdx.x == 0 && (int)threadIdx.x < a.nwait)
    wait_flag_ge(a.wait_flag[threadIdx.x], a.wait_want[threadIdx.x], a.status, 650 + threadIdx.x);
}

__global__ void wait_flags_kernel(const FlWaitArgs a) {
  const int i = threadIdx.x;
  if (i < a.n) wait_flag_ge(a.flag[i], a.want[i], a.status, 700 + i, a.limit_ns ? a.limit_ns : (uint64_t)FL_FLAG_WAIT_NS);
}

__global__ void barrier_kernel(FlSignalPtrs pads, int slot0, int rank, int world, unsigned int seq, int do_signal,
                               int do_wait, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  if (do_signal) {
    fence_sys();
    st_release_sys(pads.p[r] + slot0 + rank, seq);
  }
  if (do_wait) wait_flag_ge(pads.p[rank] + slot0 + r, seq, status, 800 + r);
}

}  // namespace fl

extern "C" int fl_put_chunks(const FlPutArgs* args, int num_ctas, int threads, cudaStream_t stream) {
  if (args->nseg < 1 || args->nseg > FL_MAX_SEGS) return -1;
  if (args->chunk_bytes == 0 || (args->chunk_bytes & 15)) return -2;
  if (threads <= 0 || threads > 1024) threads = 512;
  if (num_ctas <= 0) num_ctas = 1;
  size_t smem = args->use_bulk ? fl::BULK_SLOTS * fl::BULK_SLOT_BYTES : 0;
  if (smem > 48 * 1024) {
    static bool set_on[64];                 // per device: a process may drive several GPUs
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return -3;
    if (!set_on[dev]) {
      cudaError_t e = cudaFuncSetAttribute(fl::put_chunks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set_on[dev] = true;
    }
  }
  fl::put_chunks_kernel<<<num_ctas, threads, smem, stream>>>(*args);
  return (int)cudaGetLastError();
}

extern "C" int fl_all_to_all(const void* send, void* const* recv_peers, unsigned long long bytes_per_peer, int rank,
                             int world, FlSignalPtrs pads, int slot0, unsigned int chunk_bytes, const unsigned int* want,
                             int use_bulk, int num_ctas, int threads, int* status, cudaStream_t stream) {
  if (world < 1 || world > FL_MAX_SEGS) return -1;
  FlPutArgs a;
  memset(&a, 0, sizeof a);
  a.nseg = world;
  for (int k = 0; k < world; ++k) {
    const int p = (rank + k) % world;   // own block first, then walk the ring so peers are hit evenly
    a.seg[k].src = reinterpret_cast<const uint8_t*>(send) + (unsigned long long)p * bytes_per_peer;
    a.seg[k].dst = reinterpret_cast<uint8_t*>(recv_peers[p]) + (unsigned long long)rank * bytes_per_peer;
    a.seg[k].bytes = bytes_per_peer;
    a.seg[k].flags = pads.p[p] + slot0 + rank;
    a.seg[k].flag_mode = FL_FLAG_COUNT;
  }
  a.chunk_bytes = chunk_bytes;
  a.use_bulk = use_bulk;
  a.status = status;
  if (want) {
    a.nwait = world;
    for (int r = 0; r < world; ++r) {
      a.wait_flag[r] = pads.p[rank] + slot0 + r;
      a.wait_want[r] = want[r];
    }
  }
  return fl_put_chunks(&a, num_ctas, threads, stream);
}

extern "C" int fl_wait_flags(const FlWaitArgs* args, cudaStream_t stream) {
  if (args->n < 0 || args->n > 16) return -1;
  if (args->n == 0) return 0;
  fl::wait_flags_kernel<<<1, 32, 0, stream>>>(*args);
  return (int)cudaGetLastError();
}

extern "C" int fl_barrier(FlSignalPtrs pads, int slot0, int rank, int world, unsigned int seq, int do_signal,
                          int do_wait, int* status, cudaStream_t stream) {
  if (world < 1 || world > 8) return -1;
  fl::barrier_kernel<<<1, 32, 0, stream>>>(pads, slot0, rank, world, seq, do_signal, do_wait, status);
  return (int)cudaGetLastError();
}
