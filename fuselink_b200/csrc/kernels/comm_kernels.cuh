// Device-initiated data movement over NVLink / NVSwitch peer mappings: chunked multi-segment put
// (p2p, striped relay send, relay forward, all-to-all), flag waits and a flag barrier.
//
// Synchronisation model (shared by every kernel of this library):
//   * every rank owns a "signal pad" (uint32 words) inside its symmetric region, mapped by all peers;
//   * words are monotone: a producer either stores a sequence number (st.release.sys) or adds 1
//     (red.release.sys) after its data stores; a consumer polls with ld.acquire.sys until the word is
//     >= the value it expects.  Nothing is ever reset, so no reset/reuse races exist;
//   * every poll is bounded (2 s); on expiry the kernel records a code in `status` and returns.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define FL_MAX_SEGS 8

enum FlFlagMode : int {
  FL_FLAG_NONE = 0,
  FL_FLAG_SEQ_PER_CHUNK = 1,  // flags[chunk] = seq          (relay staging: one word per chunk)
  FL_FLAG_COUNT = 2,          // flags[0]   += 1 per chunk   (final destination: arrival counter)
};

struct FlSeg {
  const void* src;            // local or peer address
  void* dst;                  // local or peer address
  unsigned long long bytes;
  uint32_t* flags;            // see FlFlagMode (address in the consumer's signal pad)
  int flag_mode;
  const uint32_t* wait_flags; // if set: chunk c is copied only after wait_flags[c] >= seq (relay forward)
  unsigned long long* bytes_done;  // optional completion counter (mapped pinned host memory read by the monitor thread)
};

struct FlPutArgs {
  FlSeg seg[FL_MAX_SEGS];
  int nseg;
  unsigned int chunk_bytes;   // multiple of 16
  unsigned int seq;
  int use_bulk;               // 1: cp.async.bulk global->smem->global engine, 0: ld/st vectors
  int* status;
  // optional tail: after its own copies CTA 0 waits until wait_flag[i] >= wait_want[i] for i < nwait, so one
  // launch is "my data is on its way AND everybody's data for me has arrived" (multi-GPU only: the peers'
  // kernels run on other GPUs)
  const uint32_t* wait_flag[8];
  unsigned int wait_want[8];
  int nwait;
  // optional, with bytes_done: FL_MAX_SEGS + 1 zeroed 64-bit words of DEVICE memory owned by the caller's channel.  The
  // CTAs add up their finished bytes there and the last CTA of the launch forwards one total per segment to bytes_done, so
  // a launch costs one host-memory atomic per segment instead of one per chunk (each takes about a microsecond over PCIe
  // and they serialise).  Launches that share the words must be stream-ordered.  Null: one host atomic per chunk.
  unsigned long long* done_scratch;
};

struct FlWaitArgs {
  const uint32_t* flag[16];
  unsigned int want[16];
  int n;
  int* status;
  unsigned long long limit_ns;   // 0: the library default (10 s); tests of the timeout path pass a few milliseconds
};

struct FlSignalPtrs {
  uint32_t* p[8];             // p[r] = base of rank r's signal pad as mapped in THIS process
};

#ifdef __cplusplus
extern "C" {
#endif
int fl_put_chunks(const FlPutArgs* args, int num_ctas, int threads, cudaStream_t stream);
int fl_wait_flags(const FlWaitArgs* args, cudaStream_t stream);
// Uniform all-to-all in one launch: block p of `send` ([world, bytes_per_peer]) goes to recv_peers[p] + rank *
// bytes_per_peer; arrival counters live at pads.p[dst][slot0 + src]; with want != NULL the launch also waits
// until the local counters reach want[src] (cumulative chunk counts kept by the caller).
int fl_all_to_all(const void* send, void* const* recv_peers, unsigned long long bytes_per_peer, int rank, int world,
                  FlSignalPtrs pads, int slot0, unsigned int chunk_bytes, const unsigned int* want, int use_bulk,
                  int num_ctas, int threads, int* status, cudaStream_t stream);
// every rank: pads.p[r][slot0 + rank] = seq for all r, then wait pads.p[rank][slot0 + r] >= seq for all r
int fl_barrier(FlSignalPtrs pads, int slot0, int rank, int world, unsigned int seq, int do_signal, int do_wait,
               int* status, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
