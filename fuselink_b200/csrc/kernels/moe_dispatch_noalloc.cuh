// fl_moe_dispatch_noalloc: the forward MoE dispatch (count -> reserve -> scatter, see moe_dispatch.cuh) for
// callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library.
//
// Who cannot allocate: code that runs on a communication library's proxy/progress thread or inside one
// of its callbacks (cudaMalloc and cudaFree may synchronise the whole device and can then wait on the very
// kernels the thread is supposed to drive forward); a plugin living in a process whose framework has
// already handed all device memory to its own caching allocator; and a serving loop that has a hard
// latency bound per step and cannot absorb an allocation's jitter.  For them the three scratch arrays the
// dispatch kernels need (per-expert counters, per-expert base rows, per-(token,k) positions) live in one
// fixed array that is part of the library image instead of being passed in.
//
// Limits: tokens * topk <= FL_NOALLOC_MAX_ASSIGNMENTS and num_experts <= FL_NOALLOC_MAX_EXPERTS; larger
// problems are rejected with FL_NOALLOC_E_TOO_LARGE and nothing is launched.  The scratch array
// (FL_NOALLOC_SCRATCH_BYTES, about 0.5 MiB) is held by every GPU that loads the library until the process
// exits.
//
// Set-up: fl_moe_dispatch_noalloc_setup(), once per device with that device current, from a thread that may
// synchronise the device: it resolves the device address of the scratch array and makes the runtime load the
// kernels (loading a module can allocate and synchronise -- exactly what the callers above cannot afford later).
// Without it the first fl_moe_dispatch_noalloc call on a device does the same work itself; make that first
// call, or the set-up call, outside any stream capture.  After set-up a call enqueues three kernels and
// touches no allocator.
//
// Sharing: every call on a device uses the same scratch array.  The counters are cleared at the start of
// each call, so calls may follow one another on one stream, or on several streams if the caller orders
// them; two calls whose kernels overlap on the GPU race on the scratch and corrupt each other's placement.
// The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define FL_NOALLOC_MAX_ASSIGNMENTS (128 * 1024)   // tokens * topk
#define FL_NOALLOC_MAX_EXPERTS 1024
#define FL_NOALLOC_SCRATCH_BYTES (2 * FL_NOALLOC_MAX_EXPERTS * 4 + FL_NOALLOC_MAX_ASSIGNMENTS * 4)

#define FL_NOALLOC_E_TOO_LARGE (-100)
#define FL_NOALLOC_E_SETUP (-101)
#define FL_NOALLOC_E_ARGS (-102)       // an argument is out of range; fl_moe_dispatch_noalloc_error() says which

typedef struct {
  const void* x;              // [tokens, hidden] bf16
  const int* topk_idx;        // [tokens, topk] global expert ids
  const float* row_scale;     // optional [tokens, topk]
  int tokens, topk, hidden;
  int num_experts, experts_per_rank, cap;
  int rank, world;
  int* slot;                  // out: [tokens, topk] row inside the owner's expert buffer
  void* count_peers[8];       // every rank's int32 counts[2][experts_per_rank]
  int parity;
  void* x_peers[8];           // every rank's expert input buffer [experts_per_rank * cap, hidden] bf16
  void* info_peers[8];        // every rank's int32 row_info[experts_per_rank * cap]
  int* status;                // device int32[8] or null
} FlMoeDispatchNoAllocArgs;

#ifdef __cplusplus
extern "C" {
#endif
// Returns 0, a negative FL_NOALLOC_E_*, or a positive cudaError.  Nothing is enqueued unless the arguments are accepted.
int fl_moe_dispatch_noalloc(const FlMoeDispatchNoAllocArgs* args, cudaStream_t stream);
// Optional, once per device (see "Set-up" above).  Returns 0, FL_NOALLOC_E_SETUP or a positive cudaError.
int fl_moe_dispatch_noalloc_setup(void);
const char* fl_moe_dispatch_noalloc_error(void);
#ifdef __cplusplus
}
#endif
