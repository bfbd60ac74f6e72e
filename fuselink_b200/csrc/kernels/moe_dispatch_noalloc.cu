// See moe_dispatch_noalloc.cuh.  The scratch of the dispatch kernels lives in a file-scope device array;
// host code never uses that array's name as an address (in host code the name is only a stand-in for the
// symbol): the device address is looked up once per device with cudaGetSymbolAddress and that pointer is
// what the kernels receive.
#include "moe_dispatch_noalloc.cuh"
#include "moe_dispatch.cuh"
#include <stdio.h>
#include <string.h>
#include <mutex>

static __device__ __align__(256) unsigned char g_dispatch_scratch[FL_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices];   // device address of g_dispatch_scratch on each device, null until set up
std::mutex g_setup_mu;
thread_local char g_err[256] = "";

// Device code may name the array directly: the per-expert counters at its start must be zero when the
// count kernel runs, whatever the previous call left there.
__global__ void clear_counters_kernel(int num_experts) {
  int* counters = reinterpret_cast<int*>(g_dispatch_scratch);
  for (int i = threadIdx.x; i < 2 * num_experts; i += blockDim.x) counters[i] = 0;
}

int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(g_err, sizeof g_err, "device ordinal %d outside the supported range", dev);
    return FL_NOALLOC_E_SETUP;
  }
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_dispatch_scratch);   // with `dev` current: this device's copy of the array
    if (e != cudaSuccess || !p) {
      snprintf(g_err, sizeof g_err, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : FL_NOALLOC_E_SETUP;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" const char* fl_moe_dispatch_noalloc_error(void) { return g_err; }

extern "C" int fl_moe_dispatch_noalloc_setup(void) {
  g_err[0] = 0;
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, clear_counters_kernel);
  if (e == cudaSuccess) e = (cudaError_t)fl_moe_dispatch_preload();
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof g_err, "loading the dispatch kernels failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

extern "C" int fl_moe_dispatch_noalloc(const FlMoeDispatchNoAllocArgs* in, cudaStream_t stream) {
  g_err[0] = 0;
  auto bad = [](int code, const char* why) {
    snprintf(g_err, sizeof g_err, "%s", why);
    return code;
  };
  // everything fl_moe_dispatch would refuse is refused here, before anything is enqueued
  if (!in) return bad(FL_NOALLOC_E_ARGS, "null argument block");
  if (in->tokens < 0 || in->topk < 1 || in->num_experts < 1) return bad(FL_NOALLOC_E_ARGS, "tokens >= 0, topk >= 1 and num_experts >= 1 are required");
  if (in->hidden <= 0 || in->hidden % 8) return bad(FL_NOALLOC_E_ARGS, "hidden must be a positive multiple of 8 (16-byte rows pieces)");
  if (in->world < 1 || in->world > 8 || in->rank < 0 || in->rank >= in->world) return bad(FL_NOALLOC_E_ARGS, "1 <= world <= 8 and 0 <= rank < world are required");
  if (in->experts_per_rank < 1 || (long long)in->experts_per_rank * in->world != in->num_experts)
    return bad(FL_NOALLOC_E_ARGS, "experts_per_rank * world must equal num_experts");
  if (in->cap <= 0) return bad(FL_NOALLOC_E_ARGS, "cap must be positive");
  const long long assignments = (long long)in->tokens * in->topk;
  if (assignments > FL_NOALLOC_MAX_ASSIGNMENTS || in->num_experts > FL_NOALLOC_MAX_EXPERTS) {
    snprintf(g_err, sizeof g_err,
             "problem too large for the built-in scratch: tokens*topk = %lld (max %d), experts = %d (max %d)",
             assignments, FL_NOALLOC_MAX_ASSIGNMENTS, in->num_experts, FL_NOALLOC_MAX_EXPERTS);
    return FL_NOALLOC_E_TOO_LARGE;
  }
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;

  int* counters = reinterpret_cast<int*>(scratch);                     // [FL_NOALLOC_MAX_EXPERTS]
  int* base = counters + FL_NOALLOC_MAX_EXPERTS;                       // [FL_NOALLOC_MAX_EXPERTS]
  int* pos = base + FL_NOALLOC_MAX_EXPERTS;                            // [FL_NOALLOC_MAX_ASSIGNMENTS]

  FlMoeDispatchArgs a;
  memset(&a, 0, sizeof a);
  a.x = in->x; a.topk_idx = in->topk_idx; a.row_scale = in->row_scale;
  a.tokens = in->tokens; a.topk = in->topk; a.hidden = in->hidden;
  a.num_experts = in->num_experts; a.experts_per_rank = in->experts_per_rank; a.cap = in->cap;
  a.rank = in->rank; a.world = in->world;
  a.local_count = counters; a.base = base; a.pos = pos; a.slot = in->slot;
  a.ticket = in->num_experts < FL_NOALLOC_MAX_EXPERTS ? counters + in->num_experts : nullptr;   // cleared with the counters
  for (int i = 0; i < 8; ++i) {
    a.count_peers.p[i] = in->count_peers[i];
    a.x_peers.p[i] = in->x_peers[i];
    a.info_peers.p[i] = in->info_peers[i];
  }
  a.parity = in->parity; a.reuse_slots = 0; a.status = in->status;

  clear_counters_kernel<<<1, 256, 0, stream>>>(FL_NOALLOC_MAX_EXPERTS);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof g_err, "launch failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  rc = fl_moe_dispatch(&a, stream);
  if (rc < 0) snprintf(g_err, sizeof g_err, "fl_moe_dispatch refused the arguments (code %d)", rc);
  else if (rc > 0) snprintf(g_err, sizeof g_err, "launch failed: %s", cudaGetErrorString((cudaError_t)rc));
  return rc < 0 ? FL_NOALLOC_E_ARGS : rc;
}
