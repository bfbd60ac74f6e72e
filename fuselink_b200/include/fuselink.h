// C / C++ interface of fuselink_b200: everything exported by lib/libfuselink.so (no Python, no PyTorch needed).
//
//   kernels   grouped GEMM (bf16 and block-scaled fp8), chunked peer copies / all-to-all / flag waits,
//             MoE dispatch + combine, embedding-bag + all-to-all, KV page pack + send,
//             sum + update of replicated experts' weight gradients                         (launch on a cudaStream_t)
//   regions   cuMem regions that can be exported, imported, aliased and re-homed; slab pool  (vmm.h)
//   monitor   lock-free idleness table and path selection                                    (monitor.h)
//
// Build against it with   g++ -I<repo>/fuselink_b200/include -I$CUDA_HOME/include app.cc -L<repo>/fuselink_b200/lib -lfuselink
// The ncclNet plugin is a separate library (lib/libnccl-net-fuselink.so) that NCCL loads by itself.
#pragma once
#include "../csrc/kernels/comm_kernels.cuh"
#include "../csrc/kernels/embbag.cuh"
#include "../csrc/kernels/fp8_gemm.cuh"
#include "../csrc/kernels/grouped_gemm.cuh"
#include "../csrc/kernels/kv_pack.cuh"
#include "../csrc/kernels/moe_dispatch.cuh"
#include "../csrc/kernels/moe_dispatch_noalloc.cuh"
#include "../csrc/kernels/shadow_reduce.cuh"
#include "../csrc/mem/vmm.h"
#include "../csrc/monitor/monitor.h"
