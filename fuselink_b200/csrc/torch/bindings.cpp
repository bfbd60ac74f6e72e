// Python bindings (pybind11 through the torch extension headers).  Tensors are passed as torch tensors,
// peer buffers as integer device addresses (they live in other ranks' symmetric regions and have no
// tensor in this process).  Every launcher runs on the current CUDA stream.
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include "../kernels/grouped_gemm.cuh"
#include "../kernels/shadow_reduce.cuh"
#include "../kernels/comm_kernels.cuh"
#include "../kernels/embbag.cuh"
#include "../kernels/kv_pack.cuh"
#include "../kernels/moe_dispatch.cuh"
#include "../kernels/fp8_gemm.cuh"
#include "../mem/vmm.h"
#include "../monitor/monitor.h"
void fl_monitor_bind(pybind11::module& m);

namespace py = pybind11;

static cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

static void check_rc(int rc, const char* what, const char* detail = nullptr) {
  if (rc == 0) return;
  std::string msg = std::string(what) + " failed with code " + std::to_string(rc);
  if (rc > 0) msg += std::string(" (") + cudaGetErrorString((cudaError_t)rc) + ")";
  if (detail && detail[0]) msg += std::string(": ") + detail;
  throw std::runtime_error(msg);
}

static FlPeerPtrs to_peers(const std::vector<int64_t>& v) {
  FlPeerPtrs p;
  memset(&p, 0, sizeof p);
  TORCH_CHECK(v.size() <= FL_MAX_PEERS, "at most 8 peers");
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}
static void* opt_ptr(const c10::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// ------------------------------------------------------------------------------------------------ GEMM
static void grouped_gemm(int64_t group_mode, int64_t num_groups, int64_t cap, int64_t M, int64_t N, int64_t K,
                         c10::optional<torch::Tensor> counts, torch::Tensor A, bool a_mn, int64_t lda, int64_t gsa,
                         torch::Tensor B, bool b_mn, int64_t ldb, int64_t gsb, int64_t epilogue,
                         c10::optional<torch::Tensor> C, int64_t ldc, int64_t gsc, c10::optional<torch::Tensor> gu,
                         int64_t ldgu, c10::optional<torch::Tensor> dgu, c10::optional<torch::Tensor> row_info,
                         std::vector<int64_t> peers, double sgd_lr, bool zero_tail, int64_t group_m, int64_t max_ctas,
                         c10::optional<torch::Tensor> status, int64_t peer_rows) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda(), "grouped_gemm needs CUDA tensors");
  TORCH_CHECK(A.scalar_type() == torch::kBFloat16 && B.scalar_type() == torch::kBFloat16, "bf16 operands expected");
  c10::cuda::CUDAGuard guard(A.device());
  FlGemmDesc d;
  memset(&d, 0, sizeof d);
  d.group_mode = (int)group_mode; d.num_groups = (int)num_groups; d.cap = (int)cap;
  d.M = (int)M; d.N = (int)N; d.K = (int)K;
  d.counts = counts.has_value() ? counts->data_ptr<int>() : nullptr;
  d.elem_bytes = 2;
  d.A = A.data_ptr(); d.a_mn_major = a_mn; d.lda = lda; d.gsa = gsa;
  d.B = B.data_ptr(); d.b_mn_major = b_mn; d.ldb = ldb; d.gsb = gsb;
  d.epilogue = (int)epilogue;
  d.C = opt_ptr(C); d.ldc = ldc; d.gsc = gsc;
  d.gu = opt_ptr(gu); d.ldgu = ldgu; d.dgu = opt_ptr(dgu);
  d.row_info = row_info.has_value() ? row_info->data_ptr<int>() : nullptr;
  d.peers = to_peers(peers); d.num_peers = (int)peers.size(); d.peer_rows = peer_rows;
  d.sgd_lr = (float)sgd_lr; d.zero_tail = zero_tail; d.group_m = (int)group_m; d.max_ctas = (int)max_ctas;
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  check_rc(fl_grouped_gemm(&d, cur_stream()), "fl_grouped_gemm", fl_gemm_last_error());
}

// Weight-gradient GEMM whose result rows go straight to the ranks that sum them (FlGemmDesc::push_world): a: [G*cap, M],
// b: [G*cap, N] token-major, peers: every rank's staging [G][world][M / world][N].
static void grouped_gemm_wgrad_push(int64_t num_groups, int64_t cap, torch::Tensor counts, torch::Tensor A, torch::Tensor B,
                                    std::vector<int64_t> peers, int64_t rank, int64_t block_log2, int64_t group_m,
                                    int64_t max_ctas, c10::optional<torch::Tensor> status) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && counts.is_cuda(), "grouped_gemm_wgrad_push needs CUDA tensors");
  TORCH_CHECK(A.scalar_type() == torch::kBFloat16 && B.scalar_type() == torch::kBFloat16, "bf16 operands expected");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.size(0) == num_groups * cap && B.size(0) == num_groups * cap &&
              A.is_contiguous() && B.is_contiguous(), "a: [G*cap, M], b: [G*cap, N] contiguous");
  c10::cuda::CUDAGuard guard(A.device());
  const int64_t M = A.size(1), N = B.size(1);
  FlGemmDesc d;
  memset(&d, 0, sizeof d);
  d.group_mode = 1; d.num_groups = (int)num_groups; d.cap = (int)cap; d.M = (int)M; d.N = (int)N;
  d.counts = counts.data_ptr<int>(); d.elem_bytes = 2;
  d.A = A.data_ptr(); d.a_mn_major = 1; d.lda = M; d.gsa = cap * M;
  d.B = B.data_ptr(); d.b_mn_major = 1; d.ldb = N; d.gsb = cap * N;
  d.epilogue = FL_EPI_WGRAD; d.ldc = N;
  d.peers = to_peers(peers); d.num_peers = (int)peers.size();
  d.push_world = (int)peers.size(); d.push_rank = (int)rank; d.push_block_log2 = (int)block_log2;
  d.group_m = (int)group_m; d.max_ctas = (int)max_ctas;
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  check_rc(fl_grouped_gemm(&d, cur_stream()), "fl_grouped_gemm", fl_gemm_last_error());
}

// Sum of the staged partial rows over the sources, then w - lr * sum (lr != 0) or the sum itself into every rank's `out`.
static void shadow_update(torch::Tensor part, c10::optional<torch::Tensor> w, std::vector<int64_t> out_peers, int64_t groups,
                          int64_t rank, int64_t M, int64_t N, int64_t block_log2, int64_t group_stride, double lr,
                          int64_t max_ctas) {
  TORCH_CHECK(part.is_cuda() && part.scalar_type() == torch::kBFloat16 && part.is_contiguous(), "staging: contiguous bf16 on the GPU");
  TORCH_CHECK(part.numel() >= groups * M * N, "staging smaller than groups x M x N");
  TORCH_CHECK(lr == 0.0 || (w.has_value() && w->is_cuda() && w->scalar_type() == torch::kBFloat16), "weights: bf16 on the GPU");
  c10::cuda::CUDAGuard guard(part.device());
  FlShadowUpdateArgs a;
  memset(&a, 0, sizeof a);
  a.part = part.data_ptr(); a.w = opt_ptr(w); a.out_peers = to_peers(out_peers);
  a.groups = (int)groups; a.world = (int)out_peers.size(); a.rank = (int)rank; a.M = (int)M; a.N = (int)N;
  a.block_log2 = (int)block_log2; a.group_stride = group_stride; a.lr = (float)lr; a.max_ctas = (int)max_ctas;
  check_rc(fl_shadow_update(&a, cur_stream()), "fl_shadow_update", fl_shadow_update_error());
}

// ------------------------------------------------------------------------------------------------ comm
// segs: list of (src_addr, dst_addr, bytes, flags_addr, flag_mode, wait_flags_addr)
static void put_chunks(const std::vector<std::tuple<int64_t, int64_t, int64_t, int64_t, int64_t, int64_t>>& segs,
                       int64_t chunk_bytes, int64_t seq, bool use_bulk, int64_t num_ctas, int64_t threads,
                       int64_t status_addr, const std::vector<int64_t>& counters, int64_t counter_scratch) {
  FlPutArgs a;
  memset(&a, 0, sizeof a);
  TORCH_CHECK(segs.size() >= 1 && segs.size() <= FL_MAX_SEGS, "1..8 segments per launch");
  a.nseg = (int)segs.size();
  for (size_t i = 0; i < segs.size(); ++i) {
    a.seg[i].src = reinterpret_cast<const void*>(std::get<0>(segs[i]));
    a.seg[i].dst = reinterpret_cast<void*>(std::get<1>(segs[i]));
    a.seg[i].bytes = (unsigned long long)std::get<2>(segs[i]);
    a.seg[i].flags = reinterpret_cast<uint32_t*>(std::get<3>(segs[i]));
    a.seg[i].flag_mode = (int)std::get<4>(segs[i]);
    a.seg[i].wait_flags = reinterpret_cast<const uint32_t*>(std::get<5>(segs[i]));
    a.seg[i].bytes_done = i < counters.size() ? reinterpret_cast<unsigned long long*>(counters[i]) : nullptr;
  }
  a.chunk_bytes = (unsigned)chunk_bytes; a.seq = (unsigned)seq; a.use_bulk = use_bulk;
  a.status = reinterpret_cast<int*>(status_addr);
  a.done_scratch = reinterpret_cast<unsigned long long*>(counter_scratch);
  check_rc(fl_put_chunks(&a, (int)num_ctas, (int)threads, cur_stream()), "fl_put_chunks");
}
static void all_to_all(int64_t send_addr, const std::vector<int64_t>& recv_peers, int64_t bytes_per_peer, int64_t rank,
                       const std::vector<int64_t>& pads, int64_t slot0, int64_t chunk_bytes,
                       const std::vector<int64_t>& want, bool use_bulk, int64_t num_ctas, int64_t threads, int64_t status_addr) {
  const int world = (int)recv_peers.size();
  TORCH_CHECK(world >= 1 && world <= 8 && (int)pads.size() == world, "1..8 ranks");
  void* rp[8];
  FlSignalPtrs sp;
  memset(&sp, 0, sizeof sp);
  unsigned int w[8];
  for (int i = 0; i < world; ++i) {
    rp[i] = reinterpret_cast<void*>(recv_peers[i]);
    sp.p[i] = reinterpret_cast<uint32_t*>(pads[i]);
    if (!want.empty()) w[i] = (unsigned)want[i];
  }
  check_rc(fl_all_to_all(reinterpret_cast<const void*>(send_addr), rp, (unsigned long long)bytes_per_peer, (int)rank, world, sp,
                         (int)slot0, (unsigned)chunk_bytes, want.empty() ? nullptr : w, use_bulk, (int)num_ctas, (int)threads,
                         reinterpret_cast<int*>(status_addr), cur_stream()), "fl_all_to_all");
}
static void wait_flags(const std::vector<std::pair<int64_t, int64_t>>& flags, int64_t status_addr, int64_t limit_ms) {
  FlWaitArgs a;
  memset(&a, 0, sizeof a);
  TORCH_CHECK(flags.size() <= 16, "at most 16 flags per wait");
  a.n = (int)flags.size();
  for (size_t i = 0; i < flags.size(); ++i) {
    a.flag[i] = reinterpret_cast<const uint32_t*>(flags[i].first);
    a.want[i] = (unsigned)flags[i].second;
  }
  a.status = reinterpret_cast<int*>(status_addr);
  a.limit_ns = limit_ms > 0 ? (unsigned long long)limit_ms * 1000000ull : 0ull;
  check_rc(fl_wait_flags(&a, cur_stream()), "fl_wait_flags");
}
static void barrier(const std::vector<int64_t>& pads, int64_t slot0, int64_t rank, int64_t world, int64_t seq,
                    bool do_signal, bool do_wait, int64_t status_addr) {
  FlSignalPtrs p;
  memset(&p, 0, sizeof p);
  for (size_t i = 0; i < pads.size() && i < 8; ++i) p.p[i] = reinterpret_cast<uint32_t*>(pads[i]);
  check_rc(fl_barrier(p, (int)slot0, (int)rank, (int)world, (unsigned)seq, do_signal, do_wait,
                      reinterpret_cast<int*>(status_addr), cur_stream()), "fl_barrier");
}

// ------------------------------------------------------------------------------------------------ DLRM
static void embbag(bool backward, torch::Tensor weights, torch::Tensor indices, int64_t t_first, int64_t t_total,
                   int64_t b_local, std::vector<int64_t> peers, double lr, int64_t num_ctas, int64_t status_addr) {
  TORCH_CHECK(weights.is_cuda() && indices.is_cuda(), "CUDA tensors expected");
  TORCH_CHECK(weights.scalar_type() == torch::kFloat32 && weights.dim() == 3 && weights.is_contiguous(), "weights: [T_local, rows, dim] fp32");
  TORCH_CHECK(indices.scalar_type() == torch::kInt64 && indices.dim() == 3 && indices.is_contiguous(), "indices: [T_local, B_global, pooling] int64");
  c10::cuda::CUDAGuard guard(weights.device());
  FlEmbBagArgs a;
  memset(&a, 0, sizeof a);
  a.weights = weights.data_ptr<float>(); a.weights_rw = weights.data_ptr<float>();
  a.indices = reinterpret_cast<const long long*>(indices.data_ptr<int64_t>());
  a.t_local = (int)weights.size(0); a.rows = weights.size(1); a.dim = (int)weights.size(2);
  TORCH_CHECK(indices.size(0) == weights.size(0), "indices/weights table count mismatch");
  a.b_global = (int)indices.size(1); a.pooling = (int)indices.size(2);
  a.t_first = (int)t_first; a.t_total = (int)t_total; a.b_local = (int)b_local;
  a.out_peers = to_peers(peers); a.lr = (float)lr; a.status = reinterpret_cast<int*>(status_addr);
  if (backward) check_rc(fl_embbag_a2a_bwd_sgd(&a, (int)num_ctas, cur_stream()), "fl_embbag_a2a_bwd_sgd");
  else check_rc(fl_embbag_a2a_fwd(&a, (int)num_ctas, cur_stream()), "fl_embbag_a2a_fwd");
}

// ------------------------------------------------------------------------------------------------ KV
static void kv_pack_send(torch::Tensor src_k, torch::Tensor src_v, int64_t dst_k, int64_t dst_v, int64_t src_layout,
                         int64_t dst_layout, int64_t src_num_blocks, int64_t dst_num_blocks, int64_t layers,
                         int64_t heads, int64_t block_size, int64_t head_dim, int64_t layer_begin, int64_t layer_end,
                         torch::Tensor src_bt, torch::Tensor dst_bt, torch::Tensor nblocks,
                         c10::optional<torch::Tensor> hdr, int64_t hdr_dst, int64_t done_flag, int64_t seq,
                         torch::Tensor cta_counter, int64_t num_ctas, int64_t status_addr) {
  TORCH_CHECK(src_k.is_cuda() && src_v.is_cuda(), "CUDA tensors expected");
  TORCH_CHECK(src_bt.scalar_type() == torch::kInt32 && dst_bt.scalar_type() == torch::kInt32 && nblocks.scalar_type() == torch::kInt32,
              "block tables are int32");
  c10::cuda::CUDAGuard guard(src_k.device());
  FlKvSendArgs a;
  memset(&a, 0, sizeof a);
  a.src_k = src_k.data_ptr(); a.src_v = src_v.data_ptr();
  a.dst_k = reinterpret_cast<void*>(dst_k); a.dst_v = reinterpret_cast<void*>(dst_v);
  a.src_layout = (int)src_layout; a.dst_layout = (int)dst_layout;
  a.src_num_blocks = (int)src_num_blocks; a.dst_num_blocks = (int)dst_num_blocks;
  a.layers = (int)layers; a.heads = (int)heads; a.block_size = (int)block_size; a.head_dim = (int)head_dim;
  a.layer_begin = (int)layer_begin; a.layer_end = (int)layer_end;
  a.src_block_table = src_bt.data_ptr<int>(); a.dst_block_table = dst_bt.data_ptr<int>();
  a.num_blocks = nblocks.data_ptr<int>();
  a.batch = (int)src_bt.size(0); a.max_blocks = (int)src_bt.size(1);
  if (hdr.has_value()) {
    a.hdr_src = hdr->data_ptr(); a.hdr_bytes = (int)hdr->nbytes();
    a.hdr_dst = reinterpret_cast<void*>(hdr_dst);
  }
  a.done_flag = reinterpret_cast<uint32_t*>(done_flag); a.seq = (unsigned)seq;
  a.cta_counter = reinterpret_cast<unsigned*>(cta_counter.data_ptr());
  a.status = reinterpret_cast<int*>(status_addr);
  check_rc(fl_kv_pack_send(&a, (int)num_ctas, cur_stream()), "fl_kv_pack_send");
}

// ------------------------------------------------------------------------------------------------ MoE
static void moe_dispatch(torch::Tensor x, torch::Tensor topk_idx, c10::optional<torch::Tensor> row_scale,
                         int64_t num_experts, int64_t experts_per_rank, int64_t cap, int64_t rank, int64_t world,
                         torch::Tensor local_count, torch::Tensor base, torch::Tensor pos, torch::Tensor slot,
                         std::vector<int64_t> count_peers, int64_t parity, std::vector<int64_t> x_peers,
                         std::vector<int64_t> info_peers, bool reuse_slots, int64_t status_addr) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: [tokens, hidden] bf16");
  TORCH_CHECK(topk_idx.scalar_type() == torch::kInt32 && topk_idx.is_contiguous() && topk_idx.dim() == 2, "topk_idx: [tokens, topk] int32");
  c10::cuda::CUDAGuard guard(x.device());
  FlMoeDispatchArgs a;
  memset(&a, 0, sizeof a);
  a.x = x.data_ptr(); a.topk_idx = topk_idx.data_ptr<int>();
  a.row_scale = row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr;
  a.tokens = (int)x.size(0); a.topk = (int)topk_idx.size(1); a.hidden = (int)x.size(1);
  a.num_experts = (int)num_experts; a.experts_per_rank = (int)experts_per_rank; a.cap = (int)cap;
  a.rank = (int)rank; a.world = (int)world;
  a.local_count = local_count.data_ptr<int>(); a.base = base.data_ptr<int>();
  // a spare (zero) element behind the per-expert counters is the ticket that lets counting and reservation share a launch
  a.ticket = local_count.numel() > num_experts ? local_count.data_ptr<int>() + num_experts : nullptr;
  a.pos = pos.data_ptr<int>(); a.slot = slot.data_ptr<int>();
  a.count_peers = to_peers(count_peers); a.parity = (int)parity;
  a.x_peers = to_peers(x_peers); a.info_peers = to_peers(info_peers);
  a.reuse_slots = reuse_slots; a.status = reinterpret_cast<int*>(status_addr);
  check_rc(fl_moe_dispatch(&a, cur_stream()), "fl_moe_dispatch");
}
static void moe_zero_tail(int64_t buf, int64_t counts, int64_t experts_local, int64_t cap, int64_t width) {
  check_rc(fl_moe_zero_tail(reinterpret_cast<void*>(buf), reinterpret_cast<const int*>(counts), (int)experts_local,
                            (int)cap, (int)width, cur_stream()), "fl_moe_zero_tail");
}
static void moe_combine(torch::Tensor slots, c10::optional<torch::Tensor> w, torch::Tensor out, int64_t topk) {
  c10::cuda::CUDAGuard guard(out.device());
  check_rc(fl_moe_combine(slots.data_ptr(), w.has_value() ? w->data_ptr<float>() : nullptr, out.data_ptr(),
                          (int)out.size(0), (int)topk, (int)out.size(1), cur_stream()), "fl_moe_combine");
}
static void moe_combine_dw(torch::Tensor dout, torch::Tensor slots, torch::Tensor dw, int64_t topk) {
  c10::cuda::CUDAGuard guard(dout.device());
  check_rc(fl_moe_combine_dw(dout.data_ptr(), slots.data_ptr(), dw.data_ptr<float>(), (int)dout.size(0), (int)topk,
                             (int)dout.size(1), cur_stream()), "fl_moe_combine_dw");
}

// ------------------------------------------------------------------------------------------------ fp8
static void fp8_quantize_rows(torch::Tensor x, torch::Tensor q, torch::Tensor scale, c10::optional<torch::Tensor> counts,
                              int64_t cap) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: [rows, K] bf16");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(fl_fp8_quantize_rows(x.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), x.size(0), (int)x.size(1),
                                counts.has_value() ? counts->data_ptr<int>() : nullptr, (int)cap, cur_stream()),
           "fl_fp8_quantize_rows");
}
static void fp8_quantize_blocks(torch::Tensor w, torch::Tensor q, torch::Tensor scale) {
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.dim() == 3, "w: [G, R, C] bf16");
  c10::cuda::CUDAGuard guard(w.device());
  check_rc(fl_fp8_quantize_blocks(w.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), (int)w.size(0), (int)w.size(1),
                                  (int)w.size(2), cur_stream()), "fl_fp8_quantize_blocks");
}
static void fp8_grouped_gemm(int64_t num_groups, int64_t cap, int64_t N, int64_t K, c10::optional<torch::Tensor> counts,
                             torch::Tensor A, torch::Tensor a_scale, torch::Tensor B, bool b_mn, torch::Tensor b_scale,
                             int64_t epilogue, c10::optional<torch::Tensor> C, int64_t ldc, c10::optional<torch::Tensor> gu,
                             int64_t ldgu, c10::optional<torch::Tensor> dgu, c10::optional<torch::Tensor> row_info,
                             std::vector<int64_t> peers, bool zero_tail, int64_t group_m, int64_t max_ctas,
                             c10::optional<torch::Tensor> status, int64_t peer_rows) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && A.element_size() == 1 && B.element_size() == 1, "fp8 operands expected");
  c10::cuda::CUDAGuard guard(A.device());
  FlFp8GemmDesc d;
  memset(&d, 0, sizeof d);
  d.num_groups = (int)num_groups; d.cap = (int)cap; d.N = (int)N; d.K = (int)K;
  d.counts = counts.has_value() ? counts->data_ptr<int>() : nullptr;
  d.A = A.data_ptr(); d.a_scale = a_scale.data_ptr<float>();
  d.B = B.data_ptr(); d.b_mn_major = b_mn; d.b_scale = b_scale.data_ptr<float>();
  d.epilogue = (int)epilogue; d.C = opt_ptr(C); d.ldc = ldc; d.gu = opt_ptr(gu); d.ldgu = ldgu; d.dgu = opt_ptr(dgu);
  d.row_info = row_info.has_value() ? row_info->data_ptr<int>() : nullptr;
  d.peers = to_peers(peers); d.num_peers = (int)peers.size(); d.peer_rows = peer_rows;
  d.zero_tail = zero_tail; d.group_m = (int)group_m; d.max_ctas = (int)max_ctas;
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  check_rc(fl_fp8_grouped_gemm(&d, cur_stream()), "fl_fp8_grouped_gemm", fl_fp8_last_error());
}

// ------------------------------------------------------------------------------------------------ memory
static torch::Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, py::object dtype, int64_t device) {
  auto st = torch::python::detail::py_object_to_dtype(dtype);
  auto opts = torch::TensorOptions().dtype(st).device(device < 0 ? torch::Device(torch::kCPU) : torch::Device(torch::kCUDA, (c10::DeviceIndex)device));
  return torch::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}

static int64_t vmm_create(int64_t device, int64_t size, int64_t slab_bytes) {
  FlVmmRegion* r = fl_vmm_create((int)device, (size_t)size, (size_t)slab_bytes);
  if (!r) throw std::runtime_error(std::string("fl_vmm_create: ") + fl_vmm_last_error());
  return reinterpret_cast<int64_t>(r);
}
static int64_t vmm_import(int64_t device, std::vector<int> fds, int64_t slab_bytes) {
  FlVmmRegion* r = fl_vmm_import((int)device, fds.data(), (int)fds.size(), (size_t)slab_bytes);
  if (!r) throw std::runtime_error(std::string("fl_vmm_import: ") + fl_vmm_last_error());
  return reinterpret_cast<int64_t>(r);
}
static int64_t vmm_alias(int64_t region, int64_t device) {
  FlVmmRegion* r = fl_vmm_alias(reinterpret_cast<FlVmmRegion*>(region), (int)device);
  if (!r) throw std::runtime_error(std::string("fl_vmm_alias: ") + fl_vmm_last_error());
  return reinterpret_cast<int64_t>(r);
}
static int64_t vmm_adopt(int64_t ptr, int64_t size, int64_t device) {
  FlVmmRegion* r = fl_vmm_adopt(reinterpret_cast<void*>(ptr), (size_t)size, (int)device);
  if (!r) throw std::runtime_error(std::string("fl_vmm_adopt: ") + fl_vmm_last_error());
  return reinterpret_cast<int64_t>(r);
}
static int vmm_export_fd(int64_t region, int64_t slab) {
  int fd = -1;
  if (fl_vmm_export_fd(reinterpret_cast<FlVmmRegion*>(region), (int)slab, &fd))
    throw std::runtime_error(std::string("fl_vmm_export_fd: ") + fl_vmm_last_error());
  return fd;
}
static int64_t vmm_remap_slab(int64_t region, int64_t slab, int64_t target, bool keep, std::vector<int> access) {
  long usec = 0;
  if (fl_vmm_remap_slab(reinterpret_cast<FlVmmRegion*>(region), (int)slab, (int)target, keep, access.data(),
                        (int)access.size(), &usec))
    throw std::runtime_error(std::string("fl_vmm_remap_slab: ") + fl_vmm_last_error());
  return usec;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("grouped_gemm", &grouped_gemm);
  m.def("grouped_gemm_wgrad_push", &grouped_gemm_wgrad_push);
  m.def("shadow_update", &shadow_update);
  m.def("gemm_set_variant", [](int64_t v) { fl_gemm_set_variant((int)v); });
  m.def("gemm_get_variant", []() { return fl_gemm_get_variant(); });
  m.def("fp8_quantize_rows", &fp8_quantize_rows);
  m.def("fp8_quantize_blocks", &fp8_quantize_blocks);
  m.def("fp8_grouped_gemm", &fp8_grouped_gemm);
  m.def("put_chunks", &put_chunks, py::arg("segs"), py::arg("chunk_bytes"), py::arg("seq"), py::arg("use_bulk"), py::arg("num_ctas"),
        py::arg("threads"), py::arg("status_addr"), py::arg("counters") = std::vector<int64_t>(), py::arg("counter_scratch") = 0);
  m.def("wait_flags", &wait_flags, py::arg("flags"), py::arg("status_addr"), py::arg("limit_ms") = 0);
  m.def("all_to_all", &all_to_all);
  m.def("barrier", &barrier);
  m.def("embbag", &embbag);
  m.def("kv_pack_send", &kv_pack_send);
  m.def("moe_dispatch", &moe_dispatch);
  m.def("moe_zero_tail", &moe_zero_tail);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_dw", &moe_combine_dw);
  m.def("tensor_from_ptr", &tensor_from_ptr);

  m.def("vmm_init", [](int64_t backend) {
    if (fl_vmm_init((int)backend)) throw std::runtime_error(std::string("fl_vmm_init: ") + fl_vmm_last_error());
  });
  m.def("vmm_backend", []() { return fl_vmm_backend(); });
  m.def("vmm_granularity", [](int64_t dev) {
    size_t g = 0;
    if (fl_vmm_granularity((int)dev, &g)) throw std::runtime_error(std::string("fl_vmm_granularity: ") + fl_vmm_last_error());
    return (int64_t)g;
  });
  m.def("vmm_create", &vmm_create);
  m.def("vmm_import", &vmm_import);
  m.def("vmm_alias", &vmm_alias);
  m.def("vmm_adopt", &vmm_adopt);
  m.def("vmm_destroy", [](int64_t r) { fl_vmm_destroy(reinterpret_cast<FlVmmRegion*>(r)); });
  m.def("vmm_ptr", [](int64_t r) { return (int64_t)(uintptr_t)fl_vmm_ptr(reinterpret_cast<FlVmmRegion*>(r)); });
  m.def("vmm_size", [](int64_t r) { return (int64_t)fl_vmm_size(reinterpret_cast<FlVmmRegion*>(r)); });
  m.def("vmm_slab_bytes", [](int64_t r) { return (int64_t)fl_vmm_slab_bytes(reinterpret_cast<FlVmmRegion*>(r)); });
  m.def("vmm_num_slabs", [](int64_t r) { return fl_vmm_num_slabs(reinterpret_cast<FlVmmRegion*>(r)); });
  m.def("vmm_slab_device", [](int64_t r, int64_t s) { return fl_vmm_slab_device(reinterpret_cast<FlVmmRegion*>(r), (int)s); });
  m.def("vmm_export_fd", &vmm_export_fd);
  m.def("vmm_grant", [](int64_t r, int64_t dev) {
    if (fl_vmm_grant(reinterpret_cast<FlVmmRegion*>(r), (int)dev)) throw std::runtime_error(std::string("fl_vmm_grant: ") + fl_vmm_last_error());
  });
  m.def("vmm_remap_slab", &vmm_remap_slab);
  m.def("vmm_dmabuf_fd", [](int64_t p, int64_t size) {
    int fd = -1;
    uint64_t off = 0;
    if (fl_vmm_dmabuf_fd(reinterpret_cast<const void*>(p), (size_t)size, &fd, &off))
      throw std::runtime_error(std::string("fl_vmm_dmabuf_fd: ") + fl_vmm_last_error());
    return std::make_pair(fd, (int64_t)off);
  });
  m.def("vmm_ptr2dev", [](int64_t p) { return fl_vmm_ptr2dev(reinterpret_cast<const void*>(p)); });
  m.def("pool_init", [](int64_t ndev, int64_t slabs, int64_t slab_bytes) {
    if (fl_pool_init((int)ndev, (int)slabs, (size_t)slab_bytes)) throw std::runtime_error(std::string("fl_pool_init: ") + fl_vmm_last_error());
  });
  m.def("pool_shutdown", []() { fl_pool_shutdown(); });
  m.def("pool_free_slabs", [](int64_t dev) { return fl_pool_free_slabs((int)dev); });
  m.def("pool_slab_bytes", []() { return (int64_t)fl_pool_slab_bytes(); });
  m.def("pool_alloc", [](int64_t dev, int64_t size) {
    FlVmmRegion* r = fl_pool_alloc((int)dev, (size_t)size);
    if (!r) throw std::runtime_error(std::string("fl_pool_alloc: ") + fl_vmm_last_error());
    return reinterpret_cast<int64_t>(r);
  });
  m.def("pool_register", [](int64_t ptr, int64_t size, int64_t dev) {
    FlVmmRegion* r = fl_pool_register(reinterpret_cast<void*>(ptr), (size_t)size, (int)dev);
    if (!r) throw std::runtime_error(std::string("fl_pool_register: ") + fl_vmm_last_error());
    return reinterpret_cast<int64_t>(r);
  });
  m.def("pool_remap", [](int64_t r, int64_t slab, int64_t target, bool keep, std::vector<int> access) {
    long usec = 0;
    if (fl_pool_remap(reinterpret_cast<FlVmmRegion*>(r), (int)slab, (int)target, keep, access.data(), (int)access.size(), &usec))
      throw std::runtime_error(std::string("fl_pool_remap: ") + fl_vmm_last_error());
    return (int64_t)usec;
  });
  m.def("pool_release", [](int64_t r) { fl_pool_release(reinterpret_cast<FlVmmRegion*>(r)); });
  m.def("vmm_usage", [](int64_t dev) { return (int64_t)fl_vmm_usage((int)dev); });

  fl_monitor_bind(m);
}
