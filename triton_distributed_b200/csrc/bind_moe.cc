// Python bindings of the MoE kernels and the grouped GEMM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>

#include "tdb/api.h"
#include "tdb/moe.h"
#include "tdb/symm_heap.h"

namespace py = pybind11;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_cuda(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }
int32_t* i32(at::Tensor& t) { return t.data_ptr<int32_t>(); }

std::vector<at::Tensor> topk_router(const at::Tensor& logits, int64_t k, bool normalize) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous(),
              "topk_router: contiguous fp32 [T, E] expected");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  at::Tensor ids = at::empty({T, k}, logits.options().dtype(at::kInt));
  at::Tensor w = at::empty({T, k}, logits.options());
  check_cuda(tdb::launch_topk_router(logits.data_ptr<float>(), i32(ids), w.data_ptr<float>(), T, E, k, normalize ? 1 : 0,
                                     cur_stream()),
             "launch_topk_router");
  return {ids, w};
}

// Returns {sorted_ids [cap], pos_of [n], tile_expert [cap/align], offsets [E+1], meta [2]} with cap = n + E*(align-1)
// rounded up to `align`.
std::vector<at::Tensor> moe_align_sort(const at::Tensor& ids, int64_t E, int64_t align) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kInt && ids.is_contiguous(), "moe_align_sort: contiguous int32 ids");
  c10::cuda::CUDAGuard guard(ids.device());
  const int64_t n = ids.numel();
  int64_t cap = n + E * (align - 1);
  cap = (cap + align - 1) / align * align;
  if (cap == 0) cap = align;
  auto o = ids.options();
  at::Tensor counts = at::empty({E}, o), offsets = at::empty({E + 1}, o), cursor = at::empty({E}, o);
  at::Tensor sorted_ids = at::empty({cap}, o), pos_of = at::empty({std::max<int64_t>(n, 1)}, o);
  at::Tensor tile_expert = at::empty({cap / align}, o), meta = at::empty({2}, o);
  at::Tensor idsc = ids.reshape({-1});
  check_cuda(tdb::launch_moe_align_sort(idsc.data_ptr<int32_t>(), n, E, align, i32(counts), i32(offsets), i32(cursor),
                                        i32(sorted_ids), cap, i32(pos_of), i32(tile_expert), cap / align, i32(meta),
                                        cur_stream()),
             "launch_moe_align_sort");
  return {sorted_ids, pos_of, tile_expert, offsets, meta, counts};
}

at::Tensor moe_gather(const at::Tensor& src, const at::Tensor& sorted_ids, const at::Tensor& meta, int64_t k) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.dim() == 2 && src.stride(1) == 1,
              "moe_gather: bf16 [T, H] expected");
  c10::cuda::CUDAGuard guard(src.device());
  const int64_t cap = sorted_ids.numel(), H = src.size(1);
  at::Tensor out = at::empty({cap, H}, src.options());
  check_cuda(tdb::launch_moe_gather(src.data_ptr(), sorted_ids.data_ptr<int32_t>(), meta.data_ptr<int32_t>(), out.data_ptr(),
                                    cap, H, k, src.stride(0), cur_stream()),
             "launch_moe_gather");
  return out;
}

at::Tensor moe_topk_reduce(const at::Tensor& y, const at::Tensor& pos_of, c10::optional<at::Tensor> w, int64_t T, int64_t k) {
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.is_contiguous(), "moe_topk_reduce: bf16 y");
  c10::cuda::CUDAGuard guard(y.device());
  const int64_t H = y.size(1);
  at::Tensor out = at::empty({T, H}, y.options());
  const float* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == T * k, "moe_topk_reduce: fp32 [T,k] weights");
    wp = w->data_ptr<float>();
  }
  check_cuda(tdb::launch_moe_topk_reduce(y.data_ptr(), pos_of.data_ptr<int32_t>(), wp, out.data_ptr(), T, H, k, H, cur_stream()),
             "launch_moe_topk_reduce");
  return out;
}

at::Tensor moe_unsort(const at::Tensor& y, const at::Tensor& pos_of, int64_t rows) {
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.is_contiguous(), "moe_unsort: bf16 y");
  c10::cuda::CUDAGuard guard(y.device());
  at::Tensor out = at::empty({rows, y.size(1)}, y.options());
  check_cuda(tdb::launch_moe_unsort(y.data_ptr(), pos_of.data_ptr<int32_t>(), out.data_ptr(), rows, y.size(1), cur_stream()),
             "launch_moe_unsort");
  return out;
}

// Grouped GEMM over rows sorted by expert: out[r, :] = a[r, :] @ b[tile_expert[r / 128]]^T.
// a [rows (multiple of 128), K] bf16; b [E, N, K] bf16; tile_expert int32 [rows / 128] (< 0 = skip).
void group_gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, const at::Tensor& tile_expert, int block_n,
                     int num_ctas) {
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16,
              "group_gemm: bf16 expected");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3 && a.is_contiguous() && b.is_contiguous() && out.is_contiguous(),
              "group_gemm: a [rows, K], b [E, N, K], contiguous");
  const int64_t M = a.size(0), K = a.size(1), E = b.size(0), N = b.size(1);
  TORCH_CHECK(b.size(2) == K && out.size(0) == M && out.size(1) == N && M % 128 == 0, "group_gemm: shape mismatch");
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.numel() >= M / 128, "group_gemm: tile_expert too small");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "group_gemm: K and N must be multiples of 8");
  if (M == 0) return;
  c10::cuda::CUDAGuard guard(a.device());
  tdb::GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmPlain;
  g.M = M; g.N = N; g.K = K;
  g.c = out.data_ptr();
  g.ldc = N;
  g.block_n = (block_n == 128 || block_n == 256) ? block_n : (N <= 128 ? 128 : 256);
  int r = tdb::encode_tensor_map_3d(&g.tmap_a, a.data_ptr(), tdb::kBF16, 1, M, K, K * 2, static_cast<uint64_t>(M) * K * 2, 128, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (a) failed: ", r);
  r = tdb::encode_tensor_map_3d(&g.tmap_b, b.data_ptr(), tdb::kBF16, E, N, K, K * 2, static_cast<uint64_t>(N) * K * 2, g.block_n, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (b) failed: ", r);
  r = tdb::encode_tensor_map_3d(&g.tmap_c, out.data_ptr(), tdb::kBF16, 1, M, N, N * 2, static_cast<uint64_t>(M) * N * 2, 128, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (c) failed: ", r);
  g.use_tma_store = 1;
  g.tile_expert = tile_expert.data_ptr<int32_t>();
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int64_t tiles = (M / 128) * ((N + g.block_n - 1) / g.block_n);
  g.num_ctas = static_cast<int>(std::min<int64_t>(num_ctas > 0 ? num_ctas : sms, tiles));
  g.symm.world = 1;
  g.symm.timeout_ns = 2000000000ull;
  check_cuda(tdb::launch_gemm(g, cur_stream()), "launch_gemm(grouped)");
}

// (order, stage) of the tiles of an expert-sorted layout for the AG -> grouped-GEMM overlap (host computation)
std::vector<at::Tensor> moe_tile_arrival_order(const at::Tensor& sorted_ids, int64_t topk, int64_t tokens_per_rank, int64_t rank,
                                               int64_t world, int64_t block) {
  at::Tensor ids = sorted_ids.to(at::kCPU, at::kInt).contiguous();
  std::vector<int32_t> order, stage;
  tdb::moe_tile_arrival_order(ids.data_ptr<int32_t>(), ids.numel(), topk, tokens_per_rank, rank, world, block, &order, &stage);
  at::Tensor o = at::empty({static_cast<int64_t>(order.size())}, at::kInt), st = at::empty({static_cast<int64_t>(stage.size())}, at::kInt);
  std::memcpy(o.data_ptr(), order.data(), order.size() * sizeof(int32_t));
  std::memcpy(st.data_ptr(), stage.data(), stage.size() * sizeof(int32_t));
  return {o, st};
}

// Staged variant of moe_align_sort: inside an expert the rows are ordered by the ring distance of their token's source
// rank.  Returns {sorted_ids, pos_of, tile_expert, offsets, meta, counts}.
std::vector<at::Tensor> moe_align_sort_staged(const at::Tensor& ids, int64_t E, int64_t align, int64_t topk,
                                              int64_t tokens_per_rank, int64_t rank, int64_t world) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kInt && ids.is_contiguous(), "moe_align_sort_staged: contiguous int32 ids");
  c10::cuda::CUDAGuard guard(ids.device());
  const int64_t n = ids.numel();
  int64_t cap = n + E * (align - 1);
  cap = (cap + align - 1) / align * align;
  if (cap == 0) cap = align;
  auto o = ids.options();
  at::Tensor buckets = at::empty({E * world}, o), cursor = at::empty({E * world}, o);
  at::Tensor counts = at::empty({E}, o), offsets = at::empty({E + 1}, o);
  at::Tensor sorted_ids = at::empty({cap}, o), pos_of = at::empty({std::max<int64_t>(n, 1)}, o);
  at::Tensor tile_expert = at::empty({cap / align}, o), meta = at::empty({2}, o);
  at::Tensor idsc = ids.reshape({-1});
  check_cuda(tdb::launch_moe_align_sort_staged(idsc.data_ptr<int32_t>(), n, E, align, topk, tokens_per_rank, rank, world,
                                               i32(buckets), i32(counts), i32(offsets), i32(cursor), i32(sorted_ids), cap,
                                               i32(pos_of), i32(tile_expert), cap / align, i32(meta), cur_stream()),
             "launch_moe_align_sort_staged");
  return {sorted_ids, pos_of, tile_expert, offsets, meta, counts};
}

// Device-side tile schedule: {order [tiles], stage [tiles], bucket_start [world + 2]}.
std::vector<at::Tensor> moe_tile_schedule(const at::Tensor& sorted_ids, int64_t topk, int64_t tokens_per_rank, int64_t rank,
                                          int64_t world, int64_t block) {
  TORCH_CHECK(sorted_ids.is_cuda() && sorted_ids.scalar_type() == at::kInt && sorted_ids.is_contiguous(), "moe_tile_schedule: int32 ids");
  c10::cuda::CUDAGuard guard(sorted_ids.device());
  const int64_t n = sorted_ids.numel(), tiles = (n + block - 1) / block;
  auto o = sorted_ids.options();
  at::Tensor order = at::empty({tiles}, o), stage = at::empty({tiles}, o), bstart = at::empty({world + 2}, o);
  check_cuda(tdb::launch_moe_tile_schedule(sorted_ids.data_ptr<int32_t>(), n, topk, tokens_per_rank, rank, world, block,
                                           i32(stage), i32(order), i32(bstart), cur_stream()),
             "launch_moe_tile_schedule");
  return {order, stage, bstart};
}

void fill_moe_common(tdb::MoeFusedArgs& g, const at::Tensor& x, const at::Tensor& w, const at::Tensor& sorted_ids,
                     const at::Tensor& tile_expert, const c10::optional<at::Tensor>& order, const at::Tensor& meta,
                     at::Tensor& y, int64_t k_top, int64_t a_row_div, bool scatter_out,
                     const c10::optional<at::Tensor>& row_weight, int num_ctas) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "moe_fused: bf16 x [rows, K]");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 3 && w.is_contiguous(), "moe_fused: bf16 w [E, N, K]");
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1, "moe_fused: bf16 y");
  const int64_t K = x.size(1), E = w.size(0), N = w.size(1);
  TORCH_CHECK(w.size(2) == K && y.size(1) == N, "moe_fused: shape mismatch");
  TORCH_CHECK(sorted_ids.scalar_type() == at::kInt && tile_expert.scalar_type() == at::kInt && meta.scalar_type() == at::kInt,
              "moe_fused: int32 index tensors expected");
  TORCH_CHECK(sorted_ids.numel() == tile_expert.numel() * 128, "moe_fused: sorted_ids must hold 128 rows per tile");
  std::memset(&g, 0, sizeof(g));
  g.K = K; g.N = N; g.k_top = k_top;
  g.x = x.data_ptr();
  g.ldx = x.stride(0);
  g.a_row_div = a_row_div;
  g.sorted_ids = sorted_ids.data_ptr<int32_t>();
  g.tile_expert = tile_expert.data_ptr<int32_t>();
  if (order.has_value()) {
    TORCH_CHECK(order->scalar_type() == at::kInt && order->numel() >= tile_expert.numel(), "moe_fused: order too small");
    g.order = order->data_ptr<int32_t>();
  }
  g.meta = meta.data_ptr<int32_t>();
  g.max_tiles = tile_expert.numel();
  int r = tdb::encode_tensor_map_3d(&g.tmap_b, w.data_ptr(), tdb::kBF16, E, N, K, K * 2, static_cast<uint64_t>(N) * K * 2, 256, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (w) failed: ", r);
  g.y = y.data_ptr();
  g.ldy = y.stride(0);
  g.scatter_out = scatter_out ? 1 : 0;
  if (row_weight.has_value()) {
    TORCH_CHECK(row_weight->scalar_type() == at::kFloat && row_weight->is_contiguous(), "moe_fused: fp32 row weights");
    g.row_weight = row_weight->data_ptr<float>();
  }
  g.num_ctas = num_ctas > 0 ? num_ctas : at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  g.symm.world = 1;
  g.symm.timeout_ns = 2000000000ull;
}

// Grouped GEMM with the rows gathered inside the kernel (single GPU): y = x[sorted_ids / a_row_div] @ w[expert]^T.
void moe_group_gemm_gather(const at::Tensor& x, const at::Tensor& w, const at::Tensor& sorted_ids, const at::Tensor& tile_expert,
                           const c10::optional<at::Tensor>& order, const at::Tensor& meta, at::Tensor& y, int64_t k_top,
                           int64_t a_row_div, bool scatter_out, const c10::optional<at::Tensor>& row_weight, int num_ctas) {
  c10::cuda::CUDAGuard guard(x.device());
  tdb::MoeFusedArgs g;
  fill_moe_common(g, x, w, sorted_ids, tile_expert, order, meta, y, k_top, a_row_div, scatter_out, row_weight, num_ctas);
  g.mode = tdb::kMoePlain;
  check_cuda(tdb::launch_moe_fused(g, cur_stream()), "launch_moe_fused(plain)");
}

// All-gather -> grouped GEMM in one launch.  x: local tokens [t_local, K]; ws / flags in the symmetric heap.
void moe_ag_group_gemm(tdb::SymmHeap& h, const at::Tensor& x, const at::Tensor& w, const at::Tensor& sorted_ids,
                       const at::Tensor& tile_expert, const c10::optional<at::Tensor>& order, const at::Tensor& meta,
                       at::Tensor& y, int64_t k_top, bool scatter_out, at::Tensor& ws, at::Tensor& flags, at::Tensor& ctx,
                       int64_t max_t_local, int64_t max_chunks, int n_comm, int num_ctas, double timeout_s) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "moe_ag_group_gemm: contiguous local tokens expected");
  tdb::MoeFusedArgs g;
  fill_moe_common(g, x, w, sorted_ids, tile_expert, order, meta, y, k_top, k_top, scatter_out, c10::nullopt, num_ctas);
  g.mode = tdb::kMoeAllGather;
  g.t_local = x.size(0);
  g.max_t_local = max_t_local;
  g.n_comm = n_comm;
  TORCH_CHECK(static_cast<uint64_t>(ws.numel()) >= 2ull * h.world() * max_t_local * g.K, "moe_ag_group_gemm: workspace too small");
  g.ag_ws = ws.data_ptr();
  g.ag_flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  g.max_chunks = max_chunks;
  g.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  g.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  check_cuda(tdb::launch_moe_fused(g, cur_stream()), "launch_moe_fused(all-gather)");
}

// Grouped GEMM -> routing weight -> top-k reduce -> reduce-scatter (all_reduce = false) or all-reduce, one launch.
// x: [pairs or sorted rows, K]; y_sorted: scratch [cap, N]; out: [T / W, N] or [T, N].
void moe_group_gemm_reduce(tdb::SymmHeap& h, const at::Tensor& x, const at::Tensor& w, const at::Tensor& sorted_ids,
                           const at::Tensor& tile_expert, const at::Tensor& meta, at::Tensor& y_sorted, int64_t k_top,
                           int64_t a_row_div, const c10::optional<at::Tensor>& row_weight, const at::Tensor& pos_of,
                           int64_t T, at::Tensor& chunk_done, at::Tensor& slots, at::Tensor& flags, at::Tensor& ctx,
                           at::Tensor& out, int64_t n_chunks, int64_t n_red, bool all_reduce, int num_ctas, double timeout_s) {
  c10::cuda::CUDAGuard guard(x.device());
  tdb::MoeFusedArgs g;
  fill_moe_common(g, x, w, sorted_ids, tile_expert, c10::nullopt, meta, y_sorted, k_top, a_row_div, false, row_weight, num_ctas);
  const int W = h.world();
  g.mode = all_reduce ? tdb::kMoeReduceAR : tdb::kMoeReduceRS;
  g.n_chunks = n_chunks;
  g.n_red = n_red;
  g.T = T;
  TORCH_CHECK(pos_of.scalar_type() == at::kInt && pos_of.numel() >= T * k_top, "moe_group_gemm_reduce: pos_of too small");
  g.pos_of = pos_of.data_ptr<int32_t>();
  TORCH_CHECK(chunk_done.scalar_type() == at::kInt && chunk_done.numel() >= 2 * n_chunks, "moe_group_gemm_reduce: chunk counters");
  g.chunk_done = reinterpret_cast<uint32_t*>(chunk_done.data_ptr());
  const int64_t slot_rows = all_reduce ? T : T / W;
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == slot_rows && out.size(1) == g.N && out.stride(1) == 1,
              "moe_group_gemm_reduce: output shape");
  TORCH_CHECK(static_cast<uint64_t>(slots.numel()) >= 2ull * W * slot_rows * g.N, "moe_group_gemm_reduce: slot buffer too small");
  TORCH_CHECK(flags.numel() >= 2ll * W * n_chunks * n_red, "moe_group_gemm_reduce: flag buffer too small");
  g.red_slots = slots.data_ptr();
  g.red_slot_elems = static_cast<uint64_t>(slot_rows) * g.N;
  g.red_flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  g.out = out.data_ptr();
  g.ld_out = out.stride(0);
  g.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  g.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  check_cuda(tdb::launch_moe_fused(g, cur_stream()), "launch_moe_fused(reduce)");
}

}  // namespace

void bind_moe(py::module_& m) {
  m.def("moe_align_sort_staged", &moe_align_sort_staged);
  m.def("moe_tile_schedule", &moe_tile_schedule);
  m.def("moe_group_gemm_gather", &moe_group_gemm_gather);
  m.def("moe_ag_group_gemm", &moe_ag_group_gemm);
  m.def("moe_group_gemm_reduce", &moe_group_gemm_reduce);
  m.def("topk_router", &topk_router);
  m.def("moe_align_sort", &moe_align_sort);
  m.def("moe_tile_arrival_order", &moe_tile_arrival_order);
  m.def("moe_gather", &moe_gather);
  m.def("moe_topk_reduce", &moe_topk_reduce);
  m.def("moe_unsort", &moe_unsort);
  m.def("group_gemm_bf16", &group_gemm_bf16);
}
