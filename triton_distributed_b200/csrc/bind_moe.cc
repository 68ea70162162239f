// Python bindings of the MoE kernels and the grouped GEMM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>

#include "tdb/api.h"
#include "tdb/moe.h"

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

}  // namespace

void bind_moe(py::module_& m) {
  m.def("topk_router", &topk_router);
  m.def("moe_align_sort", &moe_align_sort);
  m.def("moe_tile_arrival_order", &moe_tile_arrival_order);
  m.def("moe_gather", &moe_gather);
  m.def("moe_topk_reduce", &moe_topk_reduce);
  m.def("moe_unsort", &moe_unsort);
  m.def("group_gemm_bf16", &group_gemm_bf16);
}
