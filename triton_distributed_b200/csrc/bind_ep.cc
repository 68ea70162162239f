// Python bindings of the expert-parallel all-to-all kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "tdb/ep.h"
#include "tdb/symm_heap.h"

namespace py = pybind11;
using tdb::SymmHeap;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_cuda(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }
int32_t* i32(const at::Tensor& t) { return reinterpret_cast<int32_t*>(t.data_ptr()); }
tdb::CtxDev* ctxp(const at::Tensor& t) { return reinterpret_cast<tdb::CtxDev*>(t.data_ptr()); }
uint64_t ns(double s) { return static_cast<uint64_t>(s * 1e9); }

void ep_dispatch(SymmHeap& h, const at::Tensor& x, const at::Tensor& topk_ids, int64_t E, bool quant, int64_t max_tokens,
                 at::Tensor& recv_x, at::Tensor& recv_scale, at::Tensor& recv_meta, at::Tensor& recv_count,
                 at::Tensor& flags, int64_t rows_per_parity, c10::optional<at::Tensor> base, at::Tensor& cursor,
                 at::Tensor& sent_row, at::Tensor& ctx, int64_t num_ctas, double timeout_s, int64_t parts) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "ep_dispatch: x bf16 [T,H]");
  TORCH_CHECK(topk_ids.scalar_type() == at::kInt && topk_ids.dim() == 2 && topk_ids.is_contiguous(), "ep_dispatch: int32 ids [T,k]");
  TORCH_CHECK(x.size(0) <= max_tokens, "ep_dispatch: more tokens than the context was created for");
  c10::cuda::CUDAGuard guard(x.device());
  tdb::EpDispatchArgs a;
  a.x = x.data_ptr();
  a.topk_ids = i32(topk_ids);
  a.T = x.size(0); a.H = x.size(1); a.k = topk_ids.size(1); a.E = E;
  a.quant = quant ? 1 : 0;
  a.max_tokens = max_tokens;
  a.recv_x = recv_x.data_ptr();
  a.recv_scale = recv_scale.data_ptr<float>();
  a.recv_meta = i32(recv_meta);
  a.recv_count = i32(recv_count);
  a.flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  a.rows_per_parity = rows_per_parity;
  a.base = base.has_value() ? i32(*base) : nullptr;
  a.cursor = i32(cursor);
  a.sent_row = i32(sent_row);
  a.num_ctas = num_ctas;
  a.parts = parts;
  a.ctx = ctxp(ctx);
  a.symm = h.info(ns(timeout_s));
  check_cuda(tdb::launch_ep_dispatch(a, cur_stream()), "launch_ep_dispatch");
}

void ep_count(const at::Tensor& ids, int64_t E, at::Tensor& counts) {
  check_cuda(tdb::launch_ep_count(i32(ids), ids.numel(), E, i32(counts), cur_stream()), "launch_ep_count");
}
void ep_layout(const at::Tensor& counts_all, at::Tensor& base, int64_t epr, int64_t W, int64_t E) {
  check_cuda(tdb::launch_ep_layout(i32(counts_all), i32(base), epr, W, E, cur_stream()), "launch_ep_layout");
}
void ep_recv_ids(const at::Tensor& recv_count, c10::optional<at::Tensor> base_self, at::Tensor& row_expert, int64_t epr,
                 int64_t W, int64_t max_tokens, const at::Tensor& dispatch_ctx) {
  check_cuda(tdb::launch_ep_recv_ids(i32(recv_count), base_self.has_value() ? i32(*base_self) : nullptr, i32(row_expert), epr, W,
                                     max_tokens, row_expert.numel(), ctxp(dispatch_ctx), cur_stream()),
             "launch_ep_recv_ids");
}
at::Tensor ep_gather_rows(const at::Tensor& recv_x, const at::Tensor& recv_scale, const at::Tensor& sorted_ids,
                          const at::Tensor& meta, int64_t H, bool quant, int64_t rows_per_parity, const at::Tensor& dispatch_ctx) {
  c10::cuda::CUDAGuard guard(recv_x.device());
  at::Tensor out = at::empty({sorted_ids.numel(), H}, recv_x.options().dtype(at::kBFloat16));
  check_cuda(tdb::launch_ep_gather_rows(recv_x.data_ptr(), recv_scale.data_ptr<float>(), i32(sorted_ids), i32(meta), out.data_ptr(),
                                        sorted_ids.numel(), H, quant ? 1 : 0, rows_per_parity, ctxp(dispatch_ctx), cur_stream()),
             "launch_ep_gather_rows");
  return out;
}

// Returns (x_sorted [cap, H] bf16, sorted_ids [cap], tile_expert [cap/128], offsets [epr+1], meta [2], counts [epr],
// real_rows [cap + 1]).
std::vector<at::Tensor> ep_finish(const at::Tensor& recv_x, const at::Tensor& recv_scale, const at::Tensor& recv_count,
                                  c10::optional<at::Tensor> base_self, int64_t epr, int64_t W, int64_t max_tokens, int64_t H,
                                  bool quant, int64_t rows_per_parity, const at::Tensor& dispatch_ctx, int64_t cap,
                                  int64_t num_ctas, int64_t parts) {
  c10::cuda::CUDAGuard guard(recv_x.device());
  TORCH_CHECK(cap > 0 && cap % 128 == 0, "ep_finish: cap must be a positive multiple of 128");
  auto i32o = recv_x.options().dtype(at::kInt);
  at::Tensor xs = at::empty({cap, H}, recv_x.options().dtype(at::kBFloat16));
  at::Tensor sorted_ids = at::empty({cap}, i32o);
  at::Tensor tile_expert = at::empty({cap / 128}, i32o);
  at::Tensor offsets = at::empty({epr + 1}, i32o);
  at::Tensor meta = at::empty({2}, i32o);
  at::Tensor counts = at::empty({epr}, i32o);
  at::Tensor real_rows = at::empty({cap + 1}, i32o);
  tdb::EpFinishArgs a;
  a.recv_x = recv_x.data_ptr();
  a.recv_scale = recv_scale.data_ptr<float>();
  a.recv_count = i32(recv_count);
  a.base_self = base_self.has_value() ? i32(*base_self) : nullptr;
  a.epr = epr; a.W = W; a.max_tokens = max_tokens; a.H = H; a.quant = quant ? 1 : 0;
  a.rows_per_parity = rows_per_parity;
  a.dispatch_ctx = ctxp(dispatch_ctx);
  a.x_sorted = xs.data_ptr();
  a.sorted_ids = i32(sorted_ids);
  a.tile_expert = i32(tile_expert);
  a.offsets = i32(offsets);
  a.counts = i32(counts);
  a.meta = i32(meta);
  a.real_rows = i32(real_rows);
  a.cap = cap;
  a.num_ctas = num_ctas;
  a.parts = parts;
  check_cuda(tdb::launch_ep_finish(a, cur_stream()), "launch_ep_finish");
  return {xs, sorted_ids, tile_expert, offsets, meta, counts, real_rows};
}

at::Tensor ep_combine(SymmHeap& h, const at::Tensor& y, c10::optional<at::Tensor> pos_of, const at::Tensor& recv_meta,
                      const at::Tensor& dispatch_ctx, c10::optional<at::Tensor> base_self, int64_t max_tokens,
                      int64_t recv_rows, at::Tensor& ret, at::Tensor& flags, const at::Tensor& topk_ids,
                      c10::optional<at::Tensor> topk_w, int64_t E, at::Tensor& ctx, int64_t num_ctas, double timeout_s,
                      c10::optional<at::Tensor> sorted_ids, c10::optional<at::Tensor> sort_meta,
                      c10::optional<at::Tensor> real_rows, int64_t parts) {
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.is_contiguous(), "ep_combine: y bf16 [rows,H]");
  c10::cuda::CUDAGuard guard(y.device());
  const int64_t T = topk_ids.size(0), k = topk_ids.size(1), H = y.size(1);
  at::Tensor out = at::empty({T, H}, y.options());
  tdb::EpCombineArgs a;
  a.y = y.data_ptr();
  a.pos_of = pos_of.has_value() ? i32(*pos_of) : nullptr;
  if (sorted_ids.has_value()) {
    TORCH_CHECK(sort_meta.has_value(), "ep_combine: sorted_ids needs sort_meta");
    a.sorted_ids = i32(*sorted_ids);
    a.sort_meta = i32(*sort_meta);
    if (real_rows.has_value()) {
      TORCH_CHECK(real_rows->numel() == sorted_ids->numel() + 1, "ep_combine: real_rows must have one entry more than sorted_ids");
      a.real_rows = i32(*real_rows);
      a.real_cap = sorted_ids->numel();
    }
  }
  a.recv_meta = i32(recv_meta);
  a.dispatch_ctx = ctxp(dispatch_ctx);
  a.base_self = base_self.has_value() ? i32(*base_self) : nullptr;
  a.max_tokens = max_tokens;
  a.recv_rows = recv_rows;
  a.ret = ret.data_ptr();
  a.ret_half = static_cast<uint64_t>(ret.numel()) / 2;
  a.flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  a.topk_ids = i32(topk_ids);
  a.topk_w = nullptr;
  if (topk_w.has_value()) {
    TORCH_CHECK(topk_w->scalar_type() == at::kFloat && topk_w->is_contiguous(), "ep_combine: fp32 weights");
    a.topk_w = topk_w->data_ptr<float>();
  }
  a.out = out.data_ptr();
  a.T = T; a.H = H; a.k = k; a.E = E;
  a.num_ctas = num_ctas;
  a.parts = parts;
  a.ctx = ctxp(ctx);
  a.symm = h.info(ns(timeout_s));
  TORCH_CHECK(a.ret_half >= static_cast<uint64_t>(T) * k * H, "ep_combine: return buffer too small");
  check_cuda(tdb::launch_ep_combine(a, cur_stream()), "launch_ep_combine");
  return out;
}

void a2a_single(SymmHeap& h, const at::Tensor& in, at::Tensor& out, const at::Tensor& splits_all, at::Tensor& flags,
                at::Tensor& ctx, int64_t parts, double timeout_s) {
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "a2a_single: contiguous tensors");
  const int64_t row_bytes = in.dim() > 1 ? in.stride(0) * in.element_size() : in.element_size();
  check_cuda(tdb::launch_a2a_single(in.data_ptr(), out.data_ptr(), i32(splits_all), row_bytes,
                                    reinterpret_cast<uint32_t*>(flags.data_ptr()), ctxp(ctx), h.info(ns(timeout_s)), parts,
                                    cur_stream()),
             "launch_a2a_single");
}

void a2a_cols(SymmHeap& h, const at::Tensor& in, at::Tensor& out, int64_t s_local, at::Tensor& flags, at::Tensor& ctx,
              int64_t parts, double timeout_s) {
  TORCH_CHECK(in.dim() == 2 && in.stride(1) == 1 && out.dim() == 2 && out.is_contiguous() && flags.numel() >= 16,
              "a2a_cols: in [S, C] with unit column stride, out [max s_local, W * C] contiguous, flags [2][8]");
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t row_bytes = in.size(1) * in.element_size();
  check_cuda(tdb::launch_a2a_cols(in.data_ptr(), in.stride(0) * in.element_size(), out.data_ptr(),
                                  static_cast<uint64_t>(out.numel()) * out.element_size(), row_bytes, s_local,
                                  reinterpret_cast<uint32_t*>(flags.data_ptr()), ctxp(ctx), h.info(ns(timeout_s)), parts,
                                  cur_stream()),
             "launch_a2a_cols");
}

std::vector<at::Tensor> fp8_quant(const at::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "fp8_quant: bf16 [T,H]");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0), H = x.size(1);
  at::Tensor q = at::empty({T, H}, x.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s = at::empty({T, H / 128}, x.options().dtype(at::kFloat));
  check_cuda(tdb::launch_fp8_quant(x.data_ptr(), q.data_ptr(), s.data_ptr<float>(), T, H, cur_stream()), "launch_fp8_quant");
  return {q, s};
}
at::Tensor fp8_dequant(const at::Tensor& q, const at::Tensor& s) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.is_contiguous() && s.is_contiguous(), "fp8_dequant: [T,H] fp8 + [T,H/128] fp32");
  c10::cuda::CUDAGuard guard(q.device());
  at::Tensor out = at::empty({q.size(0), q.size(1)}, q.options().dtype(at::kBFloat16));
  check_cuda(tdb::launch_fp8_dequant(q.data_ptr(), s.data_ptr<float>(), out.data_ptr(), q.size(0), q.size(1), cur_stream()),
             "launch_fp8_dequant");
  return out;
}

}  // namespace

void bind_ep(py::module_& m) {
  m.def("ep_dispatch", &ep_dispatch, py::arg("heap"), py::arg("x"), py::arg("topk_ids"), py::arg("E"), py::arg("quant"),
        py::arg("max_tokens"), py::arg("recv_x"), py::arg("recv_scale"), py::arg("recv_meta"), py::arg("recv_count"),
        py::arg("flags"), py::arg("rows_per_parity"), py::arg("base"), py::arg("cursor"), py::arg("sent_row"), py::arg("ctx"),
        py::arg("num_ctas"), py::arg("timeout_s"), py::arg("parts") = 1);
  m.def("ep_count", &ep_count);
  m.def("ep_layout", &ep_layout);
  m.def("ep_recv_ids", &ep_recv_ids);
  m.def("ep_gather_rows", &ep_gather_rows);
  m.def("ep_finish", &ep_finish, py::arg("recv_x"), py::arg("recv_scale"), py::arg("recv_count"), py::arg("base_self"),
        py::arg("epr"), py::arg("W"), py::arg("max_tokens"), py::arg("H"), py::arg("quant"), py::arg("rows_per_parity"),
        py::arg("dispatch_ctx"), py::arg("cap"), py::arg("num_ctas"), py::arg("parts") = 1);
  m.def("ep_combine", &ep_combine, py::arg("heap"), py::arg("y"), py::arg("pos_of"), py::arg("recv_meta"),
        py::arg("dispatch_ctx"), py::arg("base_self"), py::arg("max_tokens"), py::arg("recv_rows"), py::arg("ret"),
        py::arg("flags"), py::arg("topk_ids"), py::arg("topk_w"), py::arg("E"), py::arg("ctx"), py::arg("num_ctas"),
        py::arg("timeout_s"), py::arg("sorted_ids") = py::none(), py::arg("sort_meta") = py::none(),
        py::arg("real_rows") = py::none(), py::arg("parts") = 1);
  m.def("a2a_single", &a2a_single);
  m.def("a2a_cols", &a2a_cols);
  m.def("fp8_quant", &fp8_quant);
  m.def("fp8_dequant", &fp8_dequant);
}
