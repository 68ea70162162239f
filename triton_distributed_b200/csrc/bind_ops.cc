// Python bindings of the collective, MoE, attention and elementwise kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "tdb/api.h"
#include "tdb/coll.h"
#include "tdb/gdn.h"
#include "tdb/ops.h"
#include "tdb/symm_heap.h"

namespace py = pybind11;
using tdb::SymmHeap;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

tdb::DType to_dtype(at::ScalarType t) {
  switch (t) {
    case at::kBFloat16: return tdb::kBF16;
    case at::kHalf: return tdb::kF16;
    case at::kFloat: return tdb::kF32;
    default: TORCH_CHECK(false, "unsupported dtype for a collective (bf16 / fp16 / fp32)");
  }
}

uint64_t ns(double seconds) { return static_cast<uint64_t>(seconds * 1e9); }

void all_reduce(SymmHeap& h, const at::Tensor& in, at::Tensor& out, at::Tensor& ws, at::Tensor& flags, at::Tensor& ctx,
                int method, bool reduce_scatter, int64_t max_ctas, int64_t num_ctas, double timeout_s) {
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "all_reduce: contiguous tensors expected");
  c10::cuda::CUDAGuard guard(in.device());
  tdb::AllReduceArgs a;
  a.in = in.data_ptr();
  a.out = out.data_ptr();
  a.bytes = static_cast<uint64_t>(in.numel()) * in.element_size();
  a.dtype = to_dtype(in.scalar_type());
  a.method = method;
  a.reduce_scatter = reduce_scatter ? 1 : 0;
  a.ws = ws.data_ptr();
  a.ws_half_bytes = static_cast<uint64_t>(ws.numel()) * ws.element_size() / 2;
  a.flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  a.max_ctas = max_ctas;
  a.num_ctas = num_ctas;
  a.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  a.symm = h.info(ns(timeout_s));
  check_cuda(tdb::launch_allreduce(a, cur_stream()), "launch_allreduce");
}

void barrier_all(SymmHeap& h, at::Tensor& flags, at::Tensor& ctx, double timeout_s) {
  check_cuda(tdb::launch_barrier(reinterpret_cast<uint32_t*>(flags.data_ptr()),
                                 reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr()), h.info(ns(timeout_s)), cur_stream()),
             "launch_barrier");
}

void all_gather(SymmHeap& h, at::Tensor& buf, int64_t shard_bytes, at::Tensor& flags, at::Tensor& ctx, int method,
                int64_t max_ctas, int64_t num_ctas, double timeout_s) {
  tdb::AllGatherArgs a;
  a.buf = buf.data_ptr();
  a.shard_bytes = shard_bytes;
  a.method = method;
  a.flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  a.max_ctas = max_ctas;
  a.num_ctas = num_ctas;
  a.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  a.symm = h.info(ns(timeout_s));
  TORCH_CHECK(static_cast<uint64_t>(buf.numel()) * buf.element_size() >= static_cast<uint64_t>(shard_bytes) * h.world(),
              "all_gather: buffer smaller than world * shard");
  check_cuda(tdb::launch_allgather(a, cur_stream()), "launch_allgather");
}

void all_gather_ll(SymmHeap& h, const at::Tensor& in, at::Tensor& out, at::Tensor& staging, at::Tensor& ctx,
                   int64_t num_ctas, double timeout_s) {
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "all_gather_ll: contiguous tensors expected");
  tdb::AllGatherLLArgs a;
  a.in = in.data_ptr();
  a.out = out.data_ptr();
  a.shard_bytes = static_cast<uint64_t>(in.numel()) * in.element_size();
  a.staging = staging.data_ptr();
  a.staging_half_bytes = static_cast<uint64_t>(staging.numel()) * staging.element_size() / 2;
  a.num_ctas = num_ctas;
  a.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  a.symm = h.info(ns(timeout_s));
  TORCH_CHECK(static_cast<uint64_t>(out.numel()) * out.element_size() >= a.shard_bytes * h.world(),
              "all_gather_ll: output smaller than world * shard");
  check_cuda(tdb::launch_allgather_ll(a, cur_stream()), "launch_allgather_ll");
}

void primitives_test(SymmHeap& h, at::Tensor& data, at::Tensor& scratch, at::Tensor& sig, at::Tensor& bar_flags,
                     int64_t n, int64_t epoch, double timeout_s) {
  check_cuda(tdb::launch_primitives_test(reinterpret_cast<int32_t*>(data.data_ptr()),
                                         reinterpret_cast<int32_t*>(scratch.data_ptr()),
                                         reinterpret_cast<uint32_t*>(sig.data_ptr()),
                                         reinterpret_cast<uint32_t*>(bar_flags.data_ptr()), n, epoch,
                                         h.info(ns(timeout_s)), cur_stream()),
             "launch_primitives_test");
}

// cmp: 0 ==, 1 >= (wrap-safe), 2 !=
void timeout_probe(SymmHeap& h, at::Tensor& flag, int64_t expected, double timeout_s, int64_t cmp) {
  check_cuda(tdb::launch_timeout_probe(reinterpret_cast<const uint32_t*>(flag.data_ptr()), expected, cmp,
                                       h.info(ns(timeout_s)), cur_stream()),
             "launch_timeout_probe");
}

// Put `src` into the heap object `dst` of `peer` through the checked translation (what TDB200_DEBUG=1 turns on for
// every put / get / signal): a bad destination or rank is recorded as status 4 and nothing is written.
void bounds_probe(SymmHeap& h, at::Tensor& dst, const at::Tensor& src, int64_t nbytes, int64_t peer) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && nbytes >= 0 && nbytes <= static_cast<int64_t>(src.nbytes()),
              "bounds_probe: device tensors and nbytes <= src.nbytes() expected");
  check_cuda(tdb::launch_bounds_probe(dst.data_ptr(), src.data_ptr(), static_cast<uint64_t>(nbytes), static_cast<int>(peer),
                                      h.info(ns(1.0)), cur_stream()),
             "launch_bounds_probe");
}

void p2p_copy(at::Tensor& dst, const at::Tensor& src, int64_t num_ctas, int64_t mode) {
  TORCH_CHECK(dst.is_contiguous() && src.is_contiguous(), "p2p_copy: contiguous tensors expected");
  const uint64_t bytes = static_cast<uint64_t>(src.numel()) * src.element_size();
  TORCH_CHECK(static_cast<uint64_t>(dst.numel()) * dst.element_size() >= bytes, "p2p_copy: destination too small");
  check_cuda(tdb::launch_p2p_copy(dst.data_ptr(), src.data_ptr(), bytes, num_ctas, mode, cur_stream()), "launch_p2p_copy");
}

// ------------------------------------------------------------------ elementwise
void check_bf16(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, ": CUDA bf16 tensor expected");
}

at::Tensor rmsnorm(const at::Tensor& x, const at::Tensor& w, double eps, c10::optional<at::Tensor> residual) {
  check_bf16(x, "rmsnorm");
  check_bf16(w, "rmsnorm");
  TORCH_CHECK(x.stride(-1) == 1 && x.dim() >= 1, "rmsnorm: innermost dimension must be contiguous");
  const int64_t H = x.size(-1);
  at::Tensor x2 = x.dim() == 2 ? x : x.reshape({-1, H});
  TORCH_CHECK(x2.stride(1) == 1, "rmsnorm: unsupported layout");
  const int64_t T = x2.size(0);
  at::Tensor out = at::empty({T, H}, x.options());
  void* res = nullptr;
  if (residual.has_value()) {
    TORCH_CHECK(residual->is_contiguous() && residual->numel() == T * H, "rmsnorm: residual must be contiguous [T,H]");
    check_bf16(*residual, "rmsnorm");
    res = residual->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  check_cuda(tdb::launch_rmsnorm(x2.data_ptr(), res, w.data_ptr(), out.data_ptr(), T, H, x2.stride(0), eps, cur_stream()),
             "launch_rmsnorm");
  auto shape = x.sizes().vec();
  return out.reshape(shape);
}

at::Tensor silu_mul(const at::Tensor& in) {
  check_bf16(in, "silu_mul");
  TORCH_CHECK(in.stride(-1) == 1, "silu_mul: innermost dimension must be contiguous");
  const int64_t I2 = in.size(-1);
  TORCH_CHECK(I2 % 2 == 0, "silu_mul: last dimension must be even");
  at::Tensor in2 = in.dim() == 2 ? in : in.reshape({-1, I2});
  const int64_t T = in2.size(0), I = I2 / 2;
  at::Tensor out = at::empty({T, I}, in.options());
  c10::cuda::CUDAGuard guard(in.device());
  check_cuda(tdb::launch_silu_mul(in2.data_ptr(), out.data_ptr(), T, I, in2.stride(0), cur_stream()), "launch_silu_mul");
  auto shape = in.sizes().vec();
  shape.back() = I;
  return out.reshape(shape);
}

at::Tensor add(const at::Tensor& a, const at::Tensor& b) {
  check_bf16(a, "add");
  check_bf16(b, "add");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && a.numel() == b.numel(), "add: contiguous same-size tensors");
  at::Tensor out = at::empty_like(a);
  c10::cuda::CUDAGuard guard(a.device());
  check_cuda(tdb::launch_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream()), "launch_add");
  return out;
}

// qkv [T, (Hq+2Hkv)*D]; returns q [T, Hq, D]; k/v land in the caches at `slots` (flat [num_slots, Hkv, D]).
at::Tensor qk_norm_rope_kv(const at::Tensor& qkv, c10::optional<at::Tensor> qw, c10::optional<at::Tensor> kw,
                           const at::Tensor& positions, c10::optional<at::Tensor> slots, at::Tensor& k_cache,
                           at::Tensor& v_cache, int64_t Hq, int64_t Hkv, int64_t D, double eps, double theta) {
  check_bf16(qkv, "qk_norm_rope_kv");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (Hq + 2 * Hkv) * D, "qk_norm_rope_kv: bad qkv shape");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous(), "positions must be int64");
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous(), "caches must be contiguous");
  const int64_t T = qkv.size(0);
  TORCH_CHECK(k_cache.numel() == v_cache.numel() && k_cache.numel() % (Hkv * D) == 0, "qk_norm_rope_kv: cache shape mismatch");
  const int64_t cache_rows = k_cache.numel() / (Hkv * D);
  at::Tensor q = at::empty({T, Hq, D}, qkv.options());
  const int64_t* sl = nullptr;
  if (slots.has_value()) {
    TORCH_CHECK(slots->scalar_type() == at::kLong && slots->is_contiguous(), "slots must be int64");
    sl = slots->data_ptr<int64_t>();
  }
  c10::cuda::CUDAGuard guard(qkv.device());
  check_cuda(tdb::launch_qk_norm_rope_kv(qkv.data_ptr(), qw.has_value() ? qw->data_ptr() : nullptr,
                                         kw.has_value() ? kw->data_ptr() : nullptr, positions.data_ptr<int64_t>(), sl,
                                         q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, Hq, Hkv, D,
                                         qkv.stride(0), eps, theta, Hkv * D, cache_rows, cur_stream()),
             "launch_qk_norm_rope_kv");
  return q;
}

at::Tensor embedding(const at::Tensor& ids, const at::Tensor& table) {
  check_bf16(table, "embedding");
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_cuda(), "embedding: int64 CUDA ids expected");
  at::Tensor idc = ids.contiguous();
  const int64_t T = idc.numel(), H = table.size(1);
  at::Tensor out = at::empty({T, H}, table.options());
  c10::cuda::CUDAGuard guard(table.device());
  check_cuda(tdb::launch_embedding(idc.data_ptr<int64_t>(), table.data_ptr(), out.data_ptr(), T, H, table.size(0),
                                   cur_stream()),
             "launch_embedding");
  auto shape = ids.sizes().vec();
  shape.push_back(H);
  return out.reshape(shape);
}

at::Tensor argmax(const at::Tensor& logits) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous(),
              "argmax: contiguous fp32 [B,V] expected");
  at::Tensor out = at::empty({logits.size(0)}, logits.options().dtype(at::kLong));
  c10::cuda::CUDAGuard guard(logits.device());
  check_cuda(tdb::launch_argmax(logits.data_ptr<float>(), out.data_ptr<int64_t>(), logits.size(0), logits.size(1),
                                cur_stream()),
             "launch_argmax");
  return out;
}

void abs_sum(const at::Tensor& x, at::Tensor& out) {
  check_bf16(x, "abs_sum");
  TORCH_CHECK(x.is_contiguous() && out.scalar_type() == at::kFloat, "abs_sum: contiguous bf16 in, fp32 out");
  c10::cuda::CUDAGuard guard(x.device());
  check_cuda(cudaMemsetAsync(out.data_ptr(), 0, 4, cur_stream()), "memset");
  check_cuda(tdb::launch_abs_sum(x.data_ptr(), x.numel(), out.data_ptr<float>(), cur_stream()), "launch_abs_sum");
}

// Gated delta rule forward (variable length).  q, k [T, H, 128]; v [T, H, V]; g fp32 [T, H]; beta [T, H];
// cu_seqlens int32 [N + 1] on the device.  Returns (o [T, H, V] bf16, final_state fp32 [N, H, K, V] or an empty tensor).
std::tuple<at::Tensor, at::Tensor> gdn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g,
                                           const at::Tensor& beta, double scale, const c10::optional<at::Tensor>& h0,
                                           bool output_final_state, const at::Tensor& cu_seqlens) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16 && beta.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kFloat,
              "gdn_fwd: q, k, v, beta bf16 and g fp32 expected");
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && g.is_contiguous() &&
                  beta.is_contiguous(), "gdn_fwd: contiguous [T, H, *] tensors expected");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_cuda() && cu_seqlens.numel() >= 2, "gdn_fwd: cu_seqlens int32 on the device");
  const int64_t T = q.size(0), H = q.size(1), K = q.size(2), V = v.size(2);
  TORCH_CHECK(K == 128 && V % 32 == 0, "gdn_fwd: K = 128 and V a multiple of 32");
  TORCH_CHECK(k.size(0) == T && v.size(0) == T && g.numel() == T * H && beta.numel() == T * H, "gdn_fwd: shape mismatch");
  const int64_t N = cu_seqlens.numel() - 1;
  c10::cuda::CUDAGuard guard(q.device());
  at::Tensor o = at::empty({T, H, V}, q.options());
  at::Tensor ht = output_final_state ? at::empty({N, H, K, V}, q.options().dtype(at::kFloat)) : at::empty({0}, q.options().dtype(at::kFloat));
  tdb::GdnArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.g = g.data_ptr<float>();
  a.beta = beta.data_ptr();
  a.o = o.data_ptr();
  a.initial_state = nullptr;
  if (h0.has_value()) {
    TORCH_CHECK(h0->scalar_type() == at::kFloat && h0->is_contiguous() && h0->numel() == N * H * K * V, "gdn_fwd: initial_state fp32 [N, H, K, V]");
    a.initial_state = h0->data_ptr<float>();
  }
  a.final_state = output_final_state ? ht.data_ptr<float>() : nullptr;
  a.cu_seqlens = cu_seqlens.data_ptr<int32_t>();
  a.num_seqs = N; a.H = H; a.K = K; a.V = V;
  a.scale = static_cast<float>(scale);
  if (T > 0) check_cuda(tdb::launch_gdn_fwd(a, cur_stream()), "launch_gdn_fwd");
  return {o, ht};
}

// Chunk-parallel gated delta rule forward.  chunk_seq / chunk_t0 int32 [NC], seq_chunk0 int32 [N + 1] (device).
// Returns (o bf16 [T, H, V], g_cumsum fp32 [T, H], A fp32 [T, H, 64] or empty, final_state fp32 [N, H, K, V] or empty).
std::vector<at::Tensor> gdn_chunk_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g,
                                      const at::Tensor& beta, double scale, const c10::optional<at::Tensor>& h0,
                                      bool output_final_state, const at::Tensor& cu_seqlens, const at::Tensor& chunk_seq,
                                      const at::Tensor& chunk_t0, const at::Tensor& seq_chunk0, bool return_a) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16 && beta.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kFloat,
              "gdn_chunk_fwd: q, k, v, beta bf16 and g fp32 expected");
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && g.is_contiguous() &&
                  beta.is_contiguous(), "gdn_chunk_fwd: contiguous [T, H, *] tensors expected");
  for (const at::Tensor* t : {&cu_seqlens, &chunk_seq, &chunk_t0, &seq_chunk0})
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_cuda() && t->is_contiguous(), "gdn_chunk_fwd: int32 device index tensors");
  const int64_t T = q.size(0), H = q.size(1), K = q.size(2), V = v.size(2);
  TORCH_CHECK(K == 128 && V % 64 == 0 && V >= 64 && V <= 256, "gdn_chunk_fwd: K = 128 and V in {64, 128, 192, 256}");
  TORCH_CHECK(k.size(0) == T && v.size(0) == T && g.numel() == T * H && beta.numel() == T * H, "gdn_chunk_fwd: shape mismatch");
  const int64_t N = cu_seqlens.numel() - 1, NC = chunk_seq.numel();
  TORCH_CHECK(N >= 1 && chunk_t0.numel() == NC && seq_chunk0.numel() == N + 1, "gdn_chunk_fwd: chunk tables do not match");
  c10::cuda::CUDAGuard guard(q.device());
  auto f32 = q.options().dtype(at::kFloat);
  at::Tensor o = at::empty({T, H, V}, q.options());
  at::Tensor gc = at::empty({T, H}, f32);
  at::Tensor A = return_a ? at::empty({T, H, 64}, f32) : at::empty({0}, f32);
  at::Tensor ht = output_final_state ? at::empty({N, H, K, V}, f32) : at::empty({0}, f32);
  at::Tensor w = at::empty({NC, H, 64, K}, q.options());
  at::Tensor u = at::empty({NC, H, 64, V}, q.options());
  at::Tensor vn = at::empty({NC, H, 64, V}, q.options());
  at::Tensor hs = at::empty({NC, H, K, V}, q.options());
  tdb::GdnChunkArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.g = g.data_ptr<float>();
  a.beta = beta.data_ptr();
  a.cu_seqlens = cu_seqlens.data_ptr<int32_t>();
  a.chunk_seq = chunk_seq.data_ptr<int32_t>();
  a.chunk_t0 = chunk_t0.data_ptr<int32_t>();
  a.seq_chunk0 = seq_chunk0.data_ptr<int32_t>();
  a.g_cumsum = gc.data_ptr<float>();
  a.a_out = return_a ? A.data_ptr<float>() : nullptr;
  a.w = w.data_ptr(); a.u = u.data_ptr(); a.v_new = vn.data_ptr(); a.h_chunks = hs.data_ptr();
  a.initial_state = nullptr;
  if (h0.has_value()) {
    TORCH_CHECK(h0->scalar_type() == at::kFloat && h0->is_contiguous() && h0->numel() == N * H * K * V,
                "gdn_chunk_fwd: initial_state fp32 [N, H, K, V]");
    a.initial_state = h0->data_ptr<float>();
  }
  a.final_state = output_final_state ? ht.data_ptr<float>() : nullptr;
  a.o = o.data_ptr();
  a.num_seqs = N; a.num_chunks = NC; a.H = H; a.K = K; a.V = V;
  a.scale = static_cast<float>(scale);
  if (T > 0) check_cuda(tdb::launch_gdn_chunk_fwd(a, cur_stream()), "launch_gdn_chunk_fwd");
  return {o, gc, A, ht};
}

}  // namespace


void bind_attn(py::module_& m);
void bind_moe(py::module_& m);
void bind_ep(py::module_& m);
void bind_mega(py::module_& m);

void bind_more(py::module_& m) {
  bind_attn(m);
  bind_moe(m);
  bind_ep(m);
  bind_mega(m);
  m.def("all_reduce", &all_reduce);
  m.def("barrier_all", &barrier_all);
  m.def("all_gather", &all_gather);
  m.def("all_gather_ll", &all_gather_ll);
  m.def("primitives_test", &primitives_test);
  m.def("timeout_probe", &timeout_probe, py::arg("heap"), py::arg("flag"), py::arg("expected"), py::arg("timeout_s"),
        py::arg("cmp") = 1);
  m.def("bounds_probe", &bounds_probe);
  m.def("p2p_copy", &p2p_copy);
  m.def("rmsnorm", &rmsnorm, py::arg("x"), py::arg("w"), py::arg("eps"), py::arg("residual") = py::none());
  m.def("silu_mul", &silu_mul);
  m.def("add", &add);
  m.def("qk_norm_rope_kv", &qk_norm_rope_kv);
  m.def("embedding", &embedding);
  m.def("argmax", &argmax);
  m.def("abs_sum", &abs_sum);
  m.def("gdn_fwd", &gdn_fwd);
  m.def("gdn_chunk_fwd", &gdn_chunk_fwd);
}
