// Python bindings of the attention kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "tdb/attn.h"
#include "tdb/symm_heap.h"

namespace py = pybind11;
using tdb::SymmHeap;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_cuda(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }

tdb::AttnKV make_kv(const at::Tensor& k_cache, const at::Tensor& v_cache, const at::Tensor& block_table) {
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4, "KV cache must be [pages, page_size, Hkv, D]");
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous(), "KV cache must be contiguous");
  TORCH_CHECK(k_cache.scalar_type() == at::kBFloat16 && v_cache.scalar_type() == at::kBFloat16, "bf16 KV cache expected");
  TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.dim() == 2 && block_table.is_contiguous(),
              "block_table must be contiguous int32 [B, max_pages]");
  tdb::AttnKV kv;
  kv.k_cache = k_cache.data_ptr();
  kv.v_cache = v_cache.data_ptr();
  kv.block_table = block_table.data_ptr<int32_t>();
  kv.max_pages = block_table.size(1);
  kv.page_size = k_cache.size(1);
  kv.num_kv_heads = k_cache.size(2);
  return kv;
}

void check_i32(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), name, ": contiguous int32 CUDA tensor expected");
}

at::Tensor flash_fwd(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                     const at::Tensor& block_table, const at::Tensor& cu_seqlens_q, const at::Tensor& kv_lens,
                     c10::optional<at::Tensor> q_pos0, int64_t max_q_len, bool causal, double scale, double softcap,
                     c10::optional<at::Tensor> lse) {
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && q.scalar_type() == at::kBFloat16, "q must be contiguous bf16 [T, Hq, D]");
  check_i32(cu_seqlens_q, "cu_seqlens_q");
  check_i32(kv_lens, "kv_lens");
  c10::cuda::CUDAGuard guard(q.device());
  tdb::FlashFwdArgs a;
  at::Tensor out = at::empty_like(q);
  a.q = q.data_ptr();
  a.out = out.data_ptr();
  a.lse = nullptr;
  if (lse.has_value()) {
    TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == q.size(0) * q.size(1),
                "lse must be contiguous fp32 [Hq, T]");
    a.lse = lse->data_ptr<float>();
  }
  a.cu_seqlens_q = cu_seqlens_q.data_ptr<int32_t>();
  a.q_pos0 = nullptr;
  if (q_pos0.has_value()) {
    check_i32(*q_pos0, "q_pos0");
    a.q_pos0 = q_pos0->data_ptr<int32_t>();
  }
  a.kv_lens = kv_lens.data_ptr<int32_t>();
  a.kv = make_kv(k_cache, v_cache, block_table);
  a.batch = kv_lens.numel();
  a.max_q_len = max_q_len;
  a.num_q_heads = q.size(1);
  a.head_dim = q.size(2);
  a.total_q = q.size(0);
  a.causal = causal ? 1 : 0;
  a.scale = scale;
  a.softcap = softcap;
  TORCH_CHECK(k_cache.size(3) == a.head_dim, "head_dim mismatch between q and the cache");
  check_cuda(tdb::launch_flash_fwd(a, cur_stream()), "launch_flash_fwd");
  return out;
}

// Prefill attention on the tcgen05 path (head dim 128).  Returns (out, error flag int32[1]: non-zero if a bounded wait
// inside the kernel gave up).
std::vector<at::Tensor> flash_fwd_sm100(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                                        const at::Tensor& block_table, const at::Tensor& cu_seqlens_q, const at::Tensor& kv_lens,
                                        c10::optional<at::Tensor> q_pos0, int64_t max_q_len, int64_t max_kv_len, bool causal,
                                        double scale, c10::optional<at::Tensor> lse) {
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && q.scalar_type() == at::kBFloat16 && q.size(2) == 128,
              "flash_fwd_sm100: q must be contiguous bf16 [T, Hq, 128]");
  TORCH_CHECK(k_cache.scalar_type() == at::kBFloat16 && v_cache.scalar_type() == at::kBFloat16 && k_cache.is_contiguous() &&
                  v_cache.is_contiguous() && k_cache.size(3) == 128,
              "flash_fwd_sm100: contiguous bf16 caches [pages, page, Hkv, 128]");
  check_i32(cu_seqlens_q, "cu_seqlens_q");
  check_i32(kv_lens, "kv_lens");
  check_i32(block_table, "block_table");
  c10::cuda::CUDAGuard guard(q.device());
  tdb::FlashFwdSm100Args a;
  at::Tensor out = at::empty_like(q);
  at::Tensor err = at::zeros({1}, q.options().dtype(at::kInt));
  a.q = q.data_ptr();
  a.out = out.data_ptr();
  a.lse = nullptr;
  if (lse.has_value()) {
    TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == q.size(0) * q.size(1),
                "lse must be contiguous fp32 [Hq, T]");
    a.lse = lse->data_ptr<float>();
  }
  a.cu_seqlens_q = cu_seqlens_q.data_ptr<int32_t>();
  a.q_pos0 = nullptr;
  if (q_pos0.has_value()) {
    check_i32(*q_pos0, "q_pos0");
    a.q_pos0 = q_pos0->data_ptr<int32_t>();
  }
  a.kv_lens = kv_lens.data_ptr<int32_t>();
  a.kv = make_kv(k_cache, v_cache, block_table);
  a.batch = kv_lens.numel();
  a.max_q_len = max_q_len;
  a.num_q_heads = q.size(1);
  a.num_kv_heads = k_cache.size(2);
  a.head_dim = 128;
  a.total_q = q.size(0);
  a.causal = causal ? 1 : 0;
  a.scale = scale;
  TORCH_CHECK(max_kv_len >= 1, "flash_fwd_sm100: max_kv_len must be positive");
  a.Lp = static_cast<int>((max_kv_len + 63) / 64 * 64);
  at::Tensor kd = at::empty({a.batch * a.num_kv_heads, a.Lp, 128}, q.options());
  at::Tensor vt = at::empty({a.batch * a.num_kv_heads, 128, a.Lp}, q.options());
  a.k_dense = kd.data_ptr();
  a.vt_dense = vt.data_ptr();
  a.error_flag = err.data_ptr<int32_t>();
  check_cuda(tdb::launch_flash_fwd_sm100(a, cur_stream()), "launch_flash_fwd_sm100");
  return {out, err};
}

tdb::DecodeArgs decode_args(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                            const at::Tensor& block_table, const at::Tensor& kv_lens, at::Tensor& workspace,
                            int64_t splits, double scale, double softcap) {
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && q.scalar_type() == at::kBFloat16, "q must be contiguous bf16 [B, Hq, D]");
  check_i32(kv_lens, "kv_lens");
  TORCH_CHECK(workspace.scalar_type() == at::kFloat && workspace.is_contiguous(), "workspace must be fp32");
  tdb::DecodeArgs a;
  a.q = q.data_ptr();
  a.workspace = workspace.data_ptr<float>();
  a.kv_lens = kv_lens.data_ptr<int32_t>();
  a.kv = make_kv(k_cache, v_cache, block_table);
  a.batch = q.size(0);
  a.num_q_heads = q.size(1);
  a.head_dim = q.size(2);
  a.splits = splits;
  a.scale = scale;
  a.softcap = softcap;
  TORCH_CHECK(k_cache.size(3) == a.head_dim, "head_dim mismatch between q and the cache");
  TORCH_CHECK(workspace.numel() >= tdb::decode_workspace_floats(a.batch, a.num_q_heads, a.head_dim, a.splits),
              "decode workspace too small");
  return a;
}

// Split-KV decode + local combine.  Any of out / out_lse / out_f32 may be None.
void decode_attn(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, const at::Tensor& block_table,
                 const at::Tensor& kv_lens, at::Tensor& workspace, int64_t splits, double scale, double softcap,
                 c10::optional<at::Tensor> out, c10::optional<at::Tensor> out_lse, c10::optional<at::Tensor> out_f32,
                 c10::optional<at::Tensor> counters) {
  c10::cuda::CUDAGuard guard(q.device());
  tdb::DecodeArgs a = decode_args(q, k_cache, v_cache, block_table, kv_lens, workspace, splits, scale, softcap);
  if (counters.has_value() && out.has_value() && !out_lse.has_value() && !out_f32.has_value()) {
    // one launch: the last split CTA of every (sequence, KV head) merges the partials
    const int64_t group = a.num_q_heads / k_cache.size(2);
    const int64_t need = static_cast<int64_t>(a.batch) * k_cache.size(2) * ((group + 15) / 16);
    TORCH_CHECK(counters->scalar_type() == at::kInt && counters->numel() >= need, "decode_attn: counters too small");
    TORCH_CHECK(out->scalar_type() == at::kBFloat16 && out->is_contiguous(), "decode_attn: out must be contiguous bf16");
    a.fuse_counters = reinterpret_cast<uint32_t*>(counters->data_ptr());
    a.fuse_out = out->data_ptr();
    check_cuda(tdb::launch_decode_splitkv(a, cur_stream()), "launch_decode_splitkv(fused combine)");
    return;
  }
  check_cuda(tdb::launch_decode_splitkv(a, cur_stream()), "launch_decode_splitkv");
  check_cuda(tdb::launch_decode_combine(a, out.has_value() ? out->data_ptr() : nullptr,
                                        out_lse.has_value() ? out_lse->data_ptr<float>() : nullptr,
                                        out_f32.has_value() ? out_f32->data_ptr<float>() : nullptr, cur_stream()),
             "launch_decode_combine");
}

// Distributed flash-decode.  With `counters` (int32, batch x KV heads x head chunks, zero) and a problem whose head
// chunks fit the SMs: ONE launch (split-KV, local merge, packet exchange, cross-rank merge).  Otherwise split-KV and
// the exchange + merge kernel.  Returns the number of launches.
int64_t dist_decode_attn(SymmHeap& h, const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                         const at::Tensor& block_table, const at::Tensor& kv_lens, at::Tensor& workspace, int64_t splits,
                         double scale, double softcap, at::Tensor& out, at::Tensor& staging, at::Tensor& ctx,
                         double timeout_s, c10::optional<at::Tensor> counters) {
  c10::cuda::CUDAGuard guard(q.device());
  tdb::DecodeArgs a = decode_args(q, k_cache, v_cache, block_table, kv_lens, workspace, splits, scale, softcap);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous(), "dist_decode_attn: out must be contiguous bf16");
  const int64_t half = staging.numel() * staging.element_size() / 16;
  const auto info = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  if (counters.has_value()) {
    const int64_t group = a.num_q_heads / k_cache.size(2);
    const int64_t chunks = static_cast<int64_t>(a.batch) * k_cache.size(2) * ((group + 15) / 16);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (chunks <= sms && splits <= 64) {
      TORCH_CHECK(counters->scalar_type() == at::kInt && counters->numel() >= chunks, "dist_decode_attn: counters too small");
      a.fuse_counters = reinterpret_cast<uint32_t*>(counters->data_ptr());
      a.fuse_out = out.data_ptr();
      check_cuda(tdb::launch_dist_decode_fused(a, staging.data_ptr(), half, reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr()),
                                               info, cur_stream()),
                 "launch_dist_decode_fused");
      return 1;
    }
  }
  check_cuda(tdb::launch_decode_splitkv(a, cur_stream()), "launch_decode_splitkv");
  check_cuda(tdb::launch_dist_combine(a, out.data_ptr(), staging.data_ptr(), half,
                                      reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr()), info, cur_stream()),
             "launch_dist_combine");
  return 2;
}

}  // namespace

void bind_attn(py::module_& m) {
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_fwd_sm100", &flash_fwd_sm100);
  m.def("decode_attn", &decode_attn);
  m.def("dist_decode_attn", &dist_decode_attn, py::arg("heap"), py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("block_table"), py::arg("kv_lens"), py::arg("workspace"), py::arg("splits"), py::arg("scale"),
        py::arg("softcap"), py::arg("out"), py::arg("staging"), py::arg("ctx"), py::arg("timeout_s"),
        py::arg("counters") = py::none());
  m.def("decode_workspace_floats", &tdb::decode_workspace_floats);
}
