// Python bindings (pybind11 through torch/extension.h).  The only translation
// unit that sees torch headers; kernels are reached through tdb/api.h.
//
// Plays the part of the reference's pybind op registry
// (csrc/lib/registry.h, registry.cc, op_pybind.cc:29-33).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "tdb/api.h"
#include "tdb/gemv.h"
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
    case at::kInt: return tdb::kI32;
    case at::kByte: return tdb::kU8;
    case at::kFloat8_e4m3fn: return tdb::kE4M3;
    default: TORCH_CHECK(false, "unsupported dtype");
  }
}

// A torch tensor viewing `bytes` of a heap (local, peer or multicast window).
at::Tensor heap_tensor(SymmHeap& h, uint64_t offset, std::vector<int64_t> sizes, at::ScalarType dtype, int peer,
                       bool multicast) {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  const uint64_t bytes = static_cast<uint64_t>(numel) * c10::elementSize(dtype);
  TORCH_CHECK(offset + bytes <= h.heap_bytes(), "heap_tensor: out of range");
  uint64_t base;
  if (multicast) {
    TORCH_CHECK(h.has_multicast(), "heap has no multicast mapping");
    base = h.mc_base();
  } else {
    base = h.peer_base(peer < 0 ? h.rank() : peer);
  }
  int dev = 0;
  check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, dev);
  // target_device: a peer / multicast mapping is physically remote, but this process addresses it from `dev`
  return at::for_blob(reinterpret_cast<void*>(base + offset), sizes)
      .options(opts)
      .target_device(at::Device(at::kCUDA, dev))
      .deleter([](void*) {})
      .make_tensor();
}

uint64_t heap_offset_of(SymmHeap& h, const at::Tensor& t) {
  const uint64_t p = reinterpret_cast<uint64_t>(t.data_ptr());
  TORCH_CHECK(p >= h.local_base() && p < h.local_base() + h.heap_bytes(), "tensor is not in the local symmetric heap");
  return p - h.local_base();
}

py::dict read_status(SymmHeap& h) {
  py::dict d;
  tdb::StatusPage* pg = h.status_host();
  if (pg == nullptr) return d;
  volatile tdb::StatusRecord* r = &pg->rec;
  d["code"] = r->code;
  d["kernel"] = r->kernel;
  d["where"] = r->where;
  d["block"] = r->block;
  d["peer"] = r->peer;
  d["index"] = r->index;
  d["expected"] = r->expected;
  d["observed"] = r->observed;
  d["abort"] = *reinterpret_cast<volatile int32_t*>(&pg->abort_word);
  d["heartbeat"] = *reinterpret_cast<volatile int32_t*>(&pg->heartbeat);
  return d;
}
void clear_status(SymmHeap& h) {
  if (h.status_host() != nullptr) std::memset(h.status_host(), 0, sizeof(tdb::StatusPage));
}
void set_abort(SymmHeap& h, int v) {
  if (h.status_host() != nullptr) *reinterpret_cast<volatile int32_t*>(&h.status_host()->abort_word) = v;
}

tdb::TensorMap make_tmap3(const void* base, tdb::DType dt, uint64_t d2, uint64_t rows, uint64_t cols,
                          uint64_t row_stride, uint64_t d2_stride, uint32_t box_rows, uint32_t box_cols) {
  tdb::TensorMap m;
  const int r = tdb::encode_tensor_map_3d(&m, base, dt, d2, rows, cols, row_stride, d2_stride, box_rows, box_cols, 128);
  TORCH_CHECK(r == 0, "cuTensorMapEncodeTiled failed with code ", r);
  return m;
}

int pick_block_n(int64_t N, int block_n) {
  if (block_n == 128 || block_n == 256) return block_n;
  return N <= 128 ? 128 : 256;
}

// Kernel form for a GEMM whose row segments have `rows` rows: block_n 128 / 256 force the single-CTA kernel, 512 the
// CTA-pair kernel (256 x 256 tiles over two SMs), 0 picks the pair kernel when the problem is large enough for it and
// the output can go through TMA stores.  TDB200_GEMM_PAIR=0 keeps the automatic choice on the single-CTA kernel.
bool pick_cta_pair(int64_t rows, int64_t N, int block_n, bool tma_store_ok) {
  if (!tma_store_ok) return false;
  if (block_n == 512) return true;
  if (block_n != 0) return false;
  static const bool enabled = [] {
    const char* e = std::getenv("TDB200_GEMM_PAIR");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return enabled && rows >= 256 && N >= 256;
}

int sm_count() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }

// Half-width tail tiles of the pair kernel (TDB200_SPLIT_TAIL=0 turns them off).
bool split_tail_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("TDB200_SPLIT_TAIL");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return enabled;
}

// Optional stall-counter buffer: int64 [num_ctas, 8], zeroed by the caller.
void* stats_ptr(const c10::optional<at::Tensor>& stats, int num_ctas) {
  if (!stats.has_value()) return nullptr;
  TORCH_CHECK(stats->is_cuda() && stats->scalar_type() == at::kLong && stats->is_contiguous() &&
                  stats->numel() >= static_cast<int64_t>(num_ctas) * 8,
              "stats: contiguous int64 CUDA tensor of at least num_ctas * 8 elements expected");
  return stats->data_ptr();
}

// C[M,N] = A[M,K] @ B[N,K]^T   (bf16)
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, int block_n, int num_ctas,
               const c10::optional<at::Tensor>& stats) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "gemm: CUDA tensors expected");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && c.scalar_type() == at::kBFloat16,
              "gemm: bf16 expected");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2, "gemm: 2-D tensors expected");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1, "gemm: innermost dimension must be contiguous");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(b.size(1) == K && c.size(0) == M && c.size(1) == N, "gemm: shape mismatch");
  TORCH_CHECK(K % 8 == 0 && a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "gemm: K and row strides must be multiples of 8");
  if (M == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(a.device());
  tdb::GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmPlain;
  g.M = M; g.N = N; g.K = K;
  g.c = c.data_ptr();
  g.ldc = c.stride(0);
  const bool tma_store_ok = c.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(c.data_ptr()) & 15u) == 0;
  g.cta_pair = pick_cta_pair(M, N, block_n, tma_store_ok) ? 1 : 0;
  g.block_n = g.cta_pair ? 256 : pick_block_n(N, block_n);
  g.tmap_a = make_tmap3(a.data_ptr(), tdb::kBF16, 1, M, K, a.stride(0) * 2, a.stride(0) * 2 * M, 128, 64);
  g.tmap_b = make_tmap3(b.data_ptr(), tdb::kBF16, 1, N, K, b.stride(0) * 2, b.stride(0) * 2 * N,
                        g.cta_pair ? 128 : g.block_n, 64);
  if (tma_store_ok) {
    g.tmap_c = make_tmap3(c.data_ptr(), tdb::kBF16, 1, M, N, c.stride(0) * 2, c.stride(0) * 2 * M, 128, 64);
    g.use_tma_store = 1;
  }
  const int tile_m = g.cta_pair ? 256 : 128;
  const int tiles = ((M + tile_m - 1) / tile_m) * ((N + g.block_n - 1) / g.block_n) * (g.cta_pair ? 2 : 1);
  g.num_ctas = std::min<int>(num_ctas > 0 ? num_ctas : sm_count(), tiles);
  if (g.cta_pair && split_tail_enabled()) {
    g.tmap_b_half = make_tmap3(b.data_ptr(), tdb::kBF16, 1, N, K, b.stride(0) * 2, b.stride(0) * 2 * N, 64, 64);
    g.split_tail = 1;
  }
  g.stats = stats_ptr(stats, g.num_ctas);
  g.symm.world = 1;
  g.symm.timeout_ns = 2000000000ull;
  check_cuda(tdb::launch_gemm(g, cur_stream()), "launch_gemm");
}

// Fused all-gather + GEMM.  a_local [m, K]; b [N_local, K]; out [W*m, N_local];
// ws / flags / ctx live in the symmetric heap (ws, flags) and in device memory (ctx).
void ag_gemm_bf16(SymmHeap& h, const at::Tensor& a_local, const at::Tensor& b, at::Tensor& c, at::Tensor& ws,
                  at::Tensor& flags, at::Tensor& ctx, int64_t max_seg_rows, int64_t max_chunks, int n_comm,
                  int block_n, int num_ctas, bool use_multimem, double timeout_s,
                  const c10::optional<at::Tensor>& stats) {
  TORCH_CHECK(a_local.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "ag_gemm: bf16 expected");
  TORCH_CHECK(a_local.is_contiguous() && b.stride(1) == 1 && c.stride(1) == 1, "ag_gemm: contiguous inputs expected");
  const int W = h.world();
  const int64_t m = a_local.size(0), K = a_local.size(1), N = b.size(0), M = m * W;
  TORCH_CHECK(b.size(1) == K && c.size(0) == M && c.size(1) == N, "ag_gemm: shape mismatch");
  TORCH_CHECK(m <= max_seg_rows, "ag_gemm: more rows than the context was created for");
  TORCH_CHECK(K % 8 == 0, "ag_gemm: K must be a multiple of 8");
  const uint64_t buf_elems = static_cast<uint64_t>(W) * max_seg_rows * K;
  TORCH_CHECK(static_cast<uint64_t>(ws.numel()) >= 2 * buf_elems, "ag_gemm: workspace too small");
  c10::cuda::CUDAGuard guard(a_local.device());
  tdb::GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmAllGather;
  g.M = M; g.N = N; g.K = K;
  g.c = c.data_ptr();
  g.ldc = c.stride(0);
  const bool tma_store_ok = c.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(c.data_ptr()) & 15u) == 0;
  g.cta_pair = (pick_cta_pair(m, N, block_n, tma_store_ok) && n_comm % 2 == 0) ? 1 : 0;
  g.block_n = g.cta_pair ? 256 : pick_block_n(N, block_n);
  g.tmap_a = make_tmap3(ws.data_ptr(), tdb::kBF16, 2, M, K, K * 2, buf_elems * 2, 128, 64);
  g.tmap_a_local = make_tmap3(a_local.data_ptr(), tdb::kBF16, 1, m, K, K * 2, static_cast<uint64_t>(m) * K * 2, 128, 64);
  g.tmap_b = make_tmap3(b.data_ptr(), tdb::kBF16, 1, N, K, b.stride(0) * 2, b.stride(0) * 2 * N,
                        g.cta_pair ? 128 : g.block_n, 64);
  if (tma_store_ok) {
    g.tmap_c = make_tmap3(c.data_ptr(), tdb::kBF16, W, m, N, c.stride(0) * 2, c.stride(0) * 2 * m, 128, 64);
    g.use_tma_store = 1;
  }
  g.num_ctas = num_ctas > 0 ? num_ctas : sm_count();
  g.seg_rows = m;
  g.max_seg_rows = max_seg_rows;
  g.n_comm_ctas = n_comm;
  g.a_local = a_local.data_ptr();
  g.ag_ws = ws.data_ptr();
  g.ag_flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  g.max_chunks = max_chunks;
  g.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  g.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  g.use_multimem = use_multimem ? 1 : 0;
  if (g.cta_pair && split_tail_enabled()) {
    g.tmap_b_half = make_tmap3(b.data_ptr(), tdb::kBF16, 1, N, K, b.stride(0) * 2, b.stride(0) * 2 * N, 64, 64);
    g.split_tail = 1;
  }
  g.stats = stats_ptr(stats, g.num_ctas);
  check_cuda(tdb::launch_gemm(g, cur_stream()), "launch_gemm(all-gather)");
}

// Fused GEMM + reduce-scatter.  a [M, K_local]; b [N, K_local]; out [M/W, N].
void gemm_rs_bf16(SymmHeap& h, const at::Tensor& a, const at::Tensor& b, at::Tensor& out, at::Tensor& slots,
                  at::Tensor& flags, at::Tensor& ctx, int64_t max_seg_rows, int64_t max_tiles, int block_n,
                  int num_ctas, double timeout_s, const c10::optional<at::Tensor>& stats) {
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm_rs: bf16 expected");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm_rs: contiguous inputs expected");
  const int W = h.world();
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(M % W == 0, "gemm_rs: M must be divisible by the world size");
  const int64_t m = M / W;
  TORCH_CHECK(b.size(1) == K && out.size(0) == m && out.size(1) == N, "gemm_rs: shape mismatch");
  TORCH_CHECK(m <= max_seg_rows, "gemm_rs: more rows than the context was created for");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "gemm_rs: K and N must be multiples of 8");
  TORCH_CHECK(static_cast<uint64_t>(slots.numel()) >= 2ull * W * max_seg_rows * N, "gemm_rs: slot buffer too small");
  c10::cuda::CUDAGuard guard(a.device());
  tdb::GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmReduceScatter;
  g.M = M; g.N = N; g.K = K;
  const bool out_tma_ok = out.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15u) == 0;
  g.cta_pair = pick_cta_pair(m, N, block_n, out_tma_ok) ? 1 : 0;
  if (g.cta_pair)
    g.tmap_out = make_tmap3(out.data_ptr(), tdb::kBF16, 1, m, N, out.stride(0) * 2, out.stride(0) * 2 * m, 128, 64);
  g.block_n = g.cta_pair ? 256 : pick_block_n(N, block_n);
  g.tmap_a = make_tmap3(a.data_ptr(), tdb::kBF16, 1, M, K, a.stride(0) * 2, a.stride(0) * 2 * M, 128, 64);
  g.tmap_b = make_tmap3(b.data_ptr(), tdb::kBF16, 1, N, K, b.stride(0) * 2, b.stride(0) * 2 * N,
                        g.cta_pair ? 128 : g.block_n, 64);
  g.num_ctas = num_ctas > 0 ? num_ctas : sm_count();
  g.seg_rows = m;
  g.max_seg_rows = max_seg_rows;
  {
    // one store map per owner rank over that rank's slots (peer-mapped addresses of the same heap offset)
    const uint64_t off = heap_offset_of(h, slots);
    for (int r = 0; r < W; ++r) {
      g.tmap_peer_c[r] = make_tmap3(reinterpret_cast<void*>(h.peer_base(r) + off), tdb::kBF16, 2 * W, m, N, N * 2,
                                    static_cast<uint64_t>(max_seg_rows) * N * 2, 128, 64);
    }
    g.use_tma_store = 1;
  }
  g.rs_slots = slots.data_ptr();
  g.rs_flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  g.max_tiles = max_tiles;
  g.rs_out = out.data_ptr();
  g.ld_out = out.stride(0);
  g.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  g.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  if (g.cta_pair && split_tail_enabled()) {
    g.tmap_b_half = make_tmap3(b.data_ptr(), tdb::kBF16, 1, N, K, b.stride(0) * 2, b.stride(0) * 2 * N, 64, 64);
    g.split_tail = 1;
  }
  g.stats = stats_ptr(stats, g.num_ctas);
  check_cuda(tdb::launch_gemm(g, cur_stream()), "launch_gemm(reduce-scatter)");
}

// ------------------------------------------------------------------ block-scaled fp8 GEMM family
void check_fp8_operands(const at::Tensor& a_q, const at::Tensor& a_s, const at::Tensor& b_q, const at::Tensor& b_s,
                        const char* name) {
  TORCH_CHECK(a_q.is_cuda() && b_q.is_cuda() && a_s.is_cuda() && b_s.is_cuda(), name, ": CUDA tensors expected");
  TORCH_CHECK(a_q.scalar_type() == at::kFloat8_e4m3fn && b_q.scalar_type() == at::kFloat8_e4m3fn, name,
              ": e4m3 operands expected");
  TORCH_CHECK(a_s.scalar_type() == at::kFloat && b_s.scalar_type() == at::kFloat && a_s.is_contiguous() && b_s.is_contiguous(),
              name, ": contiguous fp32 scales expected");
  TORCH_CHECK(a_q.dim() == 2 && b_q.dim() == 2 && a_q.stride(1) == 1 && b_q.stride(1) == 1, name, ": 2-D K-major operands expected");
  const int64_t K = a_q.size(1);
  TORCH_CHECK(K >= 128 && K % 128 == 0 && b_q.size(1) == K, name, ": K must be a multiple of 128 and equal for both operands");
  TORCH_CHECK(a_q.stride(0) % 16 == 0 && b_q.stride(0) % 16 == 0 && (reinterpret_cast<uintptr_t>(a_q.data_ptr()) & 15u) == 0 &&
                  (reinterpret_cast<uintptr_t>(b_q.data_ptr()) & 15u) == 0, name, ": operand rows must be 16-byte aligned");
  TORCH_CHECK(a_s.dim() == 2 && a_s.size(0) == a_q.size(0) && a_s.size(1) == K / 128, name, ": a_scales must be [M, K/128]");
  TORCH_CHECK(b_s.dim() == 2 && b_s.size(0) == (b_q.size(0) + 127) / 128 && b_s.size(1) == K / 128, name,
              ": b_scales must be [ceil(N/128), K/128]");
}

// C[M,N] (bf16) = blockscaled(A8 [M,K], a_s [M,K/128]) x blockscaled(B8 [N,K], b_s [ceil(N/128),K/128])^T
void gemm_fp8(const at::Tensor& a_q, const at::Tensor& a_s, const at::Tensor& b_q, const at::Tensor& b_s, at::Tensor& c,
              int num_ctas, const c10::optional<at::Tensor>& stats) {
  check_fp8_operands(a_q, a_s, b_q, b_s, "gemm_fp8");
  const int64_t M = a_q.size(0), K = a_q.size(1), N = b_q.size(0);
  TORCH_CHECK(c.is_cuda() && c.scalar_type() == at::kBFloat16 && c.dim() == 2 && c.size(0) == M && c.size(1) == N &&
                  c.stride(1) == 1, "gemm_fp8: bf16 [M, N] output expected");
  if (M == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(a_q.device());
  tdb::GemmFp8Args g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmPlain;
  g.M = M; g.N = N; g.K = K;
  g.c = c.data_ptr();
  g.ldc = c.stride(0);
  g.a_scales = a_s.data_ptr<float>();
  g.b_scales = b_s.data_ptr<float>();
  g.tmap_a = make_tmap3(a_q.data_ptr(), tdb::kU8, 1, M, K, a_q.stride(0), a_q.stride(0) * M, 128, 128);
  g.tmap_b = make_tmap3(b_q.data_ptr(), tdb::kU8, 1, N, K, b_q.stride(0), b_q.stride(0) * N, 128, 128);
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256) * 2;
  g.num_ctas = std::max(2, std::min<int>(num_ctas > 0 ? num_ctas : sm_count(), tiles)) & ~1;
  g.stats = stats_ptr(stats, g.num_ctas);
  g.symm.world = 1;
  g.symm.timeout_ns = 2000000000ull;
  check_cuda(tdb::launch_gemm_fp8(g, cur_stream()), "launch_gemm_fp8");
}

// Fused all-gather + block-scaled fp8 GEMM: the local fp8 rows [m, K] and their scales [m, K/128] are pushed into
// every rank's workspace by comm CTAs of the launch.
void ag_gemm_fp8(SymmHeap& h, const at::Tensor& a_q, const at::Tensor& a_s, const at::Tensor& b_q, const at::Tensor& b_s,
                 at::Tensor& c, at::Tensor& ws, at::Tensor& ws_scales, at::Tensor& flags, at::Tensor& ctx,
                 int64_t max_seg_rows, int64_t max_chunks, int n_comm, int num_ctas, double timeout_s,
                 const c10::optional<at::Tensor>& stats) {
  check_fp8_operands(a_q, a_s, b_q, b_s, "ag_gemm_fp8");
  TORCH_CHECK(a_q.is_contiguous(), "ag_gemm_fp8: contiguous local shard expected");
  const int W = h.world();
  const int64_t m = a_q.size(0), K = a_q.size(1), N = b_q.size(0), M = m * W, KB = K / 128;
  TORCH_CHECK(c.scalar_type() == at::kBFloat16 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1,
              "ag_gemm_fp8: bf16 [W*m, N] output expected");
  TORCH_CHECK(m <= max_seg_rows, "ag_gemm_fp8: more rows than the context was created for");
  const uint64_t buf_rows = static_cast<uint64_t>(W) * max_seg_rows;
  TORCH_CHECK(static_cast<uint64_t>(ws.numel()) * ws.element_size() >= 2 * buf_rows * K, "ag_gemm_fp8: workspace too small");
  TORCH_CHECK(static_cast<uint64_t>(ws_scales.numel()) >= 2 * buf_rows * KB, "ag_gemm_fp8: scale workspace too small");
  TORCH_CHECK(((m % 128) * KB * 4) % 16 == 0, "ag_gemm_fp8: rows-per-rank % 128 times K/128 must be a multiple of 4");
  c10::cuda::CUDAGuard guard(a_q.device());
  tdb::GemmFp8Args g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmAllGather;
  g.M = M; g.N = N; g.K = K;
  g.c = c.data_ptr();
  g.ldc = c.stride(0);
  g.b_scales = b_s.data_ptr<float>();
  g.tmap_a = make_tmap3(ws.data_ptr(), tdb::kU8, 2, M, K, K, buf_rows * K, 128, 128);
  g.tmap_a_local = make_tmap3(a_q.data_ptr(), tdb::kU8, 1, m, K, K, static_cast<uint64_t>(m) * K, 128, 128);
  g.tmap_b = make_tmap3(b_q.data_ptr(), tdb::kU8, 1, N, K, b_q.stride(0), b_q.stride(0) * N, 128, 128);
  g.num_ctas = (num_ctas > 0 ? num_ctas : sm_count()) & ~1;
  g.seg_rows = m;
  g.max_seg_rows = max_seg_rows;
  g.n_comm_ctas = n_comm;
  g.a_local = a_q.data_ptr();
  g.a_scales_local = a_s.data_ptr<float>();
  g.ag_ws = ws.data_ptr();
  g.ag_ws_scales = ws_scales.data_ptr<float>();
  g.ag_flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  g.max_chunks = max_chunks;
  g.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  g.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  g.stats = stats_ptr(stats, g.num_ctas);
  check_cuda(tdb::launch_gemm_fp8(g, cur_stream()), "launch_gemm_fp8(all-gather)");
}

// Fused block-scaled fp8 GEMM + reduce-scatter.  a_q [M, K_local]; out [M/W, N] bf16.
void gemm_rs_fp8(SymmHeap& h, const at::Tensor& a_q, const at::Tensor& a_s, const at::Tensor& b_q, const at::Tensor& b_s,
                 at::Tensor& out, at::Tensor& slots, at::Tensor& flags, at::Tensor& ctx, int64_t max_seg_rows,
                 int64_t max_tiles, int num_ctas, double timeout_s, const c10::optional<at::Tensor>& stats) {
  check_fp8_operands(a_q, a_s, b_q, b_s, "gemm_rs_fp8");
  const int W = h.world();
  const int64_t M = a_q.size(0), K = a_q.size(1), N = b_q.size(0);
  TORCH_CHECK(M % W == 0, "gemm_rs_fp8: M must be divisible by the world size");
  const int64_t m = M / W;
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == m && out.size(1) == N && out.stride(1) == 1,
              "gemm_rs_fp8: bf16 [M/W, N] output expected");
  TORCH_CHECK(m <= max_seg_rows && N % 8 == 0, "gemm_rs_fp8: rows exceed the context / N must be a multiple of 8");
  TORCH_CHECK(static_cast<uint64_t>(slots.numel()) >= 2ull * W * max_seg_rows * N, "gemm_rs_fp8: slot buffer too small");
  c10::cuda::CUDAGuard guard(a_q.device());
  tdb::GemmFp8Args g;
  std::memset(&g, 0, sizeof(g));
  g.mode = tdb::kGemmReduceScatter;
  g.M = M; g.N = N; g.K = K;
  g.a_scales = a_s.data_ptr<float>();
  g.b_scales = b_s.data_ptr<float>();
  g.tmap_a = make_tmap3(a_q.data_ptr(), tdb::kU8, 1, M, K, a_q.stride(0), a_q.stride(0) * M, 128, 128);
  g.tmap_b = make_tmap3(b_q.data_ptr(), tdb::kU8, 1, N, K, b_q.stride(0), b_q.stride(0) * N, 128, 128);
  g.num_ctas = (num_ctas > 0 ? num_ctas : sm_count()) & ~1;
  g.seg_rows = m;
  g.max_seg_rows = max_seg_rows;
  {
    const uint64_t off = heap_offset_of(h, slots);
    for (int r = 0; r < W; ++r)
      g.tmap_peer_c[r] = make_tmap3(reinterpret_cast<void*>(h.peer_base(r) + off), tdb::kBF16, 2 * W, m, N, N * 2,
                                    static_cast<uint64_t>(max_seg_rows) * N * 2, 128, 64);
  }
  g.rs_slots = slots.data_ptr();
  g.rs_flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  g.max_tiles = max_tiles;
  g.rs_out = out.data_ptr();
  g.ld_out = out.stride(0);
  g.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  g.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  g.stats = stats_ptr(stats, g.num_ctas);
  check_cuda(tdb::launch_gemm_fp8(g, cur_stream()), "launch_gemm_fp8(reduce-scatter)");
}

// Small-M GEMM (decode): out[M,N] = x[M,K] @ w[N,K]^T with split-K; acc / counters are caller-kept scratch.
void skinny_gemm_bf16(const at::Tensor& x, const at::Tensor& w, at::Tensor& out, at::Tensor& acc, at::Tensor& counters,
                      int splits, int num_ctas, int cluster_nt, int cluster_s, int bulk_exchange) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16,
              "skinny_gemm: bf16 expected");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1,
              "skinny_gemm: 2-D tensors with contiguous rows expected");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == M && out.size(1) == N, "skinny_gemm: shape mismatch");
  TORCH_CHECK(M >= 1 && M <= 256, "skinny_gemm: 1 <= M <= 256");
  c10::cuda::CUDAGuard guard(x.device());
  tdb::SkinnyGemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K;
  const int mpad = tdb::skinny_gemm_mpad(M);
  tdb::TensorMap m;
  int r = tdb::encode_tensor_map_2d(&m, w.data_ptr(), tdb::kBF16, N, K, w.stride(0) * 2, 128, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (w) failed: ", r);
  a.tmap_w = m;
  r = tdb::encode_tensor_map_2d(&m, x.data_ptr(), tdb::kBF16, M, K, x.stride(0) * 2, mpad, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (x) failed: ", r);
  a.tmap_x = m;
  a.out = out.data_ptr();
  a.ld_out = out.stride(0);
  a.splits = splits > 0 ? splits : 0;
  a.cluster_nt = cluster_nt;
  a.cluster_s = cluster_s;
  a.bulk_exchange = bulk_exchange;
  a.num_ctas = num_ctas > 0 ? num_ctas : sm_count();
  {
    // the stream-K form accumulates column-major: [ceil(N / 128) * 128 columns][M_pad tokens] fp32
    TORCH_CHECK(acc.scalar_type() == at::kFloat && acc.numel() >= (N + 127) / 128 * 128 * mpad,
                "skinny_gemm: accumulation buffer too small (needs ceil(N / 128) * 128 * M_pad floats)");
    TORCH_CHECK(counters.scalar_type() == at::kInt && counters.numel() >= (N + 127) / 128, "skinny_gemm: counters too small");
    a.acc = acc.data_ptr<float>();
    a.counters = reinterpret_cast<uint32_t*>(counters.data_ptr());
  }
  a.symm.world = 1;
  a.symm.timeout_ns = 2000000000ull;
  check_cuda(tdb::launch_skinny_gemm(a, cur_stream()), "launch_skinny_gemm");
}

// Small-M GEMM + all-reduce in one launch.
void gemm_ar_bf16(SymmHeap& h, const at::Tensor& x, const at::Tensor& w, at::Tensor& out, at::Tensor& acc,
                  at::Tensor& counters, at::Tensor& partial, at::Tensor& flags, at::Tensor& ctx, int64_t m_cap,
                  int64_t max_tiles, int splits, int num_ctas, bool use_multimem, double timeout_s, int cluster_nt,
                  int cluster_s, int bulk_exchange) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16,
              "gemm_ar: bf16 expected");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1, "gemm_ar: contiguous rows expected");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == M && out.size(1) == N, "gemm_ar: shape mismatch");
  TORCH_CHECK(M >= 1 && M <= m_cap && m_cap <= 256, "gemm_ar: M exceeds the context's capacity (<= 256)");
  const int W = h.world();
  const bool mc = use_multimem && h.has_multicast();
  TORCH_CHECK(static_cast<uint64_t>(partial.numel()) >= 2ull * (mc ? 1 : W) * m_cap * N, "gemm_ar: partial buffer too small");
  TORCH_CHECK(acc.scalar_type() == at::kFloat && acc.numel() >= (N + 127) / 128 * 128 * tdb::skinny_gemm_mpad(M) &&
                  counters.numel() >= (N + 127) / 128,
              "gemm_ar: scratch too small (the accumulation buffer needs ceil(N / 128) * 128 * M_pad floats)");
  c10::cuda::CUDAGuard guard(x.device());
  tdb::SkinnyGemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K;
  const int mpad = tdb::skinny_gemm_mpad(M);
  tdb::TensorMap m;
  int r = tdb::encode_tensor_map_2d(&m, w.data_ptr(), tdb::kBF16, N, K, w.stride(0) * 2, 128, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (w) failed: ", r);
  a.tmap_w = m;
  r = tdb::encode_tensor_map_2d(&m, x.data_ptr(), tdb::kBF16, M, K, x.stride(0) * 2, mpad, 64, 128);
  TORCH_CHECK(r == 0, "tensor map (x) failed: ", r);
  a.tmap_x = m;
  a.out = out.data_ptr();
  a.ld_out = out.stride(0);
  a.splits = splits > 0 ? splits : 0;
  a.cluster_nt = cluster_nt;
  a.cluster_s = cluster_s;
  a.bulk_exchange = bulk_exchange;
  a.num_ctas = num_ctas > 0 ? num_ctas : sm_count();
  a.acc = acc.data_ptr<float>();
  a.counters = reinterpret_cast<uint32_t*>(counters.data_ptr());
  a.all_reduce = 1;
  a.use_multimem = mc ? 1 : 0;
  a.partial = partial.data_ptr();
  a.flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  a.max_tiles = max_tiles;
  a.m_cap = m_cap;
  a.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  a.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  check_cuda(tdb::launch_skinny_gemm(a, cur_stream()), "launch_skinny_gemm(all-reduce)");
}

// Decode GEMV (M <= 8) with the fused prologue / epilogue.  `heap` is null without all-reduce.
void fill_gemv(tdb::GemvArgs& a, const at::Tensor& x, const at::Tensor& w, at::Tensor& out,
               const c10::optional<at::Tensor>& norm_w, double eps, bool silu_mul,
               const c10::optional<at::Tensor>& residual, int num_ctas) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16,
              "gemv: bf16 expected");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1,
              "gemv: 2-D tensors with contiguous rows expected");
  const int64_t M = x.size(0), K = w.size(1), N = w.size(0);
  TORCH_CHECK(x.size(1) == (silu_mul ? 2 * K : K), "gemv: x has ", x.size(1), " columns, expected ", silu_mul ? 2 * K : K);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemv: output shape mismatch");
  TORCH_CHECK(M >= 1 && M <= 16, "gemv: 1 <= M <= 16");
  TORCH_CHECK(K <= tdb::gemv_max_k(M), "gemv: K too large for the shared-memory staging of ", M, " rows");
  std::memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K;
  a.x = x.data_ptr(); a.ldx = x.stride(0);
  a.w = w.data_ptr(); a.ldw = w.stride(0);
  a.out = out.data_ptr(); a.ld_out = out.stride(0);
  if (norm_w.has_value()) {
    TORCH_CHECK(norm_w->scalar_type() == at::kBFloat16 && norm_w->numel() == K && norm_w->is_contiguous(), "gemv: norm weight [K] bf16");
    a.norm_w = norm_w->data_ptr();
  }
  a.eps = static_cast<float>(eps);
  a.silu_mul = silu_mul ? 1 : 0;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == M &&
                    residual->size(1) == N && residual->stride(1) == 1, "gemv: residual [M, N] bf16");
    a.residual = residual->data_ptr();
    a.ld_res = residual->stride(0);
  }
  a.num_ctas = num_ctas > 0 ? num_ctas : sm_count();
  a.symm.world = 1;
  a.symm.timeout_ns = 2000000000ull;
}

void gemv_bf16(const at::Tensor& x, const at::Tensor& w, at::Tensor& out, const c10::optional<at::Tensor>& norm_w,
               double eps, bool silu_mul, const c10::optional<at::Tensor>& residual, int num_ctas) {
  c10::cuda::CUDAGuard guard(x.device());
  tdb::GemvArgs a;
  fill_gemv(a, x, w, out, norm_w, eps, silu_mul, residual, num_ctas);
  check_cuda(tdb::launch_gemv(a, cur_stream()), "launch_gemv");
}

void gemv_ar_bf16(SymmHeap& h, const at::Tensor& x, const at::Tensor& w, at::Tensor& out,
                  const c10::optional<at::Tensor>& norm_w, double eps, bool silu_mul,
                  const c10::optional<at::Tensor>& residual, at::Tensor& partial, at::Tensor& flags, at::Tensor& ctx,
                  int64_t m_cap, int64_t max_ctas, int num_ctas, bool use_multimem, double timeout_s) {
  c10::cuda::CUDAGuard guard(x.device());
  tdb::GemvArgs a;
  fill_gemv(a, x, w, out, norm_w, eps, silu_mul, residual, num_ctas);
  const int W = h.world();
  const bool mc = use_multimem && h.has_multicast();
  TORCH_CHECK(static_cast<uint64_t>(partial.numel()) >= 2ull * (mc ? 1 : W) * m_cap * a.N, "gemv_ar: partial buffer too small");
  TORCH_CHECK(flags.numel() >= static_cast<int64_t>(W) * max_ctas, "gemv_ar: flag buffer too small");
  a.all_reduce = 1;
  a.use_multimem = mc ? 1 : 0;
  a.partial = partial.data_ptr();
  a.flags = reinterpret_cast<uint32_t*>(flags.data_ptr());
  a.max_ctas = max_ctas;
  a.m_cap = m_cap;
  a.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  a.symm = h.info(static_cast<uint64_t>(timeout_s * 1e9));
  check_cuda(tdb::launch_gemv(a, cur_stream()), "launch_gemv(all-reduce)");
}

}  // namespace

void bind_more(py::module_& m);  // bind_ops.inc-style split kept in this file for build simplicity

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "triton_distributed_b200 native library (sm_100a)";

  py::class_<SymmHeap>(m, "SymmHeap")
      .def(py::init<int, int, int, uint64_t, const std::string&, bool>(), py::arg("rank"), py::arg("world"),
           py::arg("device"), py::arg("heap_bytes"), py::arg("session"), py::arg("want_multicast"))
      .def("create", &SymmHeap::create)
      .def("exchange_and_map", &SymmHeap::exchange_and_map, py::call_guard<py::gil_scoped_release>())
      .def("multicast_setup", &SymmHeap::multicast_setup, py::call_guard<py::gil_scoped_release>())
      .def("multicast_bind", &SymmHeap::multicast_bind)
      .def("create_ipc", &SymmHeap::create_ipc)
      .def("ipc_handle", [](SymmHeap& h) { return py::bytes(h.ipc_handle()); })
      .def("map_ipc",
           [](SymmHeap& h, const std::vector<py::bytes>& hs) {
             std::vector<std::string> v;
             for (auto& b : hs) v.push_back(std::string(b));
             h.map_ipc(v);
           })
      .def("destroy", &SymmHeap::destroy)
      .def("alloc", &SymmHeap::alloc, py::arg("bytes"), py::arg("align") = 256)
      .def("free", &SymmHeap::free)
      .def("tensor", &heap_tensor, py::arg("offset"), py::arg("sizes"), py::arg("dtype"), py::arg("peer") = -1,
           py::arg("multicast") = false)
      .def("offset_of", &heap_offset_of)
      .def("read_status", &read_status)
      .def("clear_status", &clear_status)
      .def("set_abort", &set_abort)
      .def_property_readonly("local_base", &SymmHeap::local_base)
      .def("peer_base", &SymmHeap::peer_base)
      .def_property_readonly("mc_base", &SymmHeap::mc_base)
      .def_property_readonly("heap_bytes", &SymmHeap::heap_bytes)
      .def_property_readonly("has_multicast", &SymmHeap::has_multicast)
      .def_property_readonly("rank", &SymmHeap::rank)
      .def_property_readonly("world", &SymmHeap::world)
      .def_property_readonly("bytes_in_use", &SymmHeap::bytes_in_use)
      .def_property_readonly("mode", &SymmHeap::mode);

  m.def("stream_write_value32", [](uint64_t addr, uint32_t v) {
    TORCH_CHECK(tdb::stream_write_value32(addr, v, cur_stream()) == 0, "cuStreamWriteValue32 failed");
  });
  m.def("stream_wait_value32", [](uint64_t addr, uint32_t v, bool geq) {
    const int r = geq ? tdb::stream_wait_value32_geq(addr, v, cur_stream()) : tdb::stream_wait_value32_eq(addr, v, cur_stream());
    TORCH_CHECK(r == 0, "cuStreamWaitValue32 failed");
  });

  m.def("gemm_bf16", &gemm_bf16, py::arg("a"), py::arg("b"), py::arg("c"), py::arg("block_n") = 0,
        py::arg("num_ctas") = 0, py::arg("stats") = py::none());
  m.def("ag_gemm_bf16", &ag_gemm_bf16, py::arg("heap"), py::arg("a_local"), py::arg("b"), py::arg("c"), py::arg("ws"),
        py::arg("flags"), py::arg("ctx"), py::arg("max_seg_rows"), py::arg("max_chunks"), py::arg("n_comm"),
        py::arg("block_n"), py::arg("num_ctas"), py::arg("use_multimem"), py::arg("timeout_s"),
        py::arg("stats") = py::none());
  m.def("gemm_rs_bf16", &gemm_rs_bf16, py::arg("heap"), py::arg("a"), py::arg("b"), py::arg("out"), py::arg("slots"),
        py::arg("flags"), py::arg("ctx"), py::arg("max_seg_rows"), py::arg("max_tiles"), py::arg("block_n"),
        py::arg("num_ctas"), py::arg("timeout_s"), py::arg("stats") = py::none());
  m.def("gemm_fp8", &gemm_fp8, py::arg("a_q"), py::arg("a_s"), py::arg("b_q"), py::arg("b_s"), py::arg("c"),
        py::arg("num_ctas") = 0, py::arg("stats") = py::none());
  m.def("ag_gemm_fp8", &ag_gemm_fp8, py::arg("heap"), py::arg("a_q"), py::arg("a_s"), py::arg("b_q"), py::arg("b_s"),
        py::arg("c"), py::arg("ws"), py::arg("ws_scales"), py::arg("flags"), py::arg("ctx"), py::arg("max_seg_rows"),
        py::arg("max_chunks"), py::arg("n_comm"), py::arg("num_ctas"), py::arg("timeout_s"), py::arg("stats") = py::none());
  m.def("gemm_rs_fp8", &gemm_rs_fp8, py::arg("heap"), py::arg("a_q"), py::arg("a_s"), py::arg("b_q"), py::arg("b_s"),
        py::arg("out"), py::arg("slots"), py::arg("flags"), py::arg("ctx"), py::arg("max_seg_rows"), py::arg("max_tiles"),
        py::arg("num_ctas"), py::arg("timeout_s"), py::arg("stats") = py::none());
  m.def("gemm_smem_bytes", &tdb::gemm_smem_bytes);
  m.def("skinny_gemm_bf16", &skinny_gemm_bf16, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("acc"),
        py::arg("counters"), py::arg("splits"), py::arg("num_ctas"), py::arg("cluster_nt") = 0, py::arg("cluster_s") = 0,
        py::arg("bulk_exchange") = 0);
  m.def("gemm_ar_bf16", &gemm_ar_bf16, py::arg("heap"), py::arg("x"), py::arg("w"), py::arg("out"), py::arg("acc"),
        py::arg("counters"), py::arg("partial"), py::arg("flags"), py::arg("ctx"), py::arg("m_cap"), py::arg("max_tiles"),
        py::arg("splits"), py::arg("num_ctas"), py::arg("use_multimem"), py::arg("timeout_s"), py::arg("cluster_nt") = 0,
        py::arg("cluster_s") = 0, py::arg("bulk_exchange") = 0);
  m.def("skinny_gemm_pick_splits", &tdb::skinny_gemm_pick_splits);
  m.def("gemv_bf16", &gemv_bf16, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("norm_w") = py::none(),
        py::arg("eps") = 1e-6, py::arg("silu_mul") = false, py::arg("residual") = py::none(), py::arg("num_ctas") = 0);
  m.def("gemv_ar_bf16", &gemv_ar_bf16);
  m.def("gemv_max_k", &tdb::gemv_max_k);
  bind_more(m);
}
