// Persistent decode megakernel: one launch runs a whole decoder step (all layers) as a statically scheduled list of
// tile tasks per SM - RMSNorm (+ residual), tcgen05 linear tiles with split-K and fused NVLS / push all-reduce,
// QK-RMSNorm + RoPE + KV-cache write, split-KV attention and its combine, SiLU * up - with dependencies resolved
// through a scoreboard of counters in global memory.
//
// One CTA per SM, 192 threads.  For a linear task warp 0 is the TMA producer, warp 1 issues tcgen05.mma, warps 2-5 are
// the epilogue (same roles and barriers as the stand-alone small-M GEMM, kept alive across tasks); for attention
// tasks warps 0-3 run the split-KV step; the element-wise tasks use all threads.  TMEM (accumulators) is allocated
// once for the lifetime of the kernel.  Every wait (scoreboard, mbarrier, cross-rank flag) is bounded.
//
// Reference behaviour being matched (not its code): mega_triton_kernel/core/{task_base,graph,scheduler,code_generator}.py
// (task graph, per-SM static queues, scoreboard), kernels/task_context.py:88-151 (wait_deps / release_tile),
// kernels/{linear,norm,flash_decode,activation,allreduce}.py (the task bodies), models/model_builder.py:508-584.
#include <cuda.h>

#include "tdb/attn_device.cuh"
#include "tdb/launch.cuh"
#include "tdb/mega.h"
#include "tdb/profiler.cuh"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kTN = 128;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
// shared-memory barrier waits follow the configured wait limit of the launch (symm.timeout_ns, TDB200_WAIT_TIMEOUT_S)
#define kMbarTimeoutNs (p.symm.timeout_ns)

template <int MPAD>
struct Layout {
  static constexpr int kWBytes = kTN * kBK * 2;
  static constexpr int kXBytesRaw = MPAD * kBK * 2;
  static constexpr int kXBytes = (kXBytesRaw + 1023) / 1024 * 1024;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = (196 * 1024) / kStageBytes > 10 ? 10 : (196 * 1024) / kStageBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 64;
  static constexpr int kTmemCols = (2 * MPAD) < 32 ? 32 : 2 * MPAD;
};

struct KP {
  const MegaTask* tasks;
  const int32_t* queue_offsets;   // [grid + 1]
  const MegaOp* ops;
  const CUtensorMap* tmaps;
  int32_t* scoreboard;
  float* acc;                     // fp32 [batch_cap, max N] split-K accumulator (zero between uses)
  uint32_t* counters;             // [max tiles]
  CtxDev* ctx;
  SymmInfo symm;
  int batch;
  int use_mc;
  ProfilerBuf prof;
};

TDB_DEVICE void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
TDB_DEVICE void attn_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

TDB_DEVICE float block_sum_192(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}

// ---- element-wise task bodies -------------------------------------------------------------------------------------
// RMSNorm of row a0: out = norm(x (+ residual)) * w; residual (if any) updated in place.
TDB_DEVICE void task_rmsnorm(const MegaOp& op, int row, float* red) {
  const int H = op.i[0];
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(op.p[0]) + static_cast<int64_t>(row) * op.i[1];
  __nv_bfloat16* res = op.p[1] ? reinterpret_cast<__nv_bfloat16*>(op.p[1]) + static_cast<int64_t>(row) * H : nullptr;
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(op.p[2]);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.p[3]) + static_cast<int64_t>(row) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < (H >> 3); i += kThreads) {
    uint4 u = reinterpret_cast<const uint4*>(x)[i];
    float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    if (res) {
      const uint4 r = reinterpret_cast<const uint4*>(res)[i];
      const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
      u.x = pack_bf16x2(f0.x + r0.x, f0.y + r0.y); u.y = pack_bf16x2(f1.x + r1.x, f1.y + r1.y);
      u.z = pack_bf16x2(f2.x + r2.x, f2.y + r2.y); u.w = pack_bf16x2(f3.x + r3.x, f3.y + r3.y);
      reinterpret_cast<uint4*>(res)[i] = u;
      f0 = unpack_bf16x2(u.x); f1 = unpack_bf16x2(u.y); f2 = unpack_bf16x2(u.z); f3 = unpack_bf16x2(u.w);
    }
    ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
  }
  const float inv = rsqrtf(block_sum_192(ss, red) / H + op.f[0]);
  const __nv_bfloat16* src = res ? res : x;   // the summed row when a residual is present (written above by this thread)
  for (int i = threadIdx.x; i < (H >> 3); i += kThreads) {
    const uint4 u = reinterpret_cast<const uint4*>(src)[i], g = reinterpret_cast<const uint4*>(w)[i];
    const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    uint4 o;
    o.x = pack_bf16x2(f0.x * inv * g0.x, f0.y * inv * g0.y); o.y = pack_bf16x2(f1.x * inv * g1.x, f1.y * inv * g1.y);
    o.z = pack_bf16x2(f2.x * inv * g2.x, f2.y * inv * g2.y); o.w = pack_bf16x2(f3.x * inv * g3.x, f3.y * inv * g3.y);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

TDB_DEVICE float silu_f(float x) { return x / (1.f + __expf(-x)); }

TDB_DEVICE void task_silu_mul(const MegaOp& op, int row, int chunk) {
  const int I = op.i[0];
  const int nchunks = op.i[2];
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(op.p[0]) + static_cast<int64_t>(row) * op.i[1];
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.p[1]) + static_cast<int64_t>(row) * I;
  const int nv = I >> 3;
  const int per = (nv + nchunks - 1) / nchunks;
  const int v0 = chunk * per, v1 = min(nv, v0 + per);
  for (int i = v0 + threadIdx.x; i < v1; i += kThreads) {
    const uint4 g = reinterpret_cast<const uint4*>(in)[i], u = reinterpret_cast<const uint4*>(in + I)[i];
    const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    const float2 u0 = unpack_bf16x2(u.x), u1 = unpack_bf16x2(u.y), u2 = unpack_bf16x2(u.z), u3 = unpack_bf16x2(u.w);
    uint4 o;
    o.x = pack_bf16x2(silu_f(g0.x) * u0.x, silu_f(g0.y) * u0.y); o.y = pack_bf16x2(silu_f(g1.x) * u1.x, silu_f(g1.y) * u1.y);
    o.z = pack_bf16x2(silu_f(g2.x) * u2.x, silu_f(g2.y) * u2.y); o.w = pack_bf16x2(silu_f(g3.x) * u3.x, silu_f(g3.y) * u3.y);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// QK-RMSNorm + RoPE + KV write of token `t` (all heads): one warp per head.
TDB_DEVICE void task_rope_kv(const MegaOp& op, int t) {
  const int Hq = op.i[0], Hkv = op.i[1], D = op.i[2];
  const int64_t ld = op.i[3];
  const int max_len = op.i[4];
  const __nv_bfloat16* qkv = reinterpret_cast<const __nv_bfloat16*>(op.p[0]);
  const __nv_bfloat16* qw = reinterpret_cast<const __nv_bfloat16*>(op.p[1]);
  const __nv_bfloat16* kw = reinterpret_cast<const __nv_bfloat16*>(op.p[2]);
  __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(op.p[3]);
  __nv_bfloat16* k_cache = reinterpret_cast<__nv_bfloat16*>(op.p[4]);
  __nv_bfloat16* v_cache = reinterpret_cast<__nv_bfloat16*>(op.p[5]);
  const int32_t* kv_off = reinterpret_cast<const int32_t*>(op.p[6]);   // tokens already cached per sequence
  const int lane = threadIdx.x & 31;
  const int half = D >> 1;
  const int pos_i = kv_off[t];
  const float pos = static_cast<float>(pos_i);
  const int64_t slot = static_cast<int64_t>(t) * max_len + pos_i;
  const bool slot_ok = pos_i >= 0 && pos_i < max_len;   // a sequence that is already full writes nothing
  const float eps = op.f[0], log2_theta = op.f[1];
  for (int h = threadIdx.x >> 5; h < Hq + 2 * Hkv; h += kThreads / 32) {
    const __nv_bfloat16* src = qkv + t * ld + static_cast<int64_t>(h) * D;
    if (h >= Hq + Hkv) {
      if (!slot_ok) continue;
      __nv_bfloat16* dst = v_cache + slot * (Hkv * D) + static_cast<int64_t>(h - Hq - Hkv) * D;
      for (int i = lane; i < (D >> 3); i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
      continue;
    }
    const bool is_q = h < Hq;
    if (!is_q && !slot_ok) continue;
    const __nv_bfloat16* wgt = is_q ? qw : kw;
    float ss = 0.f;
    for (int j = lane; j < (half >> 1); j += 32) {
      const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 2 * j));
      const float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + half + 2 * j));
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
    }
    ss = warp_sum(ss);
    const float inv = wgt ? rsqrtf(ss / D + eps) : 1.f;
    __nv_bfloat16* dst = is_q ? q_out + (static_cast<int64_t>(t) * Hq + h) * D
                              : k_cache + slot * (Hkv * D) + static_cast<int64_t>(h - Hq) * D;
    for (int j = lane; j < (half >> 1); j += 32) {
      float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 2 * j));
      float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + half + 2 * j));
      if (wgt) {
        const float2 wa = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(wgt + 2 * j));
        const float2 wb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(wgt + half + 2 * j));
        a.x = __bfloat162float(__float2bfloat16(a.x * inv * wa.x));
        a.y = __bfloat162float(__float2bfloat16(a.y * inv * wa.y));
        b.x = __bfloat162float(__float2bfloat16(b.x * inv * wb.x));
        b.y = __bfloat162float(__float2bfloat16(b.y * inv * wb.y));
      }
      const float f0 = exp2f(-(2.f * (2 * j)) / D * log2_theta), f1 = exp2f(-(2.f * (2 * j + 1)) / D * log2_theta);
      float s0, c0, s1, c1;
      sincosf(pos * f0, &s0, &c0);
      sincosf(pos * f1, &s1, &c1);
      *reinterpret_cast<uint32_t*>(dst + 2 * j) = pack_bf16x2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
      *reinterpret_cast<uint32_t*>(dst + half + 2 * j) = pack_bf16x2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    }
  }
}

// Decode-attention parameters rebuilt from a MegaOp (dense per-sequence cache: page = one sequence).
TDB_DEVICE attn::DecodeParams attn_params(const MegaOp& op, int batch) {
  attn::DecodeParams d;
  d.q = reinterpret_cast<const __nv_bfloat16*>(op.p[0]);
  d.part_out = reinterpret_cast<float*>(op.p[1]);
  d.part_lse = d.part_out + static_cast<int64_t>(batch) * op.i[0] * op.i[3] * op.i[2];
  d.kv_lens = reinterpret_cast<const int32_t*>(op.p[4]);
  d.kv.k = reinterpret_cast<const __nv_bfloat16*>(op.p[2]);
  d.kv.v = reinterpret_cast<const __nv_bfloat16*>(op.p[3]);
  d.kv.block_table = reinterpret_cast<const int32_t*>(op.p[5]);
  d.kv.max_pages = 1;
  d.kv.page_size = op.i[4];
  d.kv.Hkv = op.i[1];
  d.Hq = op.i[0];
  d.group = op.i[0] / op.i[1];
  d.head_chunks = (d.group + 15) / 16;
  d.splits = op.i[3];
  d.scale = op.f[0];
  d.softcap = 0.f;
  return d;
}

TDB_DEVICE void task_attn_combine(const MegaOp& op, int b, int h0, int batch) {
  const int Hq = op.i[0], D = op.i[2], splits = op.i[3];
  const int hper = op.i[5];   // heads per combine task
  const float* part_out = reinterpret_cast<const float*>(op.p[1]);
  const float* part_lse = part_out + static_cast<int64_t>(batch) * Hq * splits * D;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.p[6]);
  const int hbeg = h0 * hper, hend = min(Hq, hbeg + hper);
  for (int idx = threadIdx.x; idx < (hend - hbeg) * D; idx += kThreads) {
    const int h = hbeg + idx / D, d = idx % D;
    const int64_t bh = static_cast<int64_t>(b) * Hq + h;
    float v;
    attn::merge_partials(part_out + bh * splits * D, part_lse + bh * splits, splits, D, d, &v);
    out[bh * D + d] = __float2bfloat16(v);
  }
}

// L2 prefetch of chunk `chunk` of a byte range (the weights of an operator that runs later): the requests are
// asynchronous, the task ends as soon as they are issued.  op.p[0] = base (16-byte aligned), op.i[0..1] = total bytes
// (low / high word), op.i[2] = bytes per chunk (multiple of 2048).
// Reference: mega_triton_kernel/kernels/prefetch.py:31-56.
TDB_DEVICE void task_prefetch(const MegaOp& op, int chunk) {
  const uint64_t total = (static_cast<uint64_t>(static_cast<uint32_t>(op.i[1])) << 32) | static_cast<uint32_t>(op.i[0]);
  const uint64_t per = static_cast<uint32_t>(op.i[2]);
  const uint64_t b0 = static_cast<uint64_t>(chunk) * per;
  const uint64_t b1 = b0 + per < total ? b0 + per : total;
  const char* base = reinterpret_cast<const char*>(op.p[0]);
  constexpr uint32_t kPiece = 2048;
  for (uint64_t b = b0 + static_cast<uint64_t>(threadIdx.x) * kPiece; b < b1; b += static_cast<uint64_t>(kThreads) * kPiece) {
    const uint64_t left = b1 - b;
    const uint32_t n = static_cast<uint32_t>(left < kPiece ? (left & ~15ull) : kPiece);
    if (n > 0) prefetch_l2(base + b, n);
  }
}

// Stand-alone all-reduce of columns [chunk * cc, ...) of a [batch, N] bf16 tensor (sum over ranks), for partial sums
// that were not produced by a linear task with the fused all-reduce.
//   op.p: 0 x (local), 1 partial (heap; push: [W][batch][N], NVLS: [batch][N]), 2 flags (heap [W][chunks]), 3 out
//   op.i: 0 N, 1 ld_x, 2 ld_out, 3 columns per chunk (multiple of 8), 4 chunks
// Push: the chunk goes into slot [rank] of every rank's partial buffer, then the call epoch into flag [rank][chunk] of
// every rank; when all W flags of this rank carry the epoch the W slots are summed.  NVLS: the chunk is stored locally
// and summed across ranks by multimem.ld_reduce.  Reference: mega_triton_kernel/kernels/allreduce.py:35-65.
TDB_DEVICE bool task_allreduce(const KP& p, const MegaOp& op, int chunk, uint32_t epoch, volatile int* s_ok) {
  const int W = p.symm.world, rank = p.symm.rank;
  const int N = op.i[0], cc = op.i[3], chunks = op.i[4];
  const int64_t ld_x = op.i[1], ld_out = op.i[2];
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(op.p[0]);
  __nv_bfloat16* partial = reinterpret_cast<__nv_bfloat16*>(op.p[1]);
  uint32_t* flags = reinterpret_cast<uint32_t*>(op.p[2]);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.p[3]);
  const int c0 = chunk * cc, c1 = min(N, c0 + cc);
  const int vec_per_row = (c1 - c0) / 8;
  const int nvec = p.batch * vec_per_row;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    const int m = v / vec_per_row, col = c0 + (v - m * vec_per_row) * 8;
    const uint4 u = ld_v4(x + static_cast<int64_t>(m) * ld_x + col);
    if (p.use_mc) {
      st_v4(partial + static_cast<int64_t>(m) * N + col, u);
    } else {
      __nv_bfloat16* mine = partial + (static_cast<int64_t>(rank) * p.batch + m) * N + col;
      for (int j = 0; j < W; ++j) st_v4(symm_at(p.symm, mine, (rank + j) % W), u);
    }
  }
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < W) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(p.symm, flags + static_cast<int64_t>(rank) * chunks + chunk, (rank + threadIdx.x) % W), epoch);
    if (!wait_until(p.symm, flags + static_cast<int64_t>(threadIdx.x) * chunks + chunk, epoch, kCmpGe, kKernelMega, 60,
                    threadIdx.x, chunk))
      *s_ok = 0;
  }
  __syncthreads();
  if (*s_ok == 0) return false;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    const int m = v / vec_per_row, col = c0 + (v - m * vec_per_row) * 8;
    uint4 o;
    if (p.use_mc) {
      o = multimem_ld_reduce_bf16x8(mc_ptr(p.symm, partial + static_cast<int64_t>(m) * N + col));
    } else {
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int sr = 0; sr < W; ++sr) {
        const uint4 u = ld_relaxed_sys_v4(partial + (static_cast<int64_t>(sr) * p.batch + m) * N + col);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
        a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
      }
      o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]); o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
    }
    st_v4(out + static_cast<int64_t>(m) * ld_out + col, o);
  }
  return true;
}

// Spin (bounded) until scoreboard slot tk.dep_idx has reached tk.dep_need.  One thread.
TDB_DEVICE bool wait_dependency(const KP& p, const MegaTask& tk, int ti) {
  if (tk.dep_idx < 0) return true;
  const uint32_t* sb = reinterpret_cast<const uint32_t*>(p.scoreboard + tk.dep_idx);
  uint32_t v = ld_acquire_gpu(sb);
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(v) < tk.dep_need) {
    // the abort word lives in host memory: look at it (and at the clock) rarely, a read over PCIe is slow
    if ((++spins & 4095u) == 0u && (abort_requested(p.symm) || globaltimer_ns() - t0 > p.symm.timeout_ns)) {
      report(p.symm, kTimeoutFlag, kKernelMega, 1, tk.type, ti, tk.dep_need, (int)v);
      return false;
    }
    v = ld_acquire_gpu(sb);
  }
  return true;
}

template <int MPAD>
__global__ void __launch_bounds__(kThreads, 1) mega_kernel(const KP p) {
  using L = Layout<MPAD>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);
  volatile int* is_last = reinterpret_cast<volatile int*>(tmem_base_smem + 2);
  volatile int* s_wok = reinterpret_cast<volatile int*>(tmem_base_smem + 3);
  __shared__ float red[8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  const int W = p.symm.world, rank = p.symm.rank;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_smem, L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_smem;

  // pipeline state of the linear roles, kept across tasks
  uint32_t it = 0;       // k-block counter of the producer lane / the MMA lane
  int local = 0;         // accumulator-buffer counter of the MMA lane / the epilogue threads

  const int q0 = p.queue_offsets[blockIdx.x], q1 = p.queue_offsets[blockIdx.x + 1];
  for (int ti = q0; ti < q1; ++ti) {
    const MegaTask tk = p.tasks[ti];
    // ---- dependencies
    bool ok = true;
    // A linear task checks its dependency in the producer lane, after the first weight tiles (which depend on nothing)
    // have been requested; every other task type waits here.
    if (threadIdx.x == 0 && tk.type != kTaskLinear) {
      ok = wait_dependency(p, tk, ti);
      // data written through the generic proxy by other SMs may be read by TMA below
      fence_proxy_async();
    }
    if (*abort_flag) ok = false;
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (threadIdx.x == 0) profile_record(p.prof, 0, tk.type, true);
    const MegaOp& op = p.ops[tk.op];

    switch (tk.type) {
      case kTaskRmsNorm:
        task_rmsnorm(op, tk.a0, red);
        break;
      case kTaskSiluMul:
        task_silu_mul(op, tk.a0, tk.a1);
        break;
      case kTaskRopeKv:
        task_rope_kv(op, tk.a0);
        break;
      case kTaskAttnSplit:
        if (threadIdx.x < 128) {
          const attn::DecodeParams d = attn_params(op, p.batch);
          if (op.i[2] == 128) {
            attn::decode_splitkv_body<128>(d, tk.a1, tk.a2, tk.a0, smem, [] { attn_bar(); });
          } else {
            attn::decode_splitkv_body<64>(d, tk.a1, tk.a2, tk.a0, smem, [] { attn_bar(); });
          }
        }
        fence_proxy_async_smem();
        break;
      case kTaskAttnCombine:
        task_attn_combine(op, tk.a0, tk.a1, p.batch);
        break;
      case kTaskPrefetch:
        task_prefetch(op, tk.a0);
        break;
      case kTaskBarrier:
        // op.p[0] = heap flags [W] of this barrier; the call epoch is the value, so nothing is ever reset
        if (W > 1 && !rank_barrier_block(p.symm, reinterpret_cast<uint32_t*>(op.p[0]), epoch, kKernelMega, 50)) *abort_flag = 1;
        break;
      case kTaskAllReduce:
        if (W > 1) {
          if (!task_allreduce(p, op, tk.a0, epoch, s_wok)) *abort_flag = 1;
        } else {
          // one rank: the sum is the input
          const int N = op.i[0], cc = op.i[3];
          const int c0 = tk.a0 * cc, c1 = min(N, c0 + cc);
          const int vec_per_row = (c1 - c0) / 8;
          for (int v = threadIdx.x; v < p.batch * vec_per_row; v += kThreads) {
            const int m = v / vec_per_row, col = c0 + (v - m * vec_per_row) * 8;
            st_v4(reinterpret_cast<__nv_bfloat16*>(op.p[3]) + static_cast<int64_t>(m) * op.i[2] + col,
                  ld_v4(reinterpret_cast<const __nv_bfloat16*>(op.p[0]) + static_cast<int64_t>(m) * op.i[1] + col));
          }
        }
        break;
      case kTaskLinear: {
        // op.i: 0 N, 1 K, 2 splits, 3 tmap_w, 4 tmap_x, 5 ld_out, 6 all_reduce, 7 tiles_n, 8 max_tiles(flags stride)
        // op.p: 0 out, 1 partial (heap, this op's ping-pong buffer), 2 flags (heap [W][max_tiles])
        const int N = op.i[0], K = op.i[1], splits = op.i[2];
        const int nt = tk.a0, sp = tk.a1;
        const int kb_total = (K + kBK - 1) / kBK;
        const int kb_per = (kb_total + splits - 1) / splits;
        const int kb0 = sp * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        const CUtensorMap* tmap_w = p.tmaps + op.i[3];
        const CUtensorMap* tmap_x = p.tmaps + op.i[4];
        const bool ar = op.i[6] != 0 && W > 1;
        const bool direct = (splits == 1 && !ar);
        if (warp == 0) {
          if (lane == 0) {
            // The weight tiles depend on nothing: the first stages are requested before the dependency (which only
            // the activation tile has) is checked, so the DRAM latency of the weights overlaps the wait.
            const int n_pre = min(kb1 - kb0, kStages);
            int issued = 0;
            bool pok = true;
            for (int j = 0; j < n_pre; ++j) {
              const uint32_t itj = it + j;
              const int s = itj % kStages;
              const uint32_t ph = (itj / kStages) & 1;
              if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, kMbarTimeoutNs)) {
                report(p.symm, kTimeoutMbarrier, kKernelMega, 10, -1, s, (int)ph, ti);
                *abort_flag = 1;
                pok = false;
                break;
              }
              mbar_arrive_expect_tx(&full_bar[s], L::kWBytes + L::kXBytesRaw);
              tma_load_2d(smem + s * L::kStageBytes, tmap_w, &full_bar[s], (kb0 + j) * kBK, nt * kTN);
              issued = j + 1;
            }
            if (!wait_dependency(p, tk, ti)) {
              *abort_flag = 1;   // the activation loads below still run (the memory is valid) so that the barriers of
              pok = false;       // the requested stages complete; the MMA lane sees the flag and skips the tile
            }
            fence_proxy_async();
            for (int j = 0; j < issued; ++j) {
              const int s = (it + j) % kStages;
              tma_load_2d(smem + s * L::kStageBytes + L::kWBytes, tmap_x, &full_bar[s], (kb0 + j) * kBK, 0);
            }
            it += issued;
            for (int kb = kb0 + issued; kb < kb1 && pok; ++kb, ++it) {
              const int s = it % kStages;
              const uint32_t ph = (it / kStages) & 1;
              if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, kMbarTimeoutNs)) {
                report(p.symm, kTimeoutMbarrier, kKernelMega, 10, -1, s, (int)ph, ti);
                *abort_flag = 1;
                break;
              }
              uint8_t* sw = smem + s * L::kStageBytes;
              mbar_arrive_expect_tx(&full_bar[s], L::kWBytes + L::kXBytesRaw);
              tma_load_2d(sw, tmap_w, &full_bar[s], kb * kBK, nt * kTN);
              tma_load_2d(sw + L::kWBytes, tmap_x, &full_bar[s], kb * kBK, 0);
            }
          }
        } else if (warp == 1) {
          if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(1u, kTN, MPAD);
            const int b = local & 1;
            const uint32_t aph = (local >> 1) & 1;
            ++local;
            bool mok = mbar_wait(&tmem_empty[b], aph ^ 1, abort_flag, kMbarTimeoutNs);
            if (!mok) report(p.symm, kTimeoutMbarrier, kKernelMega, 20, -1, b, (int)aph, ti);
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + b * MPAD;
            for (int kb = kb0; kb < kb1 && mok; ++kb, ++it) {
              const int s = it % kStages;
              const uint32_t ph = (it / kStages) & 1;
              if (!mbar_wait(&full_bar[s], ph, abort_flag, kMbarTimeoutNs)) {
                report(p.symm, kTimeoutMbarrier, kKernelMega, 21, -1, s, (int)ph, ti);
                mok = false;
                break;
              }
              tc_fence_after_sync();
              const uint32_t sw = smem_u32(smem + s * L::kStageBytes);
              const uint64_t adesc = make_smem_desc_sw128(sw);
              const uint64_t bdesc = make_smem_desc_sw128(sw + L::kWBytes);
#pragma unroll
              for (int k = 0; k < kBK / kUmmaK; ++k)
                umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
              umma_commit(&empty_bar[s]);
            }
            if (mok) umma_commit(&tmem_full[b]); else *abort_flag = 1;
          }
        } else {
          const int q = warp & 3;
          const bool leader = (warp == 2 && lane == 0);
          const int et = threadIdx.x - 64;
          const int b = local & 1;
          const uint32_t aph = (local >> 1) & 1;
          ++local;
          bool eok = mbar_wait(&tmem_full[b], aph, abort_flag, kMbarTimeoutNs);
          if (!eok && lane == 0) report(p.symm, kTimeoutMbarrier, kKernelMega, 30, -1, b, (int)aph, ti);
          if (!eok) *abort_flag = 1;
          tc_fence_after_sync();
          const int n = nt * kTN + q * 32 + lane;
          const bool n_ok = n < N;
          const bool has_k = kb1 > kb0;
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.p[0]);
          const int64_t ld_out = op.i[5];
#pragma unroll 1
          for (int c = 0; c < MPAD / 16 && eok; ++c) {
            uint32_t r[16];
            tmem_ld_32x16(tmem_base + b * MPAD + c * 16 + (static_cast<uint32_t>(q * 32) << 16), r);
            tmem_ld_wait();
            if (!has_k || !n_ok) continue;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = c * 16 + j;
              if (m < p.batch) {
                if (direct) out[static_cast<int64_t>(m) * ld_out + n] = __float2bfloat16(__uint_as_float(r[j]));
                else atomicAdd(p.acc + static_cast<int64_t>(m) * N + n, __uint_as_float(r[j]));
              }
            }
          }
          tc_fence_before_sync();
          mbar_arrive(&tmem_empty[b]);
          bool final_tile = direct;
          if (!direct) {
            __threadfence();
            epi_bar();
            if (leader) {
              const uint32_t prev = atomicAdd(p.counters + nt, 1u);
              *is_last = (prev == static_cast<uint32_t>(splits) - 1) ? 1 : 0;
              if (*is_last) p.counters[nt] = 0;
            }
            epi_bar();
            if (*is_last) {
              __threadfence();
              __nv_bfloat16* partial = reinterpret_cast<__nv_bfloat16*>(op.p[1]);
              __nv_bfloat16* dst = ar ? (p.use_mc ? partial : partial + static_cast<int64_t>(rank) * p.batch * N) : out;
              const int64_t ld_dst = ar ? N : ld_out;
              if (n_ok) {
                for (int m0 = 0; m0 < p.batch; m0 += 8) {
                  float v[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    v[j] = (m0 + j < p.batch) ? __ldcg(p.acc + static_cast<int64_t>(m0 + j) * N + n) : 0.f;
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    if (m0 + j < p.batch) {
                      p.acc[static_cast<int64_t>(m0 + j) * N + n] = 0.f;
                      dst[static_cast<int64_t>(m0 + j) * ld_dst + n] = __float2bfloat16(v[j]);
                    }
                  }
                }
              }
              final_tile = true;
              if (ar) {
                const int tn = min(kTN, N - nt * kTN);
                const int vec_per_row = tn / 8;
                uint32_t* flags = reinterpret_cast<uint32_t*>(op.p[2]);
                const int max_tiles = op.i[8];
                epi_bar();
                if (!p.use_mc) {
                  for (int v = et; v < p.batch * vec_per_row; v += 128) {
                    const int m = v / vec_per_row, cv = v - m * vec_per_row;
                    __nv_bfloat16* src = dst + static_cast<int64_t>(m) * N + nt * kTN + cv * 8;
                    const uint4 u = ld_v4(src);
                    for (int j = 1; j < W; ++j) st_v4(symm_at(p.symm, src, (rank + j) % W), u);
                  }
                  epi_bar();
                }
                bool wok = true;
                if (et < W) {
                  fence_acq_rel_sys();
                  st_release_sys(symm_at(p.symm, flags + static_cast<int64_t>(rank) * max_tiles + nt, (rank + et) % W), epoch);
                  wok = wait_until(p.symm, flags + static_cast<int64_t>(et) * max_tiles + nt, epoch, kCmpGe, kKernelMega, 40, et, nt);
                }
                if (et == 0) *s_wok = 1;
                epi_bar();
                if (!wok) *s_wok = 0;
                epi_bar();
                if (*s_wok == 0) {
                  *abort_flag = 1;
                  final_tile = false;
                } else {
                  for (int v = et; v < p.batch * vec_per_row; v += 128) {
                    const int m = v / vec_per_row, cv = v - m * vec_per_row;
                    const int col = nt * kTN + cv * 8;
                    uint4 o;
                    if (p.use_mc) {
                      o = multimem_ld_reduce_bf16x8(mc_ptr(p.symm, partial + static_cast<int64_t>(m) * N + col));
                    } else {
                      float accv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                      for (int s = 0; s < W; ++s) {
                        const uint4 u = ld_relaxed_sys_v4(partial + (static_cast<int64_t>(s) * p.batch + m) * N + col);
                        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
                        accv[0] += f0.x; accv[1] += f0.y; accv[2] += f1.x; accv[3] += f1.y;
                        accv[4] += f2.x; accv[5] += f2.y; accv[6] += f3.x; accv[7] += f3.y;
                      }
                      o.x = pack_bf16x2(accv[0], accv[1]); o.y = pack_bf16x2(accv[2], accv[3]);
                      o.z = pack_bf16x2(accv[4], accv[5]); o.w = pack_bf16x2(accv[6], accv[7]);
                    }
                    st_v4(out + static_cast<int64_t>(m) * ld_out + col, o);
                  }
                }
              }
            }
          }
          // publish the finished output tile
          if (final_tile && tk.out_idx >= 0) {
            __threadfence();
            epi_bar();
            if (leader) red_release_gpu_add(reinterpret_cast<uint32_t*>(p.scoreboard + tk.out_idx), 1u);
          }
        }
        break;
      }
      default:
        break;
    }
    // ---- end of task
    __syncthreads();
    if (threadIdx.x == 0) {
      profile_record(p.prof, 0, tk.type, false);
      if (tk.type != kTaskLinear && tk.out_idx >= 0) {
        __threadfence();
        red_release_gpu_add(reinterpret_cast<uint32_t*>(p.scoreboard + tk.out_idx), 1u);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(&p.ctx->done, 1u);
    if (prev == gridDim.x - 1) {
      p.ctx->done = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
    }
  }
}

template <int MPAD>
cudaError_t launch_t(const KP& p, int grid, cudaStream_t stream) {
  using L = Layout<MPAD>;
  const int smem = L::kTotal + 1024;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(mega_kernel<MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    set = true;
  }
  // every CTA waits on scoreboard counters that other CTAs of the launch bump: all of them must be resident
  return launch_coop(mega_kernel<MPAD>, dim3(grid), dim3(kThreads), static_cast<size_t>(smem), stream, p);
}

}  // namespace

cudaError_t launch_megakernel(const MegaLaunchArgs& a, cudaStream_t stream) {
  if (a.batch < 1 || a.batch > 64) return cudaErrorInvalidValue;
  KP p;
  p.tasks = a.tasks;
  p.queue_offsets = a.queue_offsets;
  p.ops = a.ops;
  p.tmaps = reinterpret_cast<const CUtensorMap*>(a.tmaps);
  p.scoreboard = a.scoreboard;
  p.acc = a.acc;
  p.counters = a.counters;
  p.ctx = a.ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &a.symm, sizeof(SymmInfo));
  p.batch = a.batch;
  p.use_mc = (a.use_multimem && a.symm.mc_base != 0) ? 1 : 0;
  p.prof.buf = reinterpret_cast<unsigned long long*>(a.profile_buf);
  cudaError_t e = cudaMemsetAsync(a.scoreboard, 0, sizeof(int32_t) * a.scoreboard_size, stream);
  if (e != cudaSuccess) return e;
  const int mpad = a.batch <= 16 ? 16 : a.batch <= 32 ? 32 : 64;
  if (mpad == 16) return launch_t<16>(p, a.grid, stream);
  if (mpad == 32) return launch_t<32>(p, a.grid, stream);
  return launch_t<64>(p, a.grid, stream);
}

int megakernel_mpad(int batch) { return batch <= 16 ? 16 : batch <= 32 ? 32 : 64; }

}  // namespace tdb
