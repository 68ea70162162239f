// Gated delta rule (Gated DeltaNet linear attention), forward, variable-length batches.
//
// Per head the state S [K x V] evolves token by token:
//     S  <- exp(g_t) * S
//     v' =  beta_t * (v_t - S^T k_t)
//     S  <- S + k_t v'^T
//     o_t = scale * S^T q_t
// The reference computes this in chunks of 64 tokens with three Triton kernels (WY representation: a triangular
// solve per chunk, a sequential pass over chunk states, an output pass; python/triton_dist/kernels/nvidia/gdn.py:123,
// :482, :785, entry point :926).  Here one kernel walks the tokens with the state held in registers: a CTA owns 32
// columns of V of one (sequence, head); every column is shared by four lanes that each keep 32 of the 128 rows of
// K (32 registers), so a token costs about a hundred FMAs, a few shared-memory reads and two shuffle reductions per
// thread, and nothing is written back but o_t.  q, k, v, g, beta of 64 tokens at a time are staged in shared memory
// with cp.async, double buffered.  The state never leaves the chip, which is what the chunked form spends its three
// passes on; the price is that the tensor cores are idle, so long sequences run at CUDA-core FMA rate.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "tdb/gdn.h"

namespace tdb {

namespace {

constexpr int kK = 128;           // head dim of q / k
constexpr int kVT = 32;           // V columns per CTA
constexpr int kParts = 4;         // lanes sharing a column (K split)
constexpr int kKP = kK / kParts;  // rows of K per lane
constexpr int kThreads = kVT * kParts;
constexpr int kChunk = 64;

struct Stage {
  __nv_bfloat16 q[kChunk][kK];
  __nv_bfloat16 k[kChunk][kK];
  __nv_bfloat16 v[kChunk][kVT];
  float g[kChunk];
  float beta[kChunk];
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

struct Params {
  const __nv_bfloat16* q;     // [T_total, H, K]
  const __nv_bfloat16* k;     // [T_total, H, K]
  const __nv_bfloat16* v;     // [T_total, H, V]
  const float* g;             // [T_total, H]  log decay (<= 0)
  const __nv_bfloat16* beta;  // [T_total, H]
  __nv_bfloat16* o;           // [T_total, H, V]
  const float* h0;            // [N, H, K, V] or null
  float* ht;                  // [N, H, K, V] or null
  const int32_t* cu_seqlens;  // [N + 1]
  int H, V;
  float scale;
};

__device__ void load_chunk(const Params& p, Stage& s, int64_t t0, int n, int h, int v0) {
  // q, k: n rows of 256 bytes; v: n rows of 64 bytes; g, beta: scalars
  for (int i = threadIdx.x; i < n * (kK / 8); i += kThreads) {
    const int r = i / (kK / 8), c = i % (kK / 8);
    const int64_t row = (t0 + r) * p.H + h;
    cp_async16(&s.q[r][c * 8], p.q + row * kK + c * 8);
    cp_async16(&s.k[r][c * 8], p.k + row * kK + c * 8);
  }
  for (int i = threadIdx.x; i < n * (kVT / 8); i += kThreads) {
    const int r = i / (kVT / 8), c = i % (kVT / 8);
    cp_async16(&s.v[r][c * 8], p.v + ((t0 + r) * p.H + h) * p.V + v0 + c * 8);
  }
  for (int i = threadIdx.x; i < n; i += kThreads) {
    s.g[i] = p.g[(t0 + i) * p.H + h];
    s.beta[i] = __bfloat162float(p.beta[(t0 + i) * p.H + h]);
  }
}

__global__ void __launch_bounds__(kThreads) gdn_fwd_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  Stage* st = reinterpret_cast<Stage*>(smem_raw);
  const int vt = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int v0 = vt * kVT;
  const int col = threadIdx.x / kParts;     // column of V inside the tile
  const int part = threadIdx.x % kParts;    // which quarter of K (adjacent lanes share a column)
  const int64_t t_begin = p.cu_seqlens[seq], t_end = p.cu_seqlens[seq + 1];
  const int T = static_cast<int>(t_end - t_begin);

  float S[kKP];
  const int64_t state_off = ((static_cast<int64_t>(seq) * p.H + h) * kK + part * kKP) * p.V + v0 + col;
#pragma unroll
  for (int i = 0; i < kKP; ++i) S[i] = p.h0 ? p.h0[state_off + static_cast<int64_t>(i) * p.V] : 0.f;

  const int nchunks = (T + kChunk - 1) / kChunk;
  if (nchunks > 0) load_chunk(p, st[0], t_begin, min(kChunk, T), h, v0);
  cp_async_commit();
  for (int c = 0; c < nchunks; ++c) {
    Stage& cur = st[c & 1];
    if (c + 1 < nchunks)
      load_chunk(p, st[(c + 1) & 1], t_begin + static_cast<int64_t>(c + 1) * kChunk, min(kChunk, T - (c + 1) * kChunk), h, v0);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int n = min(kChunk, T - c * kChunk);
    for (int t = 0; t < n; ++t) {
      const float decay = __expf(cur.g[t]);
      const float bt = cur.beta[t];
      const float vt_val = __bfloat162float(cur.v[t][col]);
      const __nv_bfloat162* kr = reinterpret_cast<const __nv_bfloat162*>(&cur.k[t][part * kKP]);
      const __nv_bfloat162* qr = reinterpret_cast<const __nv_bfloat162*>(&cur.q[t][part * kKP]);
      float kf[kKP];
      float r = 0.f;
#pragma unroll
      for (int i = 0; i < kKP / 2; ++i) {
        const float2 kk = __bfloat1622float2(kr[i]);
        kf[2 * i] = kk.x;
        kf[2 * i + 1] = kk.y;
        S[2 * i] *= decay;
        S[2 * i + 1] *= decay;
        r = fmaf(S[2 * i], kk.x, r);
        r = fmaf(S[2 * i + 1], kk.y, r);
      }
      r += __shfl_xor_sync(0xffffffffu, r, 1);
      r += __shfl_xor_sync(0xffffffffu, r, 2);
      const float vn = bt * (vt_val - r);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < kKP / 2; ++i) {
        const float2 qq = __bfloat1622float2(qr[i]);
        S[2 * i] = fmaf(kf[2 * i], vn, S[2 * i]);
        S[2 * i + 1] = fmaf(kf[2 * i + 1], vn, S[2 * i + 1]);
        o = fmaf(S[2 * i], qq.x, o);
        o = fmaf(S[2 * i + 1], qq.y, o);
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (part == 0)
        p.o[((t_begin + static_cast<int64_t>(c) * kChunk + t) * p.H + h) * p.V + v0 + col] = __float2bfloat16(o * p.scale);
    }
    __syncthreads();   // the next load overwrites the stage that was just read
  }
  cp_async_wait<0>();
  if (p.ht != nullptr) {
#pragma unroll
    for (int i = 0; i < kKP; ++i) p.ht[state_off + static_cast<int64_t>(i) * p.V] = S[i];
  }
}

}  // namespace

cudaError_t launch_gdn_fwd(const GdnArgs& a, cudaStream_t stream) {
  if (a.K != kK || a.V % kVT != 0 || a.num_seqs < 1) return cudaErrorInvalidValue;
  Params p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.k = reinterpret_cast<const __nv_bfloat16*>(a.k);
  p.v = reinterpret_cast<const __nv_bfloat16*>(a.v);
  p.g = a.g;
  p.beta = reinterpret_cast<const __nv_bfloat16*>(a.beta);
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o);
  p.h0 = a.initial_state;
  p.ht = a.final_state;
  p.cu_seqlens = a.cu_seqlens;
  p.H = a.H;
  p.V = a.V;
  p.scale = a.scale;
  const int smem = 2 * static_cast<int>(sizeof(Stage));
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(gdn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    set = true;
  }
  dim3 grid(a.V / kVT, a.H, a.num_seqs);
  gdn_fwd_kernel<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace tdb
