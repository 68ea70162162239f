// Gated delta rule forward in the chunk-parallel WY form on tensor cores (64-token chunks, K = 128).
//
// Per chunk (rows i, j of one chunk, gc = chunk-local cumulative log decay):
//     L[i][j] = beta_i (k_i . k_j) exp(gc_i - gc_j)        for i > j, else 0
//     A       = (I + L)^-1                                  (unit lower triangular)
//     w       = A (beta k exp(gc)),   u = A (beta v)
// then, sequentially over the chunks of a sequence with the state S [K x V] at the start of the chunk:
//     v_new   = u - w S
//     S      <- S exp(gc_last) + (k exp(gc_last - gc))^T v_new
// and per chunk again:
//     o       = scale [ (q exp(gc)) S + tril(q k^T exp(gc_i - gc_j)) v_new ]
//
// Three kernels, as in the reference (python/triton_dist/kernels/nvidia/gdn.py:123 scaled-dot KK^T + :300 solve +
// :482 recompute w/u, :620 chunk state pass, :785 output; entry point :926):
//   gdn_chunk_prepare   grid (chunks, H): KK^T on tensor cores, forward substitution in shared memory, w / u on tensor cores
//   gdn_chunk_state     grid (V / 64, H, sequences): walks the chunks with S in shared memory (fp32), two tensor-core
//                       products per chunk; writes v_new and the chunk-start states (bf16)
//   gdn_chunk_output    grid (chunks, H, V / 64): q k^T, masking / decay, two tensor-core products
// Tensor-core products use the warp-level bf16 MMA (fragments through nvcuda::wmma, fp32 accumulation): 64 x 64 x 128
// problems are too small for a tcgen05 / TMEM pipeline to pay.  Intermediates (w, u, v_new) live in a chunk-major layout
// [chunk][H][64][*] whose padded rows are zero, so no kernel reads past a sequence end.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <mma.h>

#include <cstdint>

#include "tdb/gdn.h"
#include "tdb/launch.cuh"

namespace tdb {

namespace {

using namespace nvcuda;

constexpr int kC = 64;            // chunk length
constexpr int kK = 128;           // head dim of q / k
constexpr int kVT = 64;           // V columns per CTA in the state / output kernels
constexpr int kThreads = 128;     // four warps, each owns 16 chunk rows
constexpr int kLdK = kK + 8;      // bf16 row pitch of [64][128] tiles (272 bytes: 32-byte aligned 16-row tiles, no bank conflicts)
constexpr int kLdC = kC + 8;      // bf16 row pitch of [*][64] tiles
constexpr int kLdF = kC + 4;      // fp32 row pitch of [*][64] tiles

using FragA = wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major>;
using FragAT = wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::col_major>;
using FragB = wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::row_major>;
using FragBT = wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major>;
using FragC = wmma::fragment<wmma::accumulator, 16, 16, 16, float>;

struct ChunkParams {
  const __nv_bfloat16* q;       // [T, H, K]
  const __nv_bfloat16* k;       // [T, H, K]
  const __nv_bfloat16* v;       // [T, H, V]
  const float* g;               // [T, H]
  const __nv_bfloat16* beta;    // [T, H]
  const int32_t* cu_seqlens;    // [N + 1]
  const int32_t* chunk_seq;     // [NC] sequence of every chunk
  const int32_t* chunk_t0;      // [NC] first token of every chunk
  const int32_t* seq_chunk0;    // [N + 1] first chunk of every sequence
  float* gcum;                  // [T, H] chunk-local cumulative log decay
  float* a_out;                 // [T, H, 64] or null
  __nv_bfloat16* w;             // [NC, H, 64, K]
  __nv_bfloat16* u;             // [NC, H, 64, V]
  __nv_bfloat16* vnew;          // [NC, H, 64, V]
  __nv_bfloat16* hstate;        // [NC, H, K, V] state at the start of every chunk
  const float* h0;              // [N, H, K, V] or null
  float* ht;                    // [N, H, K, V] or null
  __nv_bfloat16* o;             // [T, H, V]
  int H, V, NC;
  float scale;
};

__device__ __forceinline__ int chunk_len(const ChunkParams& p, int c) {
  const int t0 = p.chunk_t0[c];
  const int t_end = p.cu_seqlens[p.chunk_seq[c] + 1];
  return min(kC, t_end - t0);
}

// rows [0, n) of a token-major [T, H, cols] tensor into a padded shared tile, zero beyond n
__device__ __forceinline__ void load_rows(__nv_bfloat16* dst, int ld, const __nv_bfloat16* src, int64_t t0, int n, int H, int h,
                                          int cols, int col0, int ncols) {
  const int vec = ncols / 8;
  for (int i = threadIdx.x; i < kC * vec; i += kThreads) {
    const int r = i / vec, c = (i - r * vec) * 8;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < n) val = *reinterpret_cast<const uint4*>(src + ((t0 + r) * H + h) * cols + col0 + c);
    *reinterpret_cast<uint4*>(dst + r * ld + c) = val;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Kernel 1: per (chunk, head)
// ------------------------------------------------------------------------------------------------------------------
struct PrepSmem {
  __nv_bfloat16 k[kC][kLdK];
  __nv_bfloat16 kb[kC][kLdK];     // beta k, later beta k exp(gc)
  float L[kC][kLdF];              // strictly lower part of the system, later staging of output tiles
  float A[kC][kLdF];              // (I + L)^-1
  __nv_bfloat16 Ab[kC][kLdC];
  float gc[kC];
  float beta[kC];
  // followed by vb [64][V + 8] bf16
};

__global__ void __launch_bounds__(kThreads) gdn_chunk_prepare(const ChunkParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  PrepSmem& s = *reinterpret_cast<PrepSmem*>(smem_raw);
  __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>(smem_raw + sizeof(PrepSmem));
  const int ldv = p.V + 8;
  const int c = blockIdx.x, h = blockIdx.y;
  const int64_t t0 = p.chunk_t0[c];
  const int n = chunk_len(p, c);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  load_rows(&s.k[0][0], kLdK, p.k, t0, n, p.H, h, kK, 0, kK);
  load_rows(vb, ldv, p.v, t0, n, p.H, h, p.V, 0, p.V);
  if (threadIdx.x < kC) {
    const int r = threadIdx.x;
    s.beta[r] = r < n ? __bfloat162float(p.beta[(t0 + r) * p.H + h]) : 0.f;
    s.gc[r] = r < n ? p.g[(t0 + r) * p.H + h] : 0.f;
  }
  __syncthreads();
  if (warp == 0) {
    // inclusive scan of 64 values by one warp: two per lane
    float a = s.gc[2 * lane], b = s.gc[2 * lane + 1];
    float sum = a + b, pre = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, pre, o);
      if (lane >= o) pre += t;
    }
    const float base = pre - sum;
    s.gc[2 * lane] = base + a;
    s.gc[2 * lane + 1] = base + a + b;
  }
  __syncthreads();
  if (threadIdx.x < n) p.gcum[(t0 + threadIdx.x) * p.H + h] = s.gc[threadIdx.x];
  // kb = beta k, vb = beta v
  for (int i = threadIdx.x; i < kC * (kK / 2); i += kThreads) {
    const int r = i / (kK / 2), cc = (i - r * (kK / 2)) * 2;
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&s.k[r][cc]));
    *reinterpret_cast<__nv_bfloat162*>(&s.kb[r][cc]) = __floats2bfloat162_rn(f.x * s.beta[r], f.y * s.beta[r]);
  }
  for (int i = threadIdx.x; i < kC * (p.V / 2); i += kThreads) {
    const int r = i / (p.V / 2), cc = (i - r * (p.V / 2)) * 2;
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vb + r * ldv + cc));
    *reinterpret_cast<__nv_bfloat162*>(vb + r * ldv + cc) = __floats2bfloat162_rn(f.x * s.beta[r], f.y * s.beta[r]);
  }
  __syncthreads();
  // L = (beta k) k^T: warp w owns rows [16 w, 16 w + 16)
  {
    FragC acc[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::fill_fragment(acc[nt], 0.f);
    for (int ks = 0; ks < kK / 16; ++ks) {
      FragA a;
      wmma::load_matrix_sync(a, &s.kb[16 * warp][16 * ks], kLdK);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        FragBT b;   // B[kk][nn] = k[16 nt + nn][16 ks + kk]
        wmma::load_matrix_sync(b, &s.k[16 * nt][16 * ks], kLdK);
        wmma::mma_sync(acc[nt], a, b, acc[nt]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::store_matrix_sync(&s.L[16 * warp][16 * nt], acc[nt], kLdF, wmma::mem_row_major);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kC * kC; i += kThreads) {
    const int r = i / kC, cc = i - r * kC;
    s.L[r][cc] = (r > cc) ? s.L[r][cc] * __expf(s.gc[r] - s.gc[cc]) : 0.f;
  }
  __syncthreads();
  // (I + L) A = I by forward substitution; thread j < 64 owns column j of A (its first j rows are zero)
  if (threadIdx.x < kC) {
    const int j = threadIdx.x;
    for (int i = 0; i < kC; ++i) {
      float acc = (i == j) ? 1.f : 0.f;
      for (int m = j; m < i; ++m) acc -= s.L[i][m] * s.A[m][j];
      s.A[i][j] = (i >= j) ? acc : 0.f;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kC * kC; i += kThreads) {
    const int r = i / kC, cc = i - r * kC;
    s.Ab[r][cc] = __float2bfloat16(s.A[r][cc]);
    if (p.a_out != nullptr && r < n) p.a_out[((t0 + r) * p.H + h) * kC + cc] = s.A[r][cc];
  }
  // kb <- beta k exp(gc)
  for (int i = threadIdx.x; i < kC * (kK / 2); i += kThreads) {
    const int r = i / (kK / 2), cc = (i - r * (kK / 2)) * 2;
    const float e = __expf(s.gc[r]);
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&s.kb[r][cc]));
    *reinterpret_cast<__nv_bfloat162*>(&s.kb[r][cc]) = __floats2bfloat162_rn(f.x * e, f.y * e);
  }
  __syncthreads();
  // w = A kb  [64 x 128],  u = A vb  [64 x V]; 64 output columns at a time through the warp's rows of L (staging)
  __nv_bfloat16* wout = p.w + (static_cast<int64_t>(c) * p.H + h) * kC * kK;
  __nv_bfloat16* uout = p.u + (static_cast<int64_t>(c) * p.H + h) * kC * p.V;
  const int passes_w = kK / 64, passes_u = p.V / 64;
  for (int ps = 0; ps < passes_w + passes_u; ++ps) {
    const bool is_w = ps < passes_w;
    const int col0 = (is_w ? ps : ps - passes_w) * 64;
    const __nv_bfloat16* bsrc = is_w ? &s.kb[0][0] : vb;
    const int ldb = is_w ? kLdK : ldv;
    FragC acc[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::fill_fragment(acc[nt], 0.f);
    for (int ks = 0; ks < kC / 16; ++ks) {
      FragA a;
      wmma::load_matrix_sync(a, &s.Ab[16 * warp][16 * ks], kLdC);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        FragB b;
        wmma::load_matrix_sync(b, bsrc + (16 * ks) * ldb + col0 + 16 * nt, ldb);
        wmma::mma_sync(acc[nt], a, b, acc[nt]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::store_matrix_sync(&s.L[16 * warp][16 * nt], acc[nt], kLdF, wmma::mem_row_major);
    __syncwarp();
    __nv_bfloat16* dst = is_w ? wout : uout;
    const int ldo = is_w ? kK : p.V;
    for (int i = lane; i < 16 * 32; i += 32) {
      const int r = 16 * warp + i / 32, cc = (i % 32) * 2;
      *reinterpret_cast<__nv_bfloat162*>(dst + r * ldo + col0 + cc) = __floats2bfloat162_rn(s.L[r][cc], s.L[r][cc + 1]);
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Kernel 2: per (V tile, head, sequence), sequential over the chunks.  The pass is a chain of small dependent steps, so
// everything a chunk needs from global memory (w, its u slice, k, the cumulative decay) is fetched one chunk ahead with
// cp.async into a second shared-memory stage while the current chunk is computed.
// ------------------------------------------------------------------------------------------------------------------
struct StateStage {
  __nv_bfloat16 w[kC][kLdK];
  __nv_bfloat16 k[kC][kLdK];        // k, turned into k exp(gc_last - gc) in place
  __nv_bfloat16 u[kC][kLdC];
  float gc[kC];
};
struct StateSmem {
  float S[kK][kLdF];                // state columns [v0, v0 + 64)
  __nv_bfloat16 Sb[kK][kLdC];       // bf16 copy for the tensor cores
  float vf[kC][kLdF];               // w S
  __nv_bfloat16 vn[kC][kLdC];       // v_new
  StateStage st[2];
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ void state_prefetch(const ChunkParams& p, StateStage& st, int c, int h, int v0) {
  const int64_t t0 = p.chunk_t0[c];
  const int n = chunk_len(p, c);
  const int64_t ch = static_cast<int64_t>(c) * p.H + h;
  const __nv_bfloat16* wsrc = p.w + ch * kC * kK;
  for (int i = threadIdx.x; i < kC * (kK / 8); i += kThreads) {
    const int r = i / (kK / 8), cc = (i - r * (kK / 8)) * 8;
    cp_async16(&st.w[r][cc], wsrc + r * kK + cc);
    if (r < n) cp_async16(&st.k[r][cc], p.k + ((t0 + r) * p.H + h) * kK + cc);
    else *reinterpret_cast<uint4*>(&st.k[r][cc]) = make_uint4(0u, 0u, 0u, 0u);
  }
  const __nv_bfloat16* usrc = p.u + ch * kC * p.V + v0;
  for (int i = threadIdx.x; i < kC * (kVT / 8); i += kThreads) {
    const int r = i / (kVT / 8), cc = (i - r * (kVT / 8)) * 8;
    cp_async16(&st.u[r][cc], usrc + static_cast<int64_t>(r) * p.V + cc);
  }
  if (threadIdx.x < kC) {
    const int r = min(static_cast<int>(threadIdx.x), n - 1);    // padded rows keep the last value (their g is 0)
    cp_async4(&st.gc[threadIdx.x], p.gcum + (t0 + r) * p.H + h);
  }
}

__global__ void __launch_bounds__(kThreads) gdn_chunk_state(const ChunkParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  StateSmem& s = *reinterpret_cast<StateSmem*>(smem_raw);
  const int vt = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int v0 = vt * kVT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t st_off = (static_cast<int64_t>(seq) * p.H + h) * kK * p.V;
  const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
  if (c_begin < c_end) state_prefetch(p, s.st[0], c_begin, h, v0);
  cp_async_commit();
  for (int i = threadIdx.x; i < kK * kVT; i += kThreads) {
    const int r = i / kVT, cc = i - r * kVT;
    const float val = p.h0 ? p.h0[st_off + static_cast<int64_t>(r) * p.V + v0 + cc] : 0.f;
    s.S[r][cc] = val;
    s.Sb[r][cc] = __float2bfloat16(val);
  }
  for (int c = c_begin; c < c_end; ++c) {
    StateStage& cur = s.st[(c - c_begin) & 1];
    // the other stage was last read two barriers ago (end of the previous iteration)
    if (c + 1 < c_end) state_prefetch(p, s.st[(c - c_begin + 1) & 1], c + 1, h, v0);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();   // stage `cur` (and, in the first iteration, S / Sb) visible to every warp
    const int64_t ch = static_cast<int64_t>(c) * p.H + h;
    // chunk-start state for the output kernel
    {
      __nv_bfloat16* hdst = p.hstate + ch * kK * p.V + v0;
      for (int i = threadIdx.x; i < kK * (kVT / 8); i += kThreads) {
        const int r = i / (kVT / 8), cc = (i - r * (kVT / 8)) * 8;
        *reinterpret_cast<uint4*>(hdst + static_cast<int64_t>(r) * p.V + cc) = *reinterpret_cast<const uint4*>(&s.Sb[r][cc]);
      }
    }
    // vf = w S   (rows of this warp)
    {
      FragC acc[4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) wmma::fill_fragment(acc[nt], 0.f);
#pragma unroll
      for (int ks = 0; ks < kK / 16; ++ks) {
        FragA a;
        wmma::load_matrix_sync(a, &cur.w[16 * warp][16 * ks], kLdK);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          FragB b;
          wmma::load_matrix_sync(b, &s.Sb[16 * ks][16 * nt], kLdC);
          wmma::mma_sync(acc[nt], a, b, acc[nt]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) wmma::store_matrix_sync(&s.vf[16 * warp][16 * nt], acc[nt], kLdF, wmma::mem_row_major);
    }
    __syncwarp();
    const float g_last = cur.gc[kC - 1];
    // v_new = u - w S for the warp's own 16 rows (bf16, to shared and global); k <- k exp(g_last - gc) for the same rows
    {
      __nv_bfloat16* vdst = p.vnew + ch * kC * p.V + v0;
      for (int i = lane; i < 16 * (kVT / 2); i += 32) {
        const int r = 16 * warp + i / (kVT / 2), cc = (i % (kVT / 2)) * 2;
        const float2 uu = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cur.u[r][cc]));
        const __nv_bfloat162 o = __floats2bfloat162_rn(uu.x - s.vf[r][cc], uu.y - s.vf[r][cc + 1]);
        *reinterpret_cast<__nv_bfloat162*>(&s.vn[r][cc]) = o;
        *reinterpret_cast<__nv_bfloat162*>(vdst + static_cast<int64_t>(r) * p.V + cc) = o;
      }
      for (int i = lane; i < 16 * (kK / 2); i += 32) {
        const int r = 16 * warp + i / (kK / 2), cc = (i % (kK / 2)) * 2;
        const float e = __expf(g_last - cur.gc[r]);
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cur.k[r][cc]));
        *reinterpret_cast<__nv_bfloat162*>(&cur.k[r][cc]) = __floats2bfloat162_rn(f.x * e, f.y * e);
      }
    }
    __syncthreads();   // vn and the scaled k of all rows are complete; every warp is done reading Sb
    // S <- S exp(g_last) + kd^T v_new: warp w owns state rows [32 w, 32 w + 32)
    {
      const float dec = __expf(g_last);
#pragma unroll
      for (int rt = 0; rt < 2; ++rt) {
        const int row0 = 32 * warp + 16 * rt;
        FragC acc[4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          wmma::load_matrix_sync(acc[nt], &s.S[row0][16 * nt], kLdF, wmma::mem_row_major);
#pragma unroll
          for (int e = 0; e < acc[nt].num_elements; ++e) acc[nt].x[e] *= dec;
        }
#pragma unroll
        for (int ks = 0; ks < kC / 16; ++ks) {
          FragAT a;   // A[m][kk] = kd[16 ks + kk][row0 + m]
          wmma::load_matrix_sync(a, &cur.k[16 * ks][row0], kLdK);
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            FragB b;
            wmma::load_matrix_sync(b, &s.vn[16 * ks][16 * nt], kLdC);
            wmma::mma_sync(acc[nt], a, b, acc[nt]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) wmma::store_matrix_sync(&s.S[row0][16 * nt], acc[nt], kLdF, wmma::mem_row_major);
      }
      __syncwarp();
      for (int i = lane; i < 32 * (kVT / 2); i += 32) {
        const int r = 32 * warp + i / (kVT / 2), cc = (i % (kVT / 2)) * 2;
        *reinterpret_cast<__nv_bfloat162*>(&s.Sb[r][cc]) = __floats2bfloat162_rn(s.S[r][cc], s.S[r][cc + 1]);
      }
    }
    __syncthreads();   // the new Sb is complete; stage `cur` may be overwritten by the prefetch of the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();
  if (p.ht != nullptr) {
    for (int i = threadIdx.x; i < kK * kVT; i += kThreads) {
      const int r = i / kVT, cc = i - r * kVT;
      p.ht[st_off + static_cast<int64_t>(r) * p.V + v0 + cc] = s.S[r][cc];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Kernel 3: per (chunk, head, V tile)
// ------------------------------------------------------------------------------------------------------------------
struct OutSmem {
  __nv_bfloat16 q[kC][kLdK];
  __nv_bfloat16 k[kC][kLdK];
  float P[kC][kLdF];               // q k^T, later staging of the output tile
  __nv_bfloat16 Pb[kC][kLdC];
  float gc[kC];
};

__global__ void __launch_bounds__(kThreads) gdn_chunk_output(const ChunkParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  OutSmem& s = *reinterpret_cast<OutSmem*>(smem_raw);
  const int c = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kVT;
  const int64_t t0 = p.chunk_t0[c];
  const int n = chunk_len(p, c);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t ch = static_cast<int64_t>(c) * p.H + h;
  load_rows(&s.q[0][0], kLdK, p.q, t0, n, p.H, h, kK, 0, kK);
  load_rows(&s.k[0][0], kLdK, p.k, t0, n, p.H, h, kK, 0, kK);
  if (threadIdx.x < kC) {
    const int r = min(static_cast<int>(threadIdx.x), n - 1);
    s.gc[threadIdx.x] = p.gcum[(t0 + r) * p.H + h];
  }
  __syncthreads();
  {
    FragC acc[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::fill_fragment(acc[nt], 0.f);
    for (int ks = 0; ks < kK / 16; ++ks) {
      FragA a;
      wmma::load_matrix_sync(a, &s.q[16 * warp][16 * ks], kLdK);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        FragBT b;
        wmma::load_matrix_sync(b, &s.k[16 * nt][16 * ks], kLdK);
        wmma::mma_sync(acc[nt], a, b, acc[nt]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::store_matrix_sync(&s.P[16 * warp][16 * nt], acc[nt], kLdF, wmma::mem_row_major);
  }
  __syncthreads();   // every warp is done with q as it was loaded
  for (int i = threadIdx.x; i < kC * kC; i += kThreads) {
    const int r = i / kC, cc = i - r * kC;
    s.Pb[r][cc] = __float2bfloat16(r >= cc ? s.P[r][cc] * __expf(s.gc[r] - s.gc[cc]) : 0.f);
  }
  for (int i = threadIdx.x; i < kC * (kK / 2); i += kThreads) {
    const int r = i / (kK / 2), cc = (i - r * (kK / 2)) * 2;
    const float e = __expf(s.gc[r]);
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&s.q[r][cc]));
    *reinterpret_cast<__nv_bfloat162*>(&s.q[r][cc]) = __floats2bfloat162_rn(f.x * e, f.y * e);
  }
  __syncthreads();
  {
    const __nv_bfloat16* hsrc = p.hstate + ch * kK * p.V + v0;
    const __nv_bfloat16* vsrc = p.vnew + ch * kC * p.V + v0;
    FragC acc[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::fill_fragment(acc[nt], 0.f);
    for (int ks = 0; ks < kK / 16; ++ks) {
      FragA a;
      wmma::load_matrix_sync(a, &s.q[16 * warp][16 * ks], kLdK);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        FragB b;
        wmma::load_matrix_sync(b, hsrc + static_cast<int64_t>(16 * ks) * p.V + 16 * nt, p.V);
        wmma::mma_sync(acc[nt], a, b, acc[nt]);
      }
    }
    for (int ks = 0; ks < kC / 16; ++ks) {
      FragA a;
      wmma::load_matrix_sync(a, &s.Pb[16 * warp][16 * ks], kLdC);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        FragB b;
        wmma::load_matrix_sync(b, vsrc + static_cast<int64_t>(16 * ks) * p.V + 16 * nt, p.V);
        wmma::mma_sync(acc[nt], a, b, acc[nt]);
      }
    }
    // P rows of this warp were last read (as P) before the barrier above: reuse them as staging
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) wmma::store_matrix_sync(&s.P[16 * warp][16 * nt], acc[nt], kLdF, wmma::mem_row_major);
  }
  __syncwarp();
  for (int i = lane; i < 16 * (kVT / 2); i += 32) {
    const int r = 16 * warp + i / (kVT / 2), cc = (i % (kVT / 2)) * 2;
    if (r < n)
      *reinterpret_cast<__nv_bfloat162*>(p.o + ((t0 + r) * p.H + h) * p.V + v0 + cc) =
          __floats2bfloat162_rn(s.P[r][cc] * p.scale, s.P[r][cc + 1] * p.scale);
  }
}

}  // namespace

cudaError_t launch_gdn_chunk_fwd(const GdnChunkArgs& a, cudaStream_t stream) {
  if (a.K != kK || a.V % 64 != 0 || a.V < 64 || a.V > 256 || a.num_seqs < 1 || a.num_chunks < 0) return cudaErrorInvalidValue;
  if (a.num_chunks == 0) return cudaSuccess;
  ChunkParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.k = reinterpret_cast<const __nv_bfloat16*>(a.k);
  p.v = reinterpret_cast<const __nv_bfloat16*>(a.v);
  p.g = a.g;
  p.beta = reinterpret_cast<const __nv_bfloat16*>(a.beta);
  p.cu_seqlens = a.cu_seqlens;
  p.chunk_seq = a.chunk_seq;
  p.chunk_t0 = a.chunk_t0;
  p.seq_chunk0 = a.seq_chunk0;
  p.gcum = a.g_cumsum;
  p.a_out = a.a_out;
  p.w = reinterpret_cast<__nv_bfloat16*>(a.w);
  p.u = reinterpret_cast<__nv_bfloat16*>(a.u);
  p.vnew = reinterpret_cast<__nv_bfloat16*>(a.v_new);
  p.hstate = reinterpret_cast<__nv_bfloat16*>(a.h_chunks);
  p.h0 = a.initial_state;
  p.ht = a.final_state;
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o);
  p.H = a.H; p.V = a.V; p.NC = a.num_chunks;
  p.scale = a.scale;
  static SmemOptIn opt1, opt2, opt3;
  const int smem1 = static_cast<int>(sizeof(PrepSmem)) + kC * (a.V + 8) * 2;
  const int smem2 = static_cast<int>(sizeof(StateSmem));
  const int smem3 = static_cast<int>(sizeof(OutSmem));
  cudaError_t e = opt1.ensure(gdn_chunk_prepare, 128 * 1024);
  if (e != cudaSuccess) return e;
  e = opt2.ensure(gdn_chunk_state, smem2);
  if (e != cudaSuccess) return e;
  e = opt3.ensure(gdn_chunk_output, smem3);
  if (e != cudaSuccess) return e;
  if (smem1 > 128 * 1024) return cudaErrorInvalidValue;
  gdn_chunk_prepare<<<dim3(a.num_chunks, a.H), kThreads, smem1, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gdn_chunk_state<<<dim3(a.V / kVT, a.H, a.num_seqs), kThreads, smem2, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gdn_chunk_output<<<dim3(a.num_chunks, a.H, a.V / kVT), kThreads, smem3, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace tdb
