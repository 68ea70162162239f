// Decode GEMV for one to sixteen tokens:  out[M, N] = f(x)[M, K] * W[N, K]^T  (+ all-reduce) (+ residual).
//
// With so few tokens a linear layer is a pure weight stream: the tensor cores have nothing to amortise and the cost
// of a decode step is the HBM time of the weights plus whatever each launch adds around it.  This kernel therefore
// keeps the stream as plain as possible (every warp owns whole output columns, reads their weight rows with 16-byte
// loads that stay many deep in flight, and reduces inside the warp, so there is no split-K, no atomics and no
// second pass) and folds the neighbouring small kernels of a transformer layer into its prologue and epilogue:
//   prologue   f = RMSNorm(x) * g      (the sum of squares is taken while the activations are staged)
//              f = SiLU(gate) * up     (x is the fused gate | up projection)
//   epilogue   all-reduce of the result over the tensor-parallel ranks: every CTA publishes its columns in the
//              symmetric heap, exchanges one epoch flag per peer with the CTA of the same index there, and reads the
//              sum back with multimem.ld_reduce (or sums the peers' slots after a push when there is no multicast)
//              residual add, in place if wanted
// so a decoder layer is four GEMV launches plus attention.
//
// Reference behaviour being matched (not its code): the decode path of layers/nvidia/tp_attn.py:160-213 and
// tp_mlp.py:196-229 (rmsnorm -> linear -> ... -> linear -> all-reduce -> add) and the fused GEMM+AllReduce of
// kernels/nvidia/gemm_allreduce.py:124-315, specialised to M <= 8.
#include <cuda.h>

#include <cstdlib>

#include "tdb/gemv.h"
#include "tdb/launch.cuh"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kGemvThreads = 512;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kRedBytes = 8 * 1024;   // shared memory kept for the K-slice partial sums (32 slots of 8 x 8 floats)
constexpr int kMaxSmem = 200 * 1024;

struct GemvParams {
  int M, N, K;
  const __nv_bfloat16* x;
  int64_t ldx;
  const __nv_bfloat16* w;
  int64_t ldw;
  __nv_bfloat16* out;
  int64_t ld_out;
  const __nv_bfloat16* norm_w;
  float eps;
  int silu_mul;
  const __nv_bfloat16* residual;
  int64_t ld_res;
  int rows_per_cta;
  int all_reduce;
  int use_mc;
  __nv_bfloat16* partial;
  uint64_t partial_half;
  uint32_t* flags;
  int max_ctas;
  int m_cap;
  CtxDev* ctx;
  SymmInfo symm;
};

TDB_DEVICE void unpack8(const uint4& v, float (&f)[8]) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
TDB_DEVICE uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}

// One warp-wide tensor-core step: D[16 x 8] += A[16 x 16] * B[16 x 8], bf16 in, fp32 accumulate.
TDB_DEVICE void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Work layout.  A CTA owns `rows_per_cta` (a multiple of 8) output columns = weight rows, in groups of 8.  A warp
// takes one group and one slice of K; lane (g = lane / 4, t = lane % 4) streams row g of the group with 16-byte
// loads, 32 elements of K per step across the four t lanes.  The dot products run on the tensor cores: the eight
// loaded values of a lane are fed as the A fragments of two m16n8k16 steps (rows 8..15 of A are zero), the eight
// activations of the same K positions of token g as the B fragments.  A dot product does not care in which order K
// is walked, so the K positions are simply assigned to fragment slots in the order the 16-byte loads deliver them;
// the accumulator then holds [8 rows x 8 tokens] and no lane-wise reduction is needed.  What is left per lane and
// load is one shared-memory read and two mma instructions, so the warps spend their issue slots on keeping loads
// in flight (kJ per lane, double buffered).  Slices of K are summed through shared memory at the end.
constexpr int kJ = 8;

template <int MP>   // tokens rounded up to 1, 2, 4, 8 or 16 (two 8-token MMA tiles)
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvParams p) {
  extern __shared__ uint4 smem4[];
  __shared__ float s_part[kGemvWarps][MP];
  __shared__ float s_rstd[16];
  constexpr int NT = (MP + 7) / 8;          // 8-token tiles of the MMA's N dimension
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kv = p.K >> 3;                       // 16-byte vectors per row
  const int xs_stride = kv + 4;                  // in vectors: rows 64 bytes apart modulo 128 (bank-conflict free)
  uint4* xs = smem4;                             // staged activations f(x): [MP][xs_stride]
  float* red = reinterpret_cast<float*>(smem4 + MP * xs_stride);   // [slots][8 rows][8 NT tokens] partial accumulators
  const int r0 = blockIdx.x * p.rows_per_cta;
  const int r1 = min(p.N, r0 + p.rows_per_cta);
  const int groups = (r1 - r0 + 7) >> 3;         // groups this CTA really has (the last CTA may have fewer)
  const int groups_nom = p.rows_per_cta >> 3;    // the warp layout follows the nominal count, the same in every CTA
  const int slices = groups_nom >= kGemvWarps ? 1 : kGemvWarps / groups_nom;
  const int steps_total = (kv + 3) >> 2;         // steps of 4 vectors (32 elements of K)

  // this warp's first unit: (group, K slice)
  int grp = slices == 1 ? warp : warp % groups_nom;
  const int slice = slices == 1 ? 0 : warp / groups_nom;
  const bool active = grp < groups && slice < slices;
  const int st0 = (steps_total * slice) / slices, st1 = (steps_total * (slice + 1)) / slices;

  // The weights do not depend on the previous kernel: the first loads are issued before anything else, so that
  // their latency overlaps the predecessor's tail (programmatic dependent launch) and the staging of x.
  uint4 wa[kJ], wb[kJ];
  auto issue = [&](uint4 (&dst)[kJ], int group, int step) {
    const int row = min(r0 + group * 8 + g, p.N - 1);
    const bool row_ok = r0 + group * 8 + g < r1;
    const __nv_bfloat16* wr = p.w + static_cast<int64_t>(row) * p.ldw;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const int c = (step + j) * 4 + t;
      dst[j] = (row_ok && step + j < st1 && c < kv) ? ld_nc_v4(wr + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  if (active) issue(wa, grp, st0);
  pdl_wait();
  pdl_launch_dependents();
  // the call epoch is advanced by the last CTA of the previous call: read it only after the dependency wait
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int par = epoch & 1;

  // ---- prologue: stage f(x) in shared memory; a thread takes one 16-byte column slice of every token, so the loads
  // of all tokens are in flight together and the staging time does not grow with the token count
  float ss[MP];
#pragma unroll
  for (int m = 0; m < MP; ++m) ss[m] = 0.f;
  constexpr int MB = MP < 4 ? MP : 4;      // tokens whose loads are in flight together (register budget)
  for (int c = tid; c < kv; c += kGemvThreads) {
    float gn[8];
    if (p.norm_w != nullptr) unpack8(ld_nc_v4(p.norm_w + c * 8), gn);
#pragma unroll
    for (int m0 = 0; m0 < MP; m0 += MB) {
      uint4 v[MB], u[MB];
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        const int m = m0 + i;
        v[i] = (m < p.M) ? ld_v4(p.x + static_cast<int64_t>(m) * p.ldx + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        if (p.silu_mul)
          u[i] = (m < p.M) ? ld_v4(p.x + static_cast<int64_t>(m) * p.ldx + p.K + c * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        const int m = m0 + i;
        if (p.silu_mul) {
          float gg[8], h[8];
          unpack8(v[i], gg);
          unpack8(u[i], h);
#pragma unroll
          for (int j = 0; j < 8; ++j) gg[j] = gg[j] / (1.f + __expf(-gg[j])) * h[j];
          v[i] = pack8(gg);
        } else if (p.norm_w != nullptr) {
          float a[8];
          unpack8(v[i], a);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            ss[m] += a[j] * a[j];
            a[j] *= gn[j];
          }
          v[i] = pack8(a);
        }
        xs[m * xs_stride + c] = v[i];
      }
    }
  }
  if (p.norm_w != nullptr) {
#pragma unroll
    for (int m = 0; m < MP; ++m) {
      const float tt = warp_sum(ss[m]);
      if (lane == 0) s_part[warp][m] = tt;
    }
    __syncthreads();
    if (tid < MP) {
      float tt = 0.f;
      for (int wi = 0; wi < kGemvWarps; ++wi) tt += s_part[wi][tid];
      s_rstd[tid] = rsqrtf(tt / static_cast<float>(p.K) + p.eps);
    }
  } else if (tid < 16) {
    s_rstd[tid] = 1.f;
  }
  __syncthreads();

  // ---- main loop
  auto consume = [&](const uint4 (&src)[kJ], int step, float (&c)[NT][4]) {
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const int cv = (step + j) * 4 + t;
      const bool in_range = step + j < st1 && cv < kv;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + g;               // token whose activations this lane feeds as the B fragment
        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
        if (tok < MP && in_range) xv = xs[tok * xs_stride + cv];
        mma_bf16_16816(c[nt], src[j].x, 0u, src[j].y, 0u, xv.x, xv.y);
        mma_bf16_16816(c[nt], src[j].z, 0u, src[j].w, 0u, xv.z, xv.w);
      }
    }
  };
  if (active) {
    for (; grp < groups; grp += kGemvWarps) {
      float c[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
      int st = st0;
      while (st < st1) {
        // wa holds steps [st, st + kJ); fetch the next batch into wb before consuming wa, and vice versa
        if (st + kJ < st1) issue(wb, grp, st + kJ);
        consume(wa, st, c);
        st += kJ;
        if (st >= st1) break;
        if (st + kJ < st1) issue(wa, grp, st + kJ);
        consume(wb, st, c);
        st += kJ;
      }
      // accumulator: c[0], c[1] = (row g, tokens 2t, 2t + 1); rows 8..15 of the tile are the zero half
      const int slot = grp * slices + slice;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[(slot * 8 + g) * (8 * NT) + nt * 8 + 2 * t] = c[nt][0];
        red[(slot * 8 + g) * (8 * NT) + nt * 8 + 2 * t + 1] = c[nt][1];
      }
      const int nxt = grp + kGemvWarps;
      if (slices == 1 && nxt < groups) issue(wa, nxt, st0);
      if (slices != 1) break;
    }
  }
  __syncthreads();

  // ---- sum the K slices, scale, store
  __nv_bfloat16* pdst = nullptr;   // all-reduce: where this rank's partial result goes
  if (p.all_reduce)
    pdst = p.partial + par * p.partial_half + (p.use_mc ? 0ull : static_cast<uint64_t>(p.symm.rank) * p.m_cap * p.N);
  for (int i = tid; i < groups * 8 * p.M; i += kGemvWarps * 32) {
    const int m = i / (groups * 8), rr = i - m * (groups * 8);     // consecutive threads -> consecutive columns
    const int row = r0 + rr;
    if (row >= r1) continue;
    const int gi = rr >> 3, gr = rr & 7;
    float v = 0.f;
    for (int sl = 0; sl < slices; ++sl) v += red[((gi * slices + sl) * 8 + gr) * (8 * NT) + m];
    v *= s_rstd[m];
    if (p.all_reduce) {
      pdst[static_cast<int64_t>(m) * p.N + row] = __float2bfloat16(v);
    } else {
      if (p.residual != nullptr) v += __bfloat162float(p.residual[static_cast<int64_t>(m) * p.ld_res + row]);
      p.out[static_cast<int64_t>(m) * p.ld_out + row] = __float2bfloat16(v);
    }
  }

  // ---- epilogue: all-reduce of this CTA's columns [r0, r1) (multiples of 8) with the same CTA of every rank
  if (p.all_reduce && r0 < p.N) {
    const int W = p.symm.world, rank = p.symm.rank;
    const int nvec = (r1 - r0) >> 3;
    __syncthreads();
    if (!p.use_mc) {
      // push this rank's slot of the columns to every peer
      for (int v = tid; v < p.M * nvec; v += kGemvThreads) {
        const int m = v / nvec, col = r0 + (v - m * nvec) * 8;
        __nv_bfloat16* src = pdst + static_cast<int64_t>(m) * p.N + col;
        const uint4 u = ld_v4(src);
        for (int j = 1; j < W; ++j) st_v4(symm_at(p.symm, src, (rank + j) % W), u);
      }
      __syncthreads();
    }
    bool ok = true;
    if (tid < W) {
      fence_acq_rel_sys();
      st_release_sys(symm_at(p.symm, p.flags + static_cast<int64_t>(rank) * p.max_ctas + blockIdx.x, (rank + tid) % W), epoch);
      ok = wait_until(p.symm, p.flags + static_cast<int64_t>(tid) * p.max_ctas + blockIdx.x, epoch, kCmpGe, kKernelGemv, 1,
                      tid, blockIdx.x);
    }
    ok = __syncthreads_and(ok);
    if (ok) {
      for (int v = tid; v < p.M * nvec; v += kGemvThreads) {
        const int m = v / nvec, col = r0 + (v - m * nvec) * 8;
        float s[8];
        if (p.use_mc) {
          const __nv_bfloat16* src = p.partial + par * p.partial_half + static_cast<int64_t>(m) * p.N + col;
          unpack8(multimem_ld_reduce_bf16x8(mc_ptr(p.symm, src)), s);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) s[j] = 0.f;
          for (int r = 0; r < W; ++r) {
            const __nv_bfloat16* src =
                p.partial + par * p.partial_half + (static_cast<uint64_t>(r) * p.m_cap + m) * p.N + col;
            float tt[8];
            unpack8(ld_relaxed_sys_v4(src), tt);
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] += tt[j];
          }
        }
        if (p.residual != nullptr) {
          float e[8];
          unpack8(ld_v4(p.residual + static_cast<int64_t>(m) * p.ld_res + col), e);
#pragma unroll
          for (int j = 0; j < 8; ++j) s[j] += e[j];
        }
        st_v4(p.out + static_cast<int64_t>(m) * p.ld_out + col, pack8(s));
      }
    }
  }

  // last CTA out advances the call epoch
  if (p.ctx != nullptr) {
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      const uint32_t prev = atomicAdd(&p.ctx->done, 1u);
      if (prev == gridDim.x - 1) {
        p.ctx->done = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
      }
    }
  }
}

template <int M>
cudaError_t launch_t(const GemvParams& p, int grid, size_t smem, cudaStream_t stream) {
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return e;
    set = true;
  }
  // everything the kernel reads from its predecessor comes after pdl_wait()
  return launch_pdl(gemv_kernel<M>, dim3(grid), dim3(kGemvThreads), smem, stream, p);
}

}  // namespace

int gemv_max_k(int M) {
  const int mp = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  // mp rows of (2 K + 64) bytes next to the partial-sum slots
  return (((kMaxSmem - kRedBytes) / mp - 64) / 2) & ~7;
}

cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t stream) {
  if (a.M < 1 || a.M > 16 || a.K % 8 != 0 || a.K > gemv_max_k(a.M)) return cudaErrorInvalidValue;
  if (a.ldw % 8 != 0 || a.ldx % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x)) & 15u) return cudaErrorInvalidValue;
  if (a.norm_w != nullptr && a.silu_mul) return cudaErrorInvalidValue;
  GemvParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  p.ldx = a.ldx;
  p.w = reinterpret_cast<const __nv_bfloat16*>(a.w);
  p.ldw = a.ldw;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.ld_out = a.ld_out;
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(a.norm_w);
  p.eps = a.eps;
  p.silu_mul = a.silu_mul;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ld_res = a.ld_res;
  p.all_reduce = a.all_reduce;
  p.use_mc = (a.use_multimem && a.symm.mc_base != 0) ? 1 : 0;
  p.partial = reinterpret_cast<__nv_bfloat16*>(a.partial);
  p.m_cap = a.m_cap;
  p.partial_half = p.use_mc ? static_cast<uint64_t>(a.m_cap) * a.N : static_cast<uint64_t>(a.symm.world) * a.m_cap * a.N;
  p.flags = a.flags;
  p.max_ctas = a.max_ctas;
  p.ctx = a.ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &a.symm, sizeof(SymmInfo));
  const int num_ctas = a.num_ctas < 1 ? 1 : a.num_ctas;
  // groups of 8 columns per warp; in all-reduce mode this also gives every CTA whole 16-byte vectors
  const int rows = (((a.N + num_ctas - 1) / num_ctas) + 7) & ~7;
  if (a.all_reduce) {
    // the residual / output rows must allow vector access
    if (a.N % 8 != 0 || a.ld_out % 8 != 0 || (a.residual != nullptr && a.ld_res % 8 != 0)) return cudaErrorInvalidValue;
    if (a.ctx == nullptr || a.partial == nullptr || a.flags == nullptr || a.M > a.m_cap) return cudaErrorInvalidValue;
  }
  p.rows_per_cta = rows;
  const int grid = (a.N + rows - 1) / rows;
  if (a.all_reduce && grid > a.max_ctas) return cudaErrorInvalidValue;
  const int mp = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : a.M <= 8 ? 8 : 16;
  const int groups = rows / 8;
  const int slots = groups >= kGemvWarps ? groups : groups * (kGemvWarps / groups);
  const size_t smem = static_cast<size_t>(mp) * (a.K * 2 + 64) + static_cast<size_t>(slots) * 256 * ((mp + 7) / 8);
  if (smem > static_cast<size_t>(kMaxSmem)) return cudaErrorInvalidValue;
  switch (mp) {
    case 1: return launch_t<1>(p, grid, smem, stream);
    case 2: return launch_t<2>(p, grid, smem, stream);
    case 4: return launch_t<4>(p, grid, smem, stream);
    case 8: return launch_t<8>(p, grid, smem, stream);
    default: return launch_t<16>(p, grid, smem, stream);
  }
}

}  // namespace tdb
