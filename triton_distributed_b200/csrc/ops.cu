// Memory-bound single-GPU ops of the decoder layer: RMSNorm (optionally fused with
// the residual add), SiLU-gated multiply, residual add, fused QK-RMSNorm + RoPE +
// KV-cache write, embedding gather, arg-max sampling, |x| checksum.
//
// Reference behaviour being matched (not its code):
//   mega_triton_kernel/kernels/norm.py:32-189 (qk norm + rope + kv cache update), :193 (rms norm)
//   mega_triton_kernel/kernels/activation.py:31-78, elementwise.py:31-52
//   layers/nvidia/tp_attn.py:61-67,173 (flashinfer rmsnorm / rope calls these replace)
//   models/utils.py:86 (sample_token arg-max path)
// All kernels use 16-byte accesses and fp32 math; one pass over the data.
#include "tdb/launch.cuh"
#include "tdb/ops.h"
#include "tdb/ptx.cuh"

namespace tdb {

namespace {

TDB_DEVICE float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  const float r = red[0];
  __syncthreads();
  return r;
}

// out = rmsnorm(x (+ residual)) * w ; when residual != nullptr it is updated in place with x + residual.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, int H,
                               int64_t ldx, float eps) {
  __shared__ float red[32];
  extern __shared__ uint4 row_cache[];  // H/8 vectors
  pdl_wait();                 // x and the residual come from the previous kernels
  pdl_launch_dependents();    // a weight-streaming successor may start fetching its weights now
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * H) : nullptr;
  const int nv = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 u = xr[i];
    if (rr) {
      const uint4 r = rr[i];
      float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      float2 b0 = unpack_bf16x2(r.x), b1 = unpack_bf16x2(r.y), b2 = unpack_bf16x2(r.z), b3 = unpack_bf16x2(r.w);
      u.x = pack_bf16x2(a0.x + b0.x, a0.y + b0.y);
      u.y = pack_bf16x2(a1.x + b1.x, a1.y + b1.y);
      u.z = pack_bf16x2(a2.x + b2.x, a2.y + b2.y);
      u.w = pack_bf16x2(a3.x + b3.x, a3.y + b3.y);
      rr[i] = u;
    }
    row_cache[i] = u;
    float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / H + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + row * H);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const uint4 u = row_cache[i], g = wr[i];
    float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    uint4 o;
    o.x = pack_bf16x2(f0.x * inv * g0.x, f0.y * inv * g0.y);
    o.y = pack_bf16x2(f1.x * inv * g1.x, f1.y * inv * g1.y);
    o.z = pack_bf16x2(f2.x * inv * g2.x, f2.y * inv * g2.y);
    o.w = pack_bf16x2(f3.x * inv * g3.x, f3.y * inv * g3.y);
    orow[i] = o;
  }
}

TDB_DEVICE float silu(float x) { return x / (1.f + __expf(-x)); }

// out[t, i] = silu(in[t, i]) * in[t, I + i]
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t T,
                                int I, int64_t ld_in) {
  const int nv = I >> 3;
  const int64_t total = T * nv;
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = v / nv;
    const int i = static_cast<int>(v - t * nv);
    const uint4 g = *reinterpret_cast<const uint4*>(in + t * ld_in + i * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(in + t * ld_in + I + i * 8);
    float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    float2 u0 = unpack_bf16x2(u.x), u1 = unpack_bf16x2(u.y), u2 = unpack_bf16x2(u.z), u3 = unpack_bf16x2(u.w);
    uint4 o;
    o.x = pack_bf16x2(silu(g0.x) * u0.x, silu(g0.y) * u0.y);
    o.y = pack_bf16x2(silu(g1.x) * u1.x, silu(g1.y) * u1.y);
    o.z = pack_bf16x2(silu(g2.x) * u2.x, silu(g2.y) * u2.y);
    o.w = pack_bf16x2(silu(g3.x) * u3.x, silu(g3.y) * u3.y);
    *reinterpret_cast<uint4*>(out + t * I + i * 8) = o;
  }
}

__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, int64_t nvec) {
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 x = reinterpret_cast<const uint4*>(a)[v], y = reinterpret_cast<const uint4*>(b)[v];
    float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
    float2 b0 = unpack_bf16x2(y.x), b1 = unpack_bf16x2(y.y), b2 = unpack_bf16x2(y.z), b3 = unpack_bf16x2(y.w);
    uint4 o;
    o.x = pack_bf16x2(a0.x + b0.x, a0.y + b0.y);
    o.y = pack_bf16x2(a1.x + b1.x, a1.y + b1.y);
    o.z = pack_bf16x2(a2.x + b2.x, a2.y + b2.y);
    o.w = pack_bf16x2(a3.x + b3.x, a3.y + b3.y);
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

// One warp per (token, head) of the packed qkv row [Hq*D | Hkv*D | Hkv*D].
// q heads: optional RMSNorm over D (weight qw), RoPE, written to q_out [T, Hq, D].
// k heads: optional RMSNorm (kw), RoPE, written to k_cache[slot[t], h, :].
// v heads: copied to v_cache[slot[t], h, :].
// RoPE is the rotate-half form: (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin), x2 = x[D/2:].
__global__ void qk_norm_rope_kv_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
                                       const __nv_bfloat16* __restrict__ kw, const int64_t* __restrict__ positions,
                                       const int64_t* __restrict__ slots, __nv_bfloat16* __restrict__ q_out,
                                       __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int T,
                                       int Hq, int Hkv, int D, int64_t ld_qkv, float eps, float log2_theta,
                                       int64_t cache_slot_stride, int64_t cache_rows) {
  pdl_wait();                 // qkv comes from the previous kernel
  pdl_launch_dependents();
  const int warps_per_block = blockDim.x >> 5;
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  if (wid >= static_cast<int64_t>(T) * heads) return;
  const int t = static_cast<int>(wid / heads);
  const int h = static_cast<int>(wid - static_cast<int64_t>(t) * heads);
  const __nv_bfloat16* src = qkv + t * ld_qkv + static_cast<int64_t>(h) * D;
  const int half = D >> 1;
  const int64_t slot = slots ? slots[t] : t;
  // rows outside the cache (negative = "do not store", or beyond its last row) are never written
  const bool slot_ok = slot >= 0 && slot < cache_rows;
  if (h >= Hq + Hkv) {  // v: plain copy
    if (!slot_ok) return;
    __nv_bfloat16* dst = v_cache + slot * cache_slot_stride + static_cast<int64_t>(h - Hq - Hkv) * D;
    for (int i = lane; i < (D >> 3); i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }
  const bool is_q = h < Hq;
  const __nv_bfloat16* wgt = is_q ? qw : kw;
  // each lane owns pairs (2*j, 2*j+1) for j = lane, lane+32, ... in both halves
  float ss = 0.f;
  for (int j = lane; j < (half >> 1); j += 32) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 2 * j));
    const float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + half + 2 * j));
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
  }
  ss = warp_sum(ss);
  const float inv = wgt ? rsqrtf(ss / D + eps) : 1.f;
  const float pos = static_cast<float>(positions[t]);
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (static_cast<int64_t>(t) * Hq + h) * D;
  } else {
    if (!slot_ok) return;
    dst = k_cache + slot * cache_slot_stride + static_cast<int64_t>(h - Hq) * D;
  }
  for (int j = lane; j < (half >> 1); j += 32) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 2 * j));
    float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + half + 2 * j));
    if (wgt) {
      const float2 wa = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(wgt + 2 * j));
      const float2 wb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(wgt + half + 2 * j));
      // round to bf16 after the norm, as a separate RMSNorm kernel would
      a.x = __bfloat162float(__float2bfloat16(a.x * inv * wa.x));
      a.y = __bfloat162float(__float2bfloat16(a.y * inv * wa.y));
      b.x = __bfloat162float(__float2bfloat16(b.x * inv * wb.x));
      b.y = __bfloat162float(__float2bfloat16(b.y * inv * wb.y));
    }
    const float f0 = exp2f(-(2.f * (2 * j)) / D * log2_theta);
    const float f1 = exp2f(-(2.f * (2 * j + 1)) / D * log2_theta);
    float s0, c0, s1, c1;
    sincosf(pos * f0, &s0, &c0);
    sincosf(pos * f1, &s1, &c1);
    *reinterpret_cast<uint32_t*>(dst + 2 * j) = pack_bf16x2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
    *reinterpret_cast<uint32_t*>(dst + half + 2 * j) = pack_bf16x2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
  }
}

__global__ void embedding_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int H, int64_t vocab) {
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + id * H);
  uint4* dst = reinterpret_cast<uint4*>(out + t * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
}

// arg-max over the last dimension of fp32 logits [B, V]; ties go to the lowest index.
__global__ void argmax_kernel(const float* __restrict__ logits, int64_t* __restrict__ out, int64_t V) {
  __shared__ float sval[32];
  __shared__ int64_t sidx[32];
  const float* row = logits + blockIdx.x * V;
  float best = -INFINITY;
  int64_t bi = 0;
  for (int64_t i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) {
      best = v;
      bi = i;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sval[w] = best;
    sidx[w] = bi;
  }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = l < nw ? sval[l] : -INFINITY;
    bi = l < nw ? sidx[l] : 0;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (l == 0) out[blockIdx.x] = bi;
  }
}

// out[0] += sum |x| (fp32 atomics; callers zero out first)
__global__ void abs_sum_kernel(const __nv_bfloat16* __restrict__ x, int64_t n, float* out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    s += fabsf(__bfloat162float(x[i]));
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

int grid_for(int64_t work, int threads, int cap) {
  int64_t g = (work + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

}  // namespace

cudaError_t launch_rmsnorm(const void* x, void* residual, const void* w, void* out, int64_t T, int H, int64_t ldx,
                           float eps, cudaStream_t s) {
  if (H % 8 != 0 || ldx % 8 != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  const int threads = H >= 4096 ? 512 : 256;
  const size_t smem = static_cast<size_t>(H) * 2;
  if (smem > 48 * 1024) {
    static bool set = false;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      set = true;
    }
  }
  return launch_pdl(rmsnorm_kernel, dim3(static_cast<unsigned>(T)), dim3(threads), smem, s,
                    reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(residual),
                    reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(out), H, ldx, eps);
}

cudaError_t launch_silu_mul(const void* in, void* out, int64_t T, int I, int64_t ld_in, cudaStream_t s) {
  if (I % 8 != 0 || ld_in % 8 != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  return launch_pdl(silu_mul_kernel, dim3(grid_for(T * (I / 8), 256, 148 * 8)), dim3(256), 0, s,
                    reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), T, I, ld_in);
}

cudaError_t launch_add(const void* a, const void* b, void* out, int64_t n, cudaStream_t s) {
  if (n % 8 != 0) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  add_kernel<<<grid_for(n / 8, 256, 148 * 8), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(a),
                                                           reinterpret_cast<const __nv_bfloat16*>(b),
                                                           reinterpret_cast<__nv_bfloat16*>(out), n / 8);
  return cudaGetLastError();
}

cudaError_t launch_qk_norm_rope_kv(const void* qkv, const void* qw, const void* kw, const int64_t* positions,
                                   const int64_t* slots, void* q_out, void* k_cache, void* v_cache, int T, int Hq,
                                   int Hkv, int D, int64_t ld_qkv, float eps, float rope_theta,
                                   int64_t cache_slot_stride, int64_t cache_rows, cudaStream_t s) {
  if (D % 8 != 0 || (D / 2) % 2 != 0 || ld_qkv % 8 != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  const int64_t warps = static_cast<int64_t>(T) * (Hq + 2 * Hkv);
  const int wpb = 8;
  return launch_pdl(qk_norm_rope_kv_kernel, dim3(static_cast<unsigned>((warps + wpb - 1) / wpb)), dim3(wpb * 32), 0, s,
                    reinterpret_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const __nv_bfloat16*>(qw),
                    reinterpret_cast<const __nv_bfloat16*>(kw), positions, slots, reinterpret_cast<__nv_bfloat16*>(q_out),
                    reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache), T, Hq, Hkv, D,
                    ld_qkv, eps, log2f(rope_theta), cache_slot_stride, cache_rows);
}

cudaError_t launch_embedding(const int64_t* ids, const void* table, void* out, int64_t T, int H, int64_t vocab,
                             cudaStream_t s) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  embedding_kernel<<<static_cast<unsigned>(T), 128, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(table),
                                                            reinterpret_cast<__nv_bfloat16*>(out), H, vocab);
  return cudaGetLastError();
}

cudaError_t launch_argmax(const float* logits, int64_t* out, int64_t B, int64_t V, cudaStream_t s) {
  if (B == 0) return cudaSuccess;
  argmax_kernel<<<static_cast<unsigned>(B), 1024, 0, s>>>(logits, out, V);
  return cudaGetLastError();
}

cudaError_t launch_abs_sum(const void* x, int64_t n, float* out, cudaStream_t s) {
  abs_sum_kernel<<<grid_for(n, 256 * 8, 148 * 4), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), n, out);
  return cudaGetLastError();
}

}  // namespace tdb
