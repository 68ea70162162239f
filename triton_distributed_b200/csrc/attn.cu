#include <atomic>
// Attention kernels over a paged KV cache (bf16, GQA, head dim 64 or 128):
//
//   flash_fwd_kernel         var-len causal prefill / context-parallel attention: one CTA = 64 query rows of one
//                            head (4 warps x 16 rows), KV streamed in 64-token blocks through double-buffered
//                            shared memory (cp.async), online softmax, optional LSE output.
//   decode_splitkv_kernel    one query token per sequence: the G = Hq/Hkv query heads of a KV head are packed into
//                            the 16-row MMA tile, the KV range is split over CTAs (split-KV) and over the 4 warps of
//                            a CTA; partial (out, LSE) go to a workspace.
//   decode_combine_kernel    merges the split partials by LSE; optionally keeps the LSE (for the cross-rank merge).
//   dist_combine_kernel      distributed flash-decode tail: merges the local splits, pushes the rank's (out, LSE)
//                            to every peer as low-latency packets with in-band epoch flags, waits for all peers'
//                            packets and merges the W partials - one launch, no separate all-gather.
//
// Math runs on mma.sync.m16n8k16 (bf16 in, fp32 accumulate): decode attention is bound by the KV stream from HBM,
// and the 16-row tile matches the GQA group; the tcgen05 path is reserved for the GEMMs.
//
// Reference behaviour being matched (not its code):
//   python/triton_dist/kernels/nvidia/flash_decode.py:130-239 (split-KV), :308-482 (combines), :587-760 (fused)
//   python/triton_dist/layers/nvidia/sp_flash_decode_layer.py:83-185 (partials -> LL all-gather -> LSE merge)
//   mega_triton_kernel/kernels/flash_attn.py:33-372 and kernels/nvidia/sp_ag_attention_intra_node.py:256-425 (prefill)
#include "tdb/launch.cuh"
#include "tdb/attn.h"
#include "tdb/attn_device.cuh"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

using namespace attn;

// ---------------------------------------------------------------------------
// Prefill / context-parallel forward.  q [Tq_total, Hq, D] packed over sequences (cu_seqlens_q); KV from a paged
// cache.  Query row i of sequence b sits at absolute position q_pos0[b] + i (for causal masking against the
// cache); kv_lens[b] tokens of KV are visible at most.
// ---------------------------------------------------------------------------
struct PrefillParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  float* lse;                  // [Hq, Tq_total] or nullptr
  const int32_t* cu_seqlens_q; // [B+1]
  const int32_t* q_pos0;       // [B] absolute position of the first query row (nullptr: kv_len - q_len)
  const int32_t* kv_lens;      // [B]
  PagedKV kv;
  int Hq;
  int group;                   // Hq / Hkv
  int causal;
  float scale, softcap;
  int64_t total_q;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads) flash_fwd_kernel(const PrefillParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  using T = Tiles<D>;
  const int b = blockIdx.z, head = blockIdx.y;
  const int q_begin = p.cu_seqlens_q[b], q_len = p.cu_seqlens_q[b + 1] - q_begin;
  const int row0 = blockIdx.x * 64;
  if (row0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int pos0 = p.q_pos0 ? p.q_pos0[b] : (kv_len - q_len);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int hkv = head / p.group;
  const int r_lo = row0 + warp * 16 + g, r_hi = r_lo + 8;
  WarpTile<D> w;
  w.init();
  const __nv_bfloat16* qb = p.q + (static_cast<int64_t>(q_begin) * p.Hq + head) * D;
  w.load_q(r_lo < q_len ? qb + static_cast<int64_t>(r_lo) * p.Hq * D : nullptr,
           r_hi < q_len ? qb + static_cast<int64_t>(r_hi) * p.Hq * D : nullptr);
  // visible KV range of this CTA (causal: up to the last row's position)
  const int last_row = min(q_len, row0 + 64) - 1;
  const int kv_end = p.causal ? min(kv_len, pos0 + last_row + 1) : kv_len;
  const int lim_lo = p.causal ? min(kv_len, pos0 + r_lo + 1) : kv_len;
  const int lim_hi = p.causal ? min(kv_len, pos0 + r_hi + 1) : kv_len;
  // warp-uniform bound of the visible tokens (the branch around step() must not diverge inside a warp)
  const int warp_lim = p.causal ? min(kv_len, pos0 + row0 + warp * 16 + 16) : kv_len;
  const int nblk = (kv_end + kBlockN - 1) / kBlockN;
  if (nblk > 0) {
    load_kv_block<D>(p.kv, b, hkv, 0, kv_end, smem, smem + T::kTileBytes);
    cp_async_commit();
  }
  for (int i = 0; i < nblk; ++i) {
    uint8_t* sK = smem + (i & 1) * 2 * T::kTileBytes;
    uint8_t* sV = sK + T::kTileBytes;
    if (i + 1 < nblk) {
      uint8_t* nK = smem + ((i + 1) & 1) * 2 * T::kTileBytes;
      load_kv_block<D>(p.kv, b, hkv, (i + 1) * kBlockN, kv_end, nK, nK + T::kTileBytes);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // skip blocks that are fully masked for this warp's rows
    if (i * kBlockN < warp_lim) w.template step<8>(sK, sV, i * kBlockN, 0, lim_lo, lim_hi, p.scale, p.softcap);
    __syncthreads();
  }
  float inv[2], lse[2];
  w.finish(inv, lse);
  const int c = 2 * (lane & 3);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r ? r_hi : r_lo;
    if (row >= q_len) continue;
    __nv_bfloat16* orow = p.out + ((static_cast<int64_t>(q_begin) + row) * p.Hq + head) * D;
#pragma unroll
    for (int jd = 0; jd < D / 8; ++jd)
      *reinterpret_cast<uint32_t*>(orow + 8 * jd + c) = pack_bf16x2(w.o[jd][2 * r] * inv[r], w.o[jd][2 * r + 1] * inv[r]);
    if (p.lse && (lane & 3) == 0) p.lse[static_cast<int64_t>(head) * p.total_q + q_begin + row] = lse[r];
  }
}

// ---------------------------------------------------------------------------
// Decode, split-KV.  q [B, Hq, D].  grid = (splits, Hkv * head_chunks, B).  Partials: out [B, Hq, splits, D] fp32,
// lse [B, Hq, splits].
// ---------------------------------------------------------------------------
// The last CTA to arrive for a (sequence, KV head, head chunk) merges the splits.  Returns true for that CTA only;
// the counter is left at zero for the next call.
__device__ bool splits_arrive_last(const DecodeParams& p) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ctr = p.fuse_counters + blockIdx.z * gridDim.y + blockIdx.y;
    const uint32_t prev = atomicAdd(ctr, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *ctr = 0;   // every arrival of this call has been counted: leave the counter clean for the next one
  }
  __syncthreads();
  if (!s_last) return false;
  __threadfence();
  return true;
}

// Merge of the split partials of one head chunk by its last CTA: the partials come from other CTAs, so they are read
// at L2.  First the LSEs of all heads of the chunk go to shared memory and become weights, then every thread sums four
// output dims of one head over the splits with several independent 16-byte loads in flight and hands the normalised
// float4 to emit(head in chunk, b * Hq + head, float4 index, values, LSE of the head over all splits).
template <int D, typename Emit>
__device__ void merge_chunk(const DecodeParams& p, uint8_t* smem, Emit emit) {
  const int b = blockIdx.z;
  const int hkv = blockIdx.y / p.head_chunks, hc = blockIdx.y - hkv * p.head_chunks;
  const int h_begin = hkv * p.group + hc * 16;
  const int nheads = min(p.group - hc * 16, 16);
  float* s_w = reinterpret_cast<float*>(smem);          // [nheads][splits] weights
  float* s_inv = s_w + 16 * p.splits;                   // [nheads] 1 / total
  float* s_lse = s_inv + 16;                            // [nheads] LSE over all splits
  for (int i = threadIdx.x; i < nheads * p.splits; i += kAttnThreads) {
    const int h = i / p.splits, sp = i - h * p.splits;
    s_w[i] = __ldcg(p.part_lse + (static_cast<int64_t>(b) * p.Hq + h_begin + h) * p.splits + sp);
  }
  __syncthreads();
  if (threadIdx.x < nheads) {
    float* w = s_w + threadIdx.x * p.splits;
    float mx = -INFINITY;
    for (int i = 0; i < p.splits; ++i) mx = fmaxf(mx, w[i]);
    float tot = 0.f;
    for (int i = 0; i < p.splits; ++i) {
      const float e = (mx == -INFINITY) ? 0.f : __expf(w[i] - mx);
      w[i] = e;
      tot += e;
    }
    s_inv[threadIdx.x] = tot > 0.f ? 1.f / tot : 0.f;
    s_lse[threadIdx.x] = tot > 0.f ? mx + __logf(tot) : -INFINITY;
  }
  __syncthreads();
  constexpr int kVecPerHead = D / 4;                     // float4 per head row
  constexpr int kHeadsPerPass = kAttnThreads / kVecPerHead;
  const int dv = threadIdx.x % kVecPerHead, sub = threadIdx.x / kVecPerHead;
  for (int h = sub; h < nheads; h += kHeadsPerPass) {
    const int64_t bh = static_cast<int64_t>(b) * p.Hq + h_begin + h;
    const float4* po = reinterpret_cast<const float4*>(p.part_out + bh * p.splits * D) + dv;
    const float* w = s_w + h * p.splits;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int i = 0;
    for (; i + 8 <= p.splits; i += 8) {
      float4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __ldcg(po + static_cast<int64_t>(i + j) * kVecPerHead);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc.x += w[i + j] * v[j].x; acc.y += w[i + j] * v[j].y;
        acc.z += w[i + j] * v[j].z; acc.w += w[i + j] * v[j].w;
      }
    }
    for (; i < p.splits; ++i) {
      const float4 v = __ldcg(po + static_cast<int64_t>(i) * kVecPerHead);
      acc.x += w[i] * v.x; acc.y += w[i] * v.y; acc.z += w[i] * v.z; acc.w += w[i] * v.w;
    }
    const float inv = s_inv[h];
    emit(h, bh, dv, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv), s_lse[h]);
  }
}

template <int D, int S>
__global__ void __launch_bounds__(kAttnThreads) decode_splitkv_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();   // q and the cache rows of the new token come from the previous kernel
  auto sync = [] { __syncthreads(); };
  decode_splitkv_body<D, decltype(sync), S>(p, blockIdx.x, blockIdx.y, blockIdx.z, smem, sync);
  if (p.fuse_counters == nullptr) return;
  // ---- fused combine
  pdl_launch_dependents();
  if (!splits_arrive_last(p)) return;
  merge_chunk<D>(p, smem, [&](int, int64_t bh, int dv, float4 o, float) {
    uint2 r;
    r.x = pack_bf16x2(o.x, o.y);
    r.y = pack_bf16x2(o.z, o.w);
    *reinterpret_cast<uint2*>(p.fuse_out + bh * D + dv * 4) = r;
  });
}

// ---------------------------------------------------------------------------
// Distributed flash-decode in ONE launch: split-KV over the local KV shard; the last CTA of every head chunk merges the
// local splits, pushes (out[D], LSE) of its heads as packets {value, epoch} (8 bytes each, written two at a time) into
// slot [rank] of every rank's staging, waits until all W slots of the local staging carry this call's epoch for its
// heads, merges them by LSE and writes the bf16 output.  A CTA only ever waits for REMOTE data, whose producers do not
// depend on this rank, but a waiting CTA keeps its SM: the host uses this form only while the head chunks
// (batch x KV heads x chunks) fit the SMs, so that waiting CTAs can never keep this rank's own split CTAs from running.
// staging: heap, [2][W][B*Hq][D+1] packets; buffer parity = epoch & 1; the last CTA out advances the epoch.
// The reference runs the same tail as separate kernels (python/triton_dist/kernels/nvidia/flash_decode.py:587-760).
// ---------------------------------------------------------------------------
struct DistTail {
  uint64_t* staging;
  int64_t staging_half;   // packets per buffer
  int BH;
  CtxDev* ctx;
  SymmInfo symm;
};

__device__ __forceinline__ void st_packet2(uint64_t* dst, uint64_t a, uint64_t b) {
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_packet2(const uint64_t* src, uint64_t& a, uint64_t& b) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(src) : "memory");
}
// Wait for two adjacent packets of this call; false after the time limit (status recorded).
__device__ bool wait_packet2(const DistTail& t, const uint64_t* src, uint32_t epoch, uint64_t t0, int slot, int index,
                             float& v0, float& v1) {
  uint64_t a, b;
  uint32_t spins = 0;
  while (true) {
    ld_packet2(src, a, b);
    if (static_cast<uint32_t>(a >> 32) == epoch && static_cast<uint32_t>(b >> 32) == epoch) break;
    if ((++spins & 255u) == 0u && (abort_requested(t.symm) || globaltimer_ns() - t0 > t.symm.timeout_ns)) {
      report(t.symm, kTimeoutFlag, kKernelFlashDecode, 2, slot, index, (int)epoch, (int)(a >> 32));
      return false;
    }
  }
  v0 = __uint_as_float(static_cast<uint32_t>(a));
  v1 = __uint_as_float(static_cast<uint32_t>(b));
  return true;
}
__device__ bool wait_packet1(const DistTail& t, const uint64_t* src, uint32_t epoch, uint64_t t0, int slot, int index,
                             float& v) {
  uint64_t a;
  uint32_t spins = 0;
  while (true) {
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(a) : "l"(src) : "memory");
    if (static_cast<uint32_t>(a >> 32) == epoch) break;
    if ((++spins & 255u) == 0u && (abort_requested(t.symm) || globaltimer_ns() - t0 > t.symm.timeout_ns)) {
      report(t.symm, kTimeoutFlag, kKernelFlashDecode, 3, slot, index, (int)epoch, (int)(a >> 32));
      return false;
    }
  }
  v = __uint_as_float(static_cast<uint32_t>(a));
  return true;
}

template <int D, int S>
__global__ void __launch_bounds__(kAttnThreads) decode_splitkv_dist_kernel(const DecodeParams p, const DistTail t) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();
  auto sync = [] { __syncthreads(); };
  decode_splitkv_body<D, decltype(sync), S>(p, blockIdx.x, blockIdx.y, blockIdx.z, smem, sync);
  pdl_launch_dependents();
  if (splits_arrive_last(p)) {
    // The epoch cannot advance before this CTA has counted itself out below.
    const uint32_t epoch = ld_volatile(&t.ctx->epoch);
    const int W = t.symm.world, rank = t.symm.rank;
    uint64_t* st = t.staging + (epoch & 1) * t.staging_half;
    // A row of D + 1 packets starts on an 8-byte boundary only (D + 1 is odd), so whether its packet pairs can be
    // written with 16-byte stores depends on the row: decided from the address, which symm_at does not change mod 16.
    const int64_t slot_stride = static_cast<int64_t>(t.BH) * (D + 1);
    const uint64_t tag = static_cast<uint64_t>(epoch) << 32;
    merge_chunk<D>(p, smem, [&](int, int64_t bh, int dv, float4 o, float lse) {
      uint64_t* mine = st + rank * slot_stride + bh * (D + 1);
      const bool even = (reinterpret_cast<uint64_t>(mine) & 15u) == 0;
      const uint64_t p0 = tag | __float_as_uint(o.x), p1 = tag | __float_as_uint(o.y);
      const uint64_t p2 = tag | __float_as_uint(o.z), p3 = tag | __float_as_uint(o.w);
      for (int j = 0; j < W; ++j) {
        uint64_t* dst = symm_at(t.symm, mine, (rank + j) % W) + dv * 4;
        if (even) {
          st_packet2(dst, p0, p1);
          st_packet2(dst + 2, p2, p3);
        } else {
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(p0) : "memory");
          st_packet2(dst + 1, p1, p2);
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 3), "l"(p3) : "memory");
        }
        if (dv == 0) {
          const uint64_t pl = tag | __float_as_uint(lse);
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + D), "l"(pl) : "memory");
        }
      }
    });
    // ---- receive: every thread owns four dims of one head per pass, as in the merge
    constexpr int kVecPerHead = D / 4;
    constexpr int kHeadsPerPass = kAttnThreads / kVecPerHead;
    const int b = blockIdx.z;
    const int hkv = blockIdx.y / p.head_chunks, hc = blockIdx.y - hkv * p.head_chunks;
    const int h_begin = hkv * p.group + hc * 16;
    const int nheads = min(p.group - hc * 16, 16);
    const int dv = threadIdx.x % kVecPerHead, sub = threadIdx.x / kVecPerHead;
    const uint64_t t0 = globaltimer_ns();
    for (int h = sub; h < nheads; h += kHeadsPerPass) {
      const int64_t bh = static_cast<int64_t>(b) * p.Hq + h_begin + h;
      float lse_s[kMaxRanks];
      float mx = -INFINITY;
      bool ok = true;
      for (int s = 0; s < W && ok; ++s) {
        ok = wait_packet1(t, st + s * slot_stride + bh * (D + 1) + D, epoch, t0, s, static_cast<int>(bh), lse_s[s]);
        if (ok) mx = fmaxf(mx, lse_s[s]);
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float tot = 0.f;
      for (int s = 0; s < W && ok; ++s) {
        const uint64_t* row = st + s * slot_stride + bh * (D + 1);
        const uint64_t* src = row + dv * 4;
        float v0, v1, v2, v3;
        if ((reinterpret_cast<uint64_t>(row) & 15u) == 0) {
          ok = wait_packet2(t, src, epoch, t0, s, static_cast<int>(bh), v0, v1) &&
               wait_packet2(t, src + 2, epoch, t0, s, static_cast<int>(bh), v2, v3);
        } else {
          ok = wait_packet1(t, src, epoch, t0, s, static_cast<int>(bh), v0) &&
               wait_packet2(t, src + 1, epoch, t0, s, static_cast<int>(bh), v1, v2) &&
               wait_packet1(t, src + 3, epoch, t0, s, static_cast<int>(bh), v3);
        }
        if (!ok) break;
        const float wgt = (mx == -INFINITY) ? 0.f : __expf(lse_s[s] - mx);
        tot += wgt;
        acc.x += wgt * v0; acc.y += wgt * v1; acc.z += wgt * v2; acc.w += wgt * v3;
      }
      if (ok) {
        const float inv = tot > 0.f ? 1.f / tot : 0.f;
        uint2 r;
        r.x = pack_bf16x2(acc.x * inv, acc.y * inv);
        r.y = pack_bf16x2(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(p.fuse_out + bh * D + dv * 4) = r;
      }
    }
  }
  // every CTA counts itself out; the last one advances the call epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
    const uint32_t prev = atomicAdd(&t.ctx->done, 1u);
    if (prev == total - 1) {
      const uint32_t epoch = ld_volatile(&t.ctx->epoch);
      t.ctx->done = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&t.ctx->epoch) = epoch + 1;
    }
  }
}

__global__ void decode_combine_kernel(const float* part_out, const float* part_lse, __nv_bfloat16* out, float* out_lse,
                                      float* out_f32, int splits, int D) {
  const int64_t bh = blockIdx.x;
  const int d = threadIdx.x;
  // a successor launched programmatically (the output projection's GEMV) may begin fetching its weights now
  pdl_launch_dependents();
  float v;
  const float lse = merge_partials(part_out + bh * splits * D, part_lse + bh * splits, splits, D, d, &v);
  if (out) out[bh * D + d] = __float2bfloat16(v);
  if (out_f32) out_f32[bh * (D + 1) + d] = v;
  if (d == 0) {
    if (out_lse) out_lse[bh] = lse;
    if (out_f32) out_f32[bh * (D + 1) + D] = lse;
  }
}

// ---------------------------------------------------------------------------
// Distributed flash-decode tail (one launch): CTA = one (b, head).
//   1. merge the local split partials -> (out[D], lse)
//   2. push them as packets {value, epoch} (8 bytes, written atomically) into slot [rank] of every peer's staging
//   3. wait until all W slots of the local staging carry this call's epoch, merge them by LSE, write bf16 out.
// staging: heap, [2][W][B*Hq][D+1] packets of 8 bytes; buffer parity = epoch & 1.
// ---------------------------------------------------------------------------
struct DistCombineParams {
  const float* part_out;
  const float* part_lse;
  __nv_bfloat16* out;
  uint64_t* staging;
  int64_t staging_half;   // packets per buffer
  int splits, D, BH;
  CtxDev* ctx;
  SymmInfo symm;
};

__global__ void dist_combine_kernel(const DistCombineParams p) {
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  const int W = p.symm.world, rank = p.symm.rank;
  const int64_t bh = blockIdx.x;
  const int d = threadIdx.x;  // 0..D (thread D carries the LSE)
  __shared__ float sh_lse[kMaxRanks];
  __shared__ int sh_fail;
  if (d == 0) sh_fail = 0;
  float v = 0.f, lse = -INFINITY;
  if (d < p.D) {
    lse = merge_partials(p.part_out + bh * p.splits * p.D, p.part_lse + bh * p.splits, p.splits, p.D, d, &v);
  } else {
    float dummy;
    lse = merge_partials(p.part_out + bh * p.splits * p.D, p.part_lse + bh * p.splits, p.splits, p.D, 0, &dummy);
    v = lse;
  }
  uint64_t* st = p.staging + (epoch & 1) * p.staging_half;
  const int64_t slot_stride = static_cast<int64_t>(p.BH) * (p.D + 1);
  const uint64_t pkt = (static_cast<uint64_t>(epoch) << 32) | __float_as_uint(v);
  for (int j = 0; j < W; ++j) {
    const int peer = (rank + j) % W;
    uint64_t* dst = symm_at(p.symm, st + rank * slot_stride + bh * (p.D + 1) + d, peer);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(pkt) : "memory");
  }
  __syncthreads();
  // receive
  float vals[kMaxRanks];
  const uint64_t t0 = globaltimer_ns();
  bool ok = true;
  for (int s = 0; s < W; ++s) {
    const uint64_t* src = st + s * slot_stride + bh * (p.D + 1) + d;
    uint64_t got;
    uint32_t spins = 0;
    while (true) {
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
      if (static_cast<uint32_t>(got >> 32) == epoch) break;
      if ((++spins & 255u) == 0u && (abort_requested(p.symm) || globaltimer_ns() - t0 > p.symm.timeout_ns)) {
        report(p.symm, kTimeoutFlag, kKernelFlashDecode, 1, s, static_cast<int>(bh), (int)epoch, (int)(got >> 32));
        ok = false;
        break;
      }
    }
    if (!ok) break;
    vals[s] = __uint_as_float(static_cast<uint32_t>(got));
    if (d == p.D) sh_lse[s] = vals[s];
  }
  if (!ok) sh_fail = 1;
  __syncthreads();
  if (sh_fail == 0 && d < p.D) {
    float mx = -INFINITY;
    for (int s = 0; s < W; ++s) mx = fmaxf(mx, sh_lse[s]);
    float tot = 0.f, acc = 0.f;
    for (int s = 0; s < W; ++s) {
      const float wgt = (mx == -INFINITY) ? 0.f : __expf(sh_lse[s] - mx);
      tot += wgt;
      acc += wgt * vals[s];
    }
    p.out[bh * p.D + d] = __float2bfloat16(tot > 0.f ? acc / tot : 0.f);
  }
  // last CTA out advances the epoch
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

template <typename K>
cudaError_t ensure_smem(K kernel, int bytes, SmemOptIn* st) {
  return st->ensure(kernel, bytes);
}

PagedKV make_kv(const AttnKV& kv) {
  PagedKV r;
  r.k = reinterpret_cast<const __nv_bfloat16*>(kv.k_cache);
  r.v = reinterpret_cast<const __nv_bfloat16*>(kv.v_cache);
  r.block_table = kv.block_table;
  r.max_pages = kv.max_pages;
  r.page_size = kv.page_size;
  r.Hkv = kv.num_kv_heads;
  return r;
}

}  // namespace

cudaError_t launch_flash_fwd(const FlashFwdArgs& a, cudaStream_t stream) {
  if (a.head_dim != 64 && a.head_dim != 128) return cudaErrorInvalidValue;
  if (a.num_q_heads % a.kv.num_kv_heads != 0) return cudaErrorInvalidValue;
  PrefillParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.lse = a.lse;
  p.cu_seqlens_q = a.cu_seqlens_q;
  p.q_pos0 = a.q_pos0;
  p.kv_lens = a.kv_lens;
  p.kv = make_kv(a.kv);
  p.Hq = a.num_q_heads;
  p.group = a.num_q_heads / a.kv.num_kv_heads;
  p.causal = a.causal;
  p.scale = a.scale;
  p.softcap = a.softcap;
  p.total_q = a.total_q;
  if (a.batch == 0 || a.max_q_len == 0) return cudaSuccess;
  dim3 grid((a.max_q_len + 63) / 64, a.num_q_heads, a.batch);
  if (a.head_dim == 128) {
    static SmemOptIn set;
    cudaError_t e = ensure_smem(flash_fwd_kernel<128>, Tiles<128>::kSmem, &set);
    if (e != cudaSuccess) return e;
    flash_fwd_kernel<128><<<grid, kAttnThreads, Tiles<128>::kSmem, stream>>>(p);
  } else {
    static SmemOptIn set;
    cudaError_t e = ensure_smem(flash_fwd_kernel<64>, Tiles<64>::kSmem, &set);
    if (e != cudaSuccess) return e;
    flash_fwd_kernel<64><<<grid, kAttnThreads, Tiles<64>::kSmem, stream>>>(p);
  }
  return cudaGetLastError();
}

int decode_workspace_floats(int batch, int num_q_heads, int head_dim, int splits) {
  return batch * num_q_heads * splits * (head_dim + 1);
}

namespace {
// Shared by the local and the one-launch distributed form.  `tail` == nullptr: local.
cudaError_t launch_splitkv_impl(const DecodeArgs& a, const DistTail* tail, cudaStream_t stream) {
  if (a.head_dim != 64 && a.head_dim != 128) return cudaErrorInvalidValue;
  if (a.num_q_heads % a.kv.num_kv_heads != 0 || a.splits < 1) return cudaErrorInvalidValue;
  if (a.batch == 0) return cudaSuccess;
  DecodeParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.part_out = a.workspace;
  p.part_lse = a.workspace + static_cast<int64_t>(a.batch) * a.num_q_heads * a.splits * a.head_dim;
  p.kv_lens = a.kv_lens;
  p.kv = make_kv(a.kv);
  p.Hq = a.num_q_heads;
  p.group = a.num_q_heads / a.kv.num_kv_heads;
  p.head_chunks = (p.group + 15) / 16;
  p.splits = a.splits;
  p.scale = a.scale;
  p.softcap = a.softcap;
  p.fuse_counters = (a.fuse_counters != nullptr && a.fuse_out != nullptr) ? a.fuse_counters : nullptr;
  p.fuse_out = reinterpret_cast<__nv_bfloat16*>(a.fuse_out);
  dim3 grid(a.splits, a.kv.num_kv_heads * p.head_chunks, a.batch);
  // A grid of at most one CTA per SM is latency-bound: four stages (three blocks in flight per CTA) instead of two.
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool deep = static_cast<int64_t>(grid.x) * grid.y * grid.z <= sms;
  if (tail != nullptr) {
    // the merge tail keeps 16 * splits + 32 floats in shared memory; waiting chunk CTAs must leave SMs for the rest
    if (p.fuse_counters == nullptr || static_cast<int64_t>(grid.y) * grid.z > sms) return cudaErrorInvalidValue;
    auto launch = [&](auto kernel, int smem, SmemOptIn* set) -> cudaError_t {
      cudaError_t e = ensure_smem(kernel, smem, set);
      if (e != cudaSuccess) return e;
      return launch_pdl(kernel, grid, dim3(kAttnThreads), static_cast<size_t>(smem), stream, p, *tail);
    };
    static SmemOptIn d128_2, d128_4, d64_2, d64_4;
    if (a.head_dim == 128) {
      return deep ? launch(decode_splitkv_dist_kernel<128, 4>, 2 * Tiles<128>::kSmem, &d128_4)
                  : launch(decode_splitkv_dist_kernel<128, 2>, Tiles<128>::kSmem, &d128_2);
    }
    return deep ? launch(decode_splitkv_dist_kernel<64, 4>, 2 * Tiles<64>::kSmem, &d64_4)
                : launch(decode_splitkv_dist_kernel<64, 2>, Tiles<64>::kSmem, &d64_2);
  }
  auto launch = [&](auto kernel, int smem, SmemOptIn* set) -> cudaError_t {
    cudaError_t e = ensure_smem(kernel, smem, set);
    if (e != cudaSuccess) return e;
    return launch_pdl(kernel, grid, dim3(kAttnThreads), static_cast<size_t>(smem), stream, p);
  };
  static SmemOptIn set128_2, set128_4, set64_2, set64_4;
  if (a.head_dim == 128) {
    return deep ? launch(decode_splitkv_kernel<128, 4>, 2 * Tiles<128>::kSmem, &set128_4)
                : launch(decode_splitkv_kernel<128, 2>, Tiles<128>::kSmem, &set128_2);
  }
  return deep ? launch(decode_splitkv_kernel<64, 4>, 2 * Tiles<64>::kSmem, &set64_4)
              : launch(decode_splitkv_kernel<64, 2>, Tiles<64>::kSmem, &set64_2);
}
}  // namespace

cudaError_t launch_decode_splitkv(const DecodeArgs& a, cudaStream_t stream) { return launch_splitkv_impl(a, nullptr, stream); }

cudaError_t launch_dist_decode_fused(const DecodeArgs& a, void* staging, int64_t staging_half_packets, CtxDev* ctx,
                                     const SymmInfoHost& symm, cudaStream_t stream) {
  if (a.batch == 0) return cudaSuccess;
  DistTail t;
  t.staging = reinterpret_cast<uint64_t*>(staging);
  t.staging_half = staging_half_packets;
  t.BH = a.batch * a.num_q_heads;
  t.ctx = ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&t.symm, &symm, sizeof(SymmInfo));
  if (static_cast<int64_t>(symm.world) * t.BH * (a.head_dim + 1) > staging_half_packets) return cudaErrorInvalidValue;
  return launch_splitkv_impl(a, &t, stream);
}

cudaError_t launch_decode_combine(const DecodeArgs& a, void* out_bf16, float* out_lse, float* out_f32,
                                  cudaStream_t stream) {
  if (a.batch == 0) return cudaSuccess;
  const float* part_out = a.workspace;
  const float* part_lse = a.workspace + static_cast<int64_t>(a.batch) * a.num_q_heads * a.splits * a.head_dim;
  decode_combine_kernel<<<a.batch * a.num_q_heads, a.head_dim, 0, stream>>>(
      part_out, part_lse, reinterpret_cast<__nv_bfloat16*>(out_bf16), out_lse, out_f32, a.splits, a.head_dim);
  return cudaGetLastError();
}

cudaError_t launch_dist_combine(const DecodeArgs& a, void* out_bf16, void* staging, int64_t staging_half_packets,
                                CtxDev* ctx, const SymmInfoHost& symm, cudaStream_t stream) {
  if (a.batch == 0) return cudaSuccess;
  DistCombineParams p;
  p.part_out = a.workspace;
  p.part_lse = a.workspace + static_cast<int64_t>(a.batch) * a.num_q_heads * a.splits * a.head_dim;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.staging = reinterpret_cast<uint64_t*>(staging);
  p.staging_half = staging_half_packets;
  p.splits = a.splits;
  p.D = a.head_dim;
  p.BH = a.batch * a.num_q_heads;
  p.ctx = ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &symm, sizeof(SymmInfo));
  if (static_cast<int64_t>(symm.world) * p.BH * (p.D + 1) > staging_half_packets) return cudaErrorInvalidValue;
  dist_combine_kernel<<<p.BH, a.head_dim + 1, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace tdb

// ---------------------------------------------------------------------------
// Allocation-free decode attention (see tdb/noalloc.h for the contract and for who needs it).
// The split-KV partials live in a fixed array of the library image.  In host code the array's name is only a
// stand-in for the symbol, not a device address, so the address is fetched per device with
// cudaGetSymbolAddress before it is handed to the kernels.
// ---------------------------------------------------------------------------
#include <cstdio>

#include "tdb/noalloc.h"

namespace {

constexpr int64_t kNoAllocFloats = 1 << 20;  // 4 MiB
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) float g_decode_scratch[kNoAllocFloats];

// device address of the array per device ordinal; published once, concurrent first calls store the same value
std::atomic<float*> g_scratch_addr[kNoAllocMaxDevices];
thread_local char g_noalloc_err[256] = "";

int noalloc_fail(int code, const char* what, const char* detail) {
  snprintf(g_noalloc_err, sizeof(g_noalloc_err), "%s%s%s", what, detail ? ": " : "", detail ? detail : "");
  return code;
}

}  // namespace

extern "C" int64_t tdb_decode_attn_noalloc_capacity(void) { return kNoAllocFloats; }

extern "C" const char* tdb_noalloc_last_error(void) { return g_noalloc_err; }

extern "C" int tdb_decode_attn_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* block_table, const int32_t* kv_lens, void* out, int batch,
                                       int num_q_heads, int num_kv_heads, int head_dim, int page_size, int max_pages,
                                       int splits, float scale, float softcap, void* stream) {
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || block_table == nullptr || kv_lens == nullptr ||
      out == nullptr)
    return noalloc_fail(TDB_NOALLOC_BAD_ARGUMENT, "null pointer argument", nullptr);
  if (batch < 0 || num_q_heads < 1 || num_kv_heads < 1 || num_q_heads % num_kv_heads != 0 || page_size < 1 ||
      max_pages < 1 || splits < 1 || (head_dim != 64 && head_dim != 128))
    return noalloc_fail(TDB_NOALLOC_BAD_ARGUMENT, "bad shape argument (head_dim must be 64 or 128, heads divisible)",
                        nullptr);
  const int64_t need = static_cast<int64_t>(batch) * num_q_heads * splits * (head_dim + 1);
  if (need > kNoAllocFloats) {
    char msg[160];
    snprintf(msg, sizeof(msg), "batch*heads*splits*(head_dim+1) = %lld floats exceeds the built-in scratch of %lld floats",
             static_cast<long long>(need), static_cast<long long>(kNoAllocFloats));
    return noalloc_fail(TDB_NOALLOC_TOO_LARGE, "request too large", msg);
  }
  if (batch == 0) return TDB_NOALLOC_OK;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(TDB_NOALLOC_CUDA_ERROR, "cudaGetDevice", cudaGetErrorString(e));
  if (dev < 0 || dev >= kNoAllocMaxDevices) return noalloc_fail(TDB_NOALLOC_BAD_ARGUMENT, "device ordinal out of range", nullptr);
  float* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // first call on this device (it is the current one): resolve the symbol to its address on this device
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_decode_scratch);
    if (e != cudaSuccess || scratch == nullptr)
      return noalloc_fail(TDB_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress", cudaGetErrorString(e));
    g_scratch_addr[dev].store(scratch, std::memory_order_release);
  }
  tdb::DecodeArgs a;
  a.q = q;
  a.workspace = scratch;
  a.kv_lens = kv_lens;
  a.kv.k_cache = k_cache;
  a.kv.v_cache = v_cache;
  a.kv.block_table = block_table;
  a.kv.max_pages = max_pages;
  a.kv.page_size = page_size;
  a.kv.num_kv_heads = num_kv_heads;
  a.batch = batch;
  a.num_q_heads = num_q_heads;
  a.head_dim = head_dim;
  a.splits = splits;
  a.scale = scale;
  a.softcap = softcap;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  e = tdb::launch_decode_splitkv(a, s);
  if (e != cudaSuccess) return noalloc_fail(TDB_NOALLOC_CUDA_ERROR, "split-KV launch", cudaGetErrorString(e));
  e = tdb::launch_decode_combine(a, out, nullptr, nullptr, s);
  if (e != cudaSuccess) return noalloc_fail(TDB_NOALLOC_CUDA_ERROR, "combine launch", cudaGetErrorString(e));
  return TDB_NOALLOC_OK;
}
