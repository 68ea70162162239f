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
#include "tdb/attn.h"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kBlockN = 64;   // KV tokens per shared-memory block
constexpr int kAttnThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

TDB_DEVICE void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t sz = valid ? 16u : 0u;  // src-size 0 -> 16 bytes of zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
TDB_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
TDB_DEVICE void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
TDB_DEVICE void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
TDB_DEVICE void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}

template <int D>
struct Tiles {
  static constexpr int kPitch = D * 2 + 16;        // bytes per token row in shared memory (conflict-free)
  static constexpr int kTileBytes = kBlockN * kPitch;
  static constexpr int kSmem = 4 * kTileBytes;     // K and V, double buffered
};

// Physical address of token `tok` of sequence `b`, KV head `h` in a paged cache [pages, page_size, Hkv, D].
struct PagedKV {
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const int32_t* block_table;   // [B, max_pages]
  int max_pages;
  int page_size;
  int Hkv;
  TDB_DEVICE int64_t token_offset(int b, int tok, int h, int D) const {
    const int page = block_table[static_cast<int64_t>(b) * max_pages + tok / page_size];
    return ((static_cast<int64_t>(page) * page_size + tok % page_size) * Hkv + h) * D;
  }
};

// Cooperative load of one 64-token K and V block (tokens [t0, t0+64) of the sequence) into shared memory.
template <int D>
TDB_DEVICE void load_kv_block(const PagedKV& kv, int b, int h, int t0, int kv_end, uint8_t* sK, uint8_t* sV) {
  constexpr int kChunksPerRow = D / 8;
  constexpr int kPitch = Tiles<D>::kPitch;
  for (int c = threadIdx.x; c < kBlockN * kChunksPerRow; c += kAttnThreads) {
    const int r = c / kChunksPerRow, ch = c - r * kChunksPerRow;
    const int tok = t0 + r;
    const bool valid = tok < kv_end;
    const int64_t off = valid ? kv.token_offset(b, tok, h, D) + ch * 8 : 0;
    cp_async16(sK + r * kPitch + ch * 16, kv.k + off, valid);
    cp_async16(sV + r * kPitch + ch * 16, kv.v + off, valid);
  }
}

// Per-warp state of a 16-row attention tile.
template <int D>
struct WarpTile {
  uint32_t qf[D / 16][4];
  float o[D / 8][4];
  float m[2], l[2];   // running max (log2 domain) and sum of the rows lane/4 and lane/4 + 8

  TDB_DEVICE void init() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
  // q_lo / q_hi: pointers to the D elements of rows lane/4 and lane/4 + 8 (nullptr = zero row)
  TDB_DEVICE void load_q(const __nv_bfloat16* q_lo, const __nv_bfloat16* q_hi) {
    const int c = 2 * (lane_id() & 3);
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qf[ks][0] = q_lo ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + c) : 0u;
      qf[ks][1] = q_hi ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + c) : 0u;
      qf[ks][2] = q_lo ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + 8 + c) : 0u;
      qf[ks][3] = q_hi ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + 8 + c) : 0u;
    }
  }
  // One step over NT 8-token tiles that start at row `tok_in_block` of the shared-memory block whose first token
  // is global token `t0`.  Scores of tokens >= limit_lo / limit_hi (per row) are masked.
  template <int NT>
  TDB_DEVICE void step(const uint8_t* sK, const uint8_t* sV, int t0, int tok_in_block, int limit_lo, int limit_hi,
                       float scale, float softcap) {
    constexpr int kPitch = Tiles<D>::kPitch;
    const int lane = lane_id();
    const int g = lane >> 2, c = 2 * (lane & 3);
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const uint8_t* krow = sK + (tok_in_block + 8 * j + g) * kPitch;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + (16 * ks + c) * 2);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + (16 * ks + 8 + c) * 2);
        mma_bf16(s[j], qf[ks], b0, b1);
      }
    }
    // scale, soft-cap, mask; row maxima
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = t0 + tok_in_block + 8 * j + c + (e & 1);
        float v = s[j][e] * scale;
        if (softcap > 0.f) v = softcap * tanhf(v / softcap);
        v *= kLog2e;
        const int lim = (e < 2) ? limit_lo : limit_hi;
        v = (tok < lim) ? v : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], mnew[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mnew[r] = fmaxf(m[r], mx[r]);
      const float base = (mnew[r] == -INFINITY) ? 0.f : mnew[r];
      corr[r] = exp2f(m[r] - base);   // m = -inf -> 0
      m[r] = mnew[r];
      mnew[r] = base;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pexp = exp2f(s[j][e] - mnew[e >> 1]);
        s[j][e] = pexp;
        rs[e >> 1] += pexp;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + rs[r];   // per-lane partial sums; reduced at the end
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int t = 0; t < NT / 2; ++t) {
      uint32_t pa[4];
      pa[0] = pack_bf16x2(s[2 * t][0], s[2 * t][1]);
      pa[1] = pack_bf16x2(s[2 * t][2], s[2 * t][3]);
      pa[2] = pack_bf16x2(s[2 * t + 1][0], s[2 * t + 1][1]);
      pa[3] = pack_bf16x2(s[2 * t + 1][2], s[2 * t + 1][3]);
      // ldmatrix.x4.trans: matrices 0/1 = tokens +0..7 / +8..15 of dim tile jd, matrices 2/3 = the same of jd + 1
      const int mat = lane >> 3, row = lane & 7;
      const uint8_t* vbase = sV + (tok_in_block + 16 * t + (mat & 1) * 8 + row) * kPitch + (mat >> 1) * 16;
#pragma unroll
      for (int jd = 0; jd < D / 8; jd += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vbase + jd * 16);
        mma_bf16(o[jd], pa, vb[0], vb[1]);
        mma_bf16(o[jd + 1], pa, vb[2], vb[3]);
      }
    }
  }
  // Finish: reduce the row sums over the quad; returns 1/l and the natural-log LSE of both rows.
  TDB_DEVICE void finish(float (&inv)[2], float (&lse)[2]) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      inv[r] = l[r] > 0.f ? 1.f / l[r] : 0.f;
      lse[r] = l[r] > 0.f ? (m[r] + log2f(l[r])) / kLog2e : -INFINITY;
    }
  }
};

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
struct DecodeParams {
  const __nv_bfloat16* q;
  float* part_out;
  float* part_lse;
  const int32_t* kv_lens;
  PagedKV kv;
  int Hq, group, head_chunks, splits;
  float scale, softcap;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads) decode_splitkv_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  using T = Tiles<D>;
  const int split = blockIdx.x, b = blockIdx.z;
  const int hkv = blockIdx.y / p.head_chunks, hc = blockIdx.y - hkv * p.head_chunks;
  const int kv_len = p.kv_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2;
  // split boundaries in units of 64-token blocks
  const int total_blk = (kv_len + kBlockN - 1) / kBlockN;
  const int per = (total_blk + p.splits - 1) / p.splits;
  const int blk0 = min(total_blk, split * per), blk1 = min(total_blk, blk0 + per);
  // rows = query heads of this KV head (chunk hc of 16)
  const int h_lo = hc * 16 + g, h_hi = h_lo + 8;
  const int head0 = hkv * p.group;
  WarpTile<D> w;
  w.init();
  const __nv_bfloat16* qb = p.q + static_cast<int64_t>(b) * p.Hq * D;
  w.load_q(h_lo < p.group ? qb + static_cast<int64_t>(head0 + h_lo) * D : nullptr,
           h_hi < p.group ? qb + static_cast<int64_t>(head0 + h_hi) * D : nullptr);
  const int nblk = blk1 - blk0;
  if (nblk > 0) {
    load_kv_block<D>(p.kv, b, hkv, blk0 * kBlockN, kv_len, smem, smem + T::kTileBytes);
    cp_async_commit();
  }
  for (int i = 0; i < nblk; ++i) {
    uint8_t* sK = smem + (i & 1) * 2 * T::kTileBytes;
    uint8_t* sV = sK + T::kTileBytes;
    if (i + 1 < nblk) {
      uint8_t* nK = smem + ((i + 1) & 1) * 2 * T::kTileBytes;
      load_kv_block<D>(p.kv, b, hkv, (blk0 + i + 1) * kBlockN, kv_len, nK, nK + T::kTileBytes);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // each warp takes 16 of the block's 64 tokens
    w.template step<2>(sK, sV, (blk0 + i) * kBlockN, warp * 16, kv_len, kv_len, p.scale, p.softcap);
    __syncthreads();
  }
  // merge the 4 warps (different token subsets, same rows) through shared memory
  float inv[2], lse[2];
  w.finish(inv, lse);
  float* red_o = reinterpret_cast<float*>(smem);          // [4 warps][16 rows][D]
  float* red_m = red_o + 4 * 16 * D;                      // [4][16] log2-domain max
  float* red_l = red_m + 64;                              // [4][16] sums
  const int c = 2 * (lane & 3);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
#pragma unroll
    for (int jd = 0; jd < D / 8; ++jd) {
      red_o[(warp * 16 + row) * D + 8 * jd + c] = w.o[jd][2 * r];
      red_o[(warp * 16 + row) * D + 8 * jd + c + 1] = w.o[jd][2 * r + 1];
    }
    if ((lane & 3) == 0) {
      red_m[warp * 16 + row] = w.m[r];
      red_l[warp * 16 + row] = w.l[r];
    }
  }
  __syncthreads();
  // thread t handles row t / 8 and a D/8-wide slice of the dims
  const int row = threadIdx.x >> 3, sl = threadIdx.x & 7;
  const int h = hc * 16 + row;
  if (h < p.group) {
    float mm = -INFINITY;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) mm = fmaxf(mm, red_m[wi * 16 + row]);
    float ll = 0.f, sc[4];
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      sc[wi] = (mm == -INFINITY) ? 0.f : exp2f(red_m[wi * 16 + row] - mm);
      ll += red_l[wi * 16 + row] * sc[wi];
    }
    const float invl = ll > 0.f ? 1.f / ll : 0.f;
    const int64_t base = ((static_cast<int64_t>(b) * p.Hq + head0 + h) * p.splits + split);
    for (int d = sl * (D / 8); d < (sl + 1) * (D / 8); ++d) {
      float acc = 0.f;
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) acc += red_o[(wi * 16 + row) * D + d] * sc[wi];
      p.part_out[base * D + d] = acc * invl;
    }
    if (sl == 0) p.part_lse[base] = ll > 0.f ? (mm + log2f(ll)) / kLog2e : -INFINITY;
  }
}

// Merge `n` partials (out [n, D] with stride, lse [n]) for one (b, head): returns merged row in `acc` (per thread d)
// and the merged LSE.
TDB_DEVICE float merge_partials(const float* part_out, const float* part_lse, int n, int64_t stride_out, int d,
                                float* out_val) {
  float mx = -INFINITY;
  for (int i = 0; i < n; ++i) mx = fmaxf(mx, part_lse[i]);
  float tot = 0.f, acc = 0.f;
  for (int i = 0; i < n; ++i) {
    const float wgt = (mx == -INFINITY) ? 0.f : __expf(part_lse[i] - mx);
    tot += wgt;
    acc += wgt * part_out[i * stride_out + d];
  }
  *out_val = tot > 0.f ? acc / tot : 0.f;
  return tot > 0.f ? mx + __logf(tot) : -INFINITY;
}

// grid = B * Hq, block = D threads.
__global__ void decode_combine_kernel(const float* part_out, const float* part_lse, __nv_bfloat16* out, float* out_lse,
                                      float* out_f32, int splits, int D) {
  const int64_t bh = blockIdx.x;
  const int d = threadIdx.x;
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
cudaError_t ensure_smem(K kernel, int bytes, bool* flag) {
  if (*flag) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) *flag = true;
  return e;
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
    static bool set = false;
    cudaError_t e = ensure_smem(flash_fwd_kernel<128>, Tiles<128>::kSmem, &set);
    if (e != cudaSuccess) return e;
    flash_fwd_kernel<128><<<grid, kAttnThreads, Tiles<128>::kSmem, stream>>>(p);
  } else {
    static bool set = false;
    cudaError_t e = ensure_smem(flash_fwd_kernel<64>, Tiles<64>::kSmem, &set);
    if (e != cudaSuccess) return e;
    flash_fwd_kernel<64><<<grid, kAttnThreads, Tiles<64>::kSmem, stream>>>(p);
  }
  return cudaGetLastError();
}

int decode_workspace_floats(int batch, int num_q_heads, int head_dim, int splits) {
  return batch * num_q_heads * splits * (head_dim + 1);
}

cudaError_t launch_decode_splitkv(const DecodeArgs& a, cudaStream_t stream) {
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
  dim3 grid(a.splits, a.kv.num_kv_heads * p.head_chunks, a.batch);
  if (a.head_dim == 128) {
    static bool set = false;
    cudaError_t e = ensure_smem(decode_splitkv_kernel<128>, Tiles<128>::kSmem, &set);
    if (e != cudaSuccess) return e;
    decode_splitkv_kernel<128><<<grid, kAttnThreads, Tiles<128>::kSmem, stream>>>(p);
  } else {
    static bool set = false;
    cudaError_t e = ensure_smem(decode_splitkv_kernel<64>, Tiles<64>::kSmem, &set);
    if (e != cudaSuccess) return e;
    decode_splitkv_kernel<64><<<grid, kAttnThreads, Tiles<64>::kSmem, stream>>>(p);
  }
  return cudaGetLastError();
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

float* g_scratch_addr[kNoAllocMaxDevices] = {nullptr};
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
  if (g_scratch_addr[dev] == nullptr) {
    // first call on this device (it is the current one): resolve the symbol to its address on this device
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_scratch);
    if (e != cudaSuccess || p == nullptr)
      return noalloc_fail(TDB_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress", cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  tdb::DecodeArgs a;
  a.q = q;
  a.workspace = g_scratch_addr[dev];
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
