// Device-side building blocks of the attention kernels, shared by the stand-alone kernels (attn.cu) and the decode
// megakernel: cp.async staging of paged K/V blocks, the per-warp 16-row online-softmax tile on mma.sync.m16n8k16, the
// split-KV decode step and the LSE merge.
#pragma once
#include "ptx.cuh"

namespace tdb {
namespace attn {

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

struct DecodeParams {
  const __nv_bfloat16* q;
  float* part_out;
  float* part_lse;
  const int32_t* kv_lens;
  PagedKV kv;
  int Hq, group, head_chunks, splits;
  float scale, softcap;
  uint32_t* fuse_counters = nullptr;    // fused combine (see DecodeArgs); null = partials only
  __nv_bfloat16* fuse_out = nullptr;
};

// Body of the split-KV decode step for one (split, kv head x head chunk, sequence).  Executed by 128 threads
// (threadIdx.x < 128); `sync` is a barrier over exactly those threads.
// S = shared-memory stages of (K, V) blocks: S - 1 blocks are in flight while one is computed.
template <int D, typename Sync, int S = 2>
TDB_DEVICE void decode_splitkv_body(const DecodeParams& p, int split, int yidx, int b, uint8_t* smem, Sync sync) {
  using T = Tiles<D>;
  const int hkv = yidx / p.head_chunks, hc = yidx - hkv * p.head_chunks;
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
  // one commit group per block, empty when there is no block left, so that "all but the newest S - 1 groups are
  // complete" always means "block i has landed"
#pragma unroll
  for (int j = 0; j < S - 1; ++j) {
    if (j < nblk) {
      uint8_t* nK = smem + j * 2 * T::kTileBytes;
      load_kv_block<D>(p.kv, b, hkv, (blk0 + j) * kBlockN, kv_len, nK, nK + T::kTileBytes);
    }
    cp_async_commit();
  }
  for (int i = 0; i < nblk; ++i) {
    uint8_t* sK = smem + (i % S) * 2 * T::kTileBytes;
    uint8_t* sV = sK + T::kTileBytes;
    if (i + S - 1 < nblk) {
      uint8_t* nK = smem + ((i + S - 1) % S) * 2 * T::kTileBytes;
      load_kv_block<D>(p.kv, b, hkv, (blk0 + i + S - 1) * kBlockN, kv_len, nK, nK + T::kTileBytes);
    }
    cp_async_commit();
    cp_async_wait<S - 1>();
    sync();
    // each warp takes 16 of the block's 64 tokens
    w.template step<2>(sK, sV, (blk0 + i) * kBlockN, warp * 16, kv_len, kv_len, p.scale, p.softcap);
    sync();
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
  sync();
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
}  // namespace attn
}  // namespace tdb
