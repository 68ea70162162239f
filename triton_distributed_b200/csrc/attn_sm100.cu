// Prefill / context attention on the 5th-generation tensor cores (head dim 128, bf16, GQA, var-len, causal).
//
// Two launches:
//   attn_pack_kv_kernel     gathers the visible KV of every sequence out of the paged cache into TMA-friendly dense
//                           tensors: K [B * Hkv][Lp][D] and V transposed, Vt [B * Hkv][D][Lp] (Lp = padded max length,
//                           zero beyond a sequence's length).  With V transposed both products of attention are plain
//                           K-major x K-major UMMAs, and paging no longer concerns the main kernel.  One read and one
//                           write of the KV, against O(S^2) work in the main kernel.
//   flash_fwd_sm100_kernel  one CTA = 128 query rows of one head.  Warp 0 loads Q once and streams K / Vt blocks of
//                           64 tokens by TMA (two stages); warp 1 issues tcgen05.mma: S = Q K^T (128 x 64, K = 128)
//                           into TMEM, and after the softmax warps have written P (bf16, 128B-swizzled shared
//                           memory) O += P V (128 x 128, K = 64), accumulated in a second TMEM buffer over all blocks;
//                           warps 2-5 (one thread per query row) read S with tcgen05.ld, apply scale / mask / softmax
//                           in the log2 domain and write P.  The output is NOT read back per block: the exponentials
//                           use a reference maximum that is only raised when the row maximum has grown by more than
//                           2^8 (P stays below 256, exact in the final division because O and the row sum share the
//                           reference); only then the warp rescales its O rows in TMEM (tcgen05.ld / st).  S of block
//                           j + 1 is issued as soon as S of block j has been read, so the tensor core works during the
//                           exponentials; the output row is read once, after the last block.
// Every wait is bounded; a timeout is recorded, the CTA stops issuing work, frees its TMEM and returns.
//
// Reference behaviour being matched (not its code): mega_triton_kernel/kernels/flash_attn.py:33-372 (TMA +
// warp-specialised prefill attention), kernels/nvidia/sp_ag_attention_intra_node.py:256-425 (var-len cu_seqlens,
// causal offsets of context-parallel chunks).
#include <cuda.h>
#include <cuda_bf16.h>

#include "tdb/attn.h"
#include "tdb/launch.cuh"
#include "tdb/ptx.cuh"
#include "tdb/status.h"

namespace tdb {

namespace {

constexpr int kD = 128;            // head dim
constexpr int kBM = 128;           // query rows per CTA
constexpr int kBN = 64;            // KV tokens per block
constexpr int kThreads = 192;      // warp 0 TMA, warp 1 MMA, warps 2-5 softmax
constexpr int kUmmaK = 16;
constexpr int kQBytes = kBM * kD * 2;        // 32 KB: two [128 x 64] swizzled halves
constexpr int kKBytes = kBN * kD * 2;        // 16 KB: two [64 x 64] halves
constexpr int kVBytes = kD * kBN * 2;        // 16 KB: Vt block [128 d x 64 tokens]
constexpr int kPBytes = kBM * kBN * 2;       // 16 KB
// Shared-memory layout for a ring of STAGES K / Vt blocks: Q | K ring | Vt ring | P | barriers
template <int STAGES>
struct Lay {
  static constexpr int kOffK = kQBytes;
  static constexpr int kOffV = kOffK + STAGES * kKBytes;
  static constexpr int kOffP = kOffV + STAGES * kVBytes;
  static constexpr int kOffBar = kOffP + kPBytes;
  static constexpr int kSmem = kOffBar + (2 * STAGES + 8) * 8 + 64;
};
static_assert(2 * (Lay<2>::kSmem + 1024) <= 227 * 1024, "two CTAs of the two-stage prefill kernel must fit one SM");
static_assert(Lay<5>::kSmem + 1024 <= 227 * 1024, "the five-stage prefill kernel must fit one SM");
constexpr int kTmemCols = 256;     // S: columns [0, 64), PV: columns [64, 192)
constexpr uint64_t kWaitNs = 4000000000ull;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct FwdParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  float* lse;                  // [Hq, total_q] or null
  const int32_t* cu_seqlens_q;
  const int32_t* q_pos0;
  const int32_t* kv_lens;
  int Hq, Hkv, group, causal;
  float scale_log2;            // scale * log2(e)
  int64_t total_q;
  int* error_flag;             // device int, set on a timeout
};

// ------------------------------------------------------------------------------------------------------------------
// KV packing: grid (Lp / 64, Hkv, B), 256 threads
// ------------------------------------------------------------------------------------------------------------------
struct PackParams {
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int32_t* block_table;
  const int32_t* kv_lens;
  int max_pages, page_size, Hkv, Lp;
  __nv_bfloat16* k_out;        // [B * Hkv][Lp][D]
  __nv_bfloat16* vt_out;       // [B * Hkv][D][Lp]
};

__global__ void __launch_bounds__(256) attn_pack_kv_kernel(const PackParams p) {
  __shared__ __align__(16) __nv_bfloat16 vs[kBN][kD + 8];
  const int t0 = blockIdx.x * kBN, h = blockIdx.y, b = blockIdx.z;
  const int kv_len = p.kv_lens[b];
  const int64_t bh = static_cast<int64_t>(b) * p.Hkv + h;
  for (int i = threadIdx.x; i < kBN * (kD / 8); i += 256) {
    const int r = i / (kD / 8), c = (i % (kD / 8)) * 8;
    const int tok = t0 + r;
    uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = make_uint4(0u, 0u, 0u, 0u);
    if (tok < kv_len) {
      const int page = p.block_table[static_cast<int64_t>(b) * p.max_pages + tok / p.page_size];
      const int64_t off = ((static_cast<int64_t>(page) * p.page_size + tok % p.page_size) * p.Hkv + h) * kD + c;
      kv = *reinterpret_cast<const uint4*>(p.k_cache + off);
      vv = *reinterpret_cast<const uint4*>(p.v_cache + off);
    }
    *reinterpret_cast<uint4*>(p.k_out + (bh * p.Lp + tok) * kD + c) = kv;
    *reinterpret_cast<uint4*>(&vs[r][c]) = vv;
  }
  __syncthreads();
  // Vt[d][t0 .. t0 + 63]: a thread writes 32 consecutive tokens of one d
  const int d = threadIdx.x % kD, half = threadIdx.x / kD;
  __nv_bfloat16* dst = p.vt_out + (bh * kD + d) * p.Lp + t0 + half * 32;
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    __align__(16) __nv_bfloat16 tmp[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) tmp[j] = vs[half * 32 + i + j][d];
    *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(tmp);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Main kernel
// ------------------------------------------------------------------------------------------------------------------
// What one softmax thread (one query row of one 128-row tile) does over all KV blocks of its tile, then the output row.
struct TileCtx {
  uint64_t* s_full;
  uint64_t* s_free;
  uint64_t* p_full;
  uint64_t* pv_full;
  uint32_t tmem_s, tmem_pv;
  uint8_t* p_smem;             // this tile's P buffer
  int row0, rows_here, nblk;
};

__device__ __forceinline__ void softmax_tile(const FwdParams& p, const TileCtx& t, int warp, int lane, int q_begin, int head,
                                             int kv_len, int pos0, volatile int* abort_flag) {
  uint64_t* s_full = t.s_full;
  uint64_t* s_free = t.s_free;
  uint64_t* p_full = t.p_full;
  uint64_t* pv_full = t.pv_full;
  const uint32_t tmem_s = t.tmem_s, tmem_pv = t.tmem_pv;
  const int row0 = t.row0, rows_here = t.rows_here, nblk = t.nblk;
  const int qd = warp & 3;                       // TMEM lane quarter this warp may access
  const int row = qd * 32 + lane;                // row inside the tile
  const bool row_ok = row < rows_here;
  const int pos = pos0 + row0 + row;             // absolute position of the query
  const int lim = p.causal ? min(kv_len, pos + 1) : kv_len;   // tokens [0, lim) are visible
  const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
  constexpr float kRescaleStep = 8.f;            // log2: the reference maximum follows the row maximum in steps of 2^8
  float m = -INFINITY, l = 0.f;                  // m: reference maximum the exponentials of this row use
  uint8_t* prow = t.p_smem + row * 128;
  const int sw = row & 7;
  bool ok = true;
  for (int j = 0; j < nblk; ++j) {
    if (!mbar_wait(s_full, j & 1, abort_flag, kWaitNs)) { ok = false; break; }
    tc_fence_after_sync();
    uint32_t s0[32], s1[32];
    tmem_ld_32x32(tmem_s + lane_off, s0);
    tmem_ld_32x32(tmem_s + lane_off + 32, s1);
    tmem_ld_wait();
    tc_fence_before_sync();
    mbar_arrive(s_free);                          // S may be overwritten by the next block's product
    const int t0 = j * kBN;
    // Blocks that every row of the warp sees completely (all but the ones on the causal diagonal and the last one of
    // a sequence) skip the masking; the scale is folded into the exponent (one FMA per element), so an element
    // costs a max, an FMA, an ex2, an add and half a pack.
    const bool full = __all_sync(0xffffffffu, t0 + kBN <= lim);
    if (!full) {
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        if (t0 + c >= lim) s0[c] = 0xff800000u;          // -inf
        if (t0 + 32 + c >= lim) s1[c] = 0xff800000u;
      }
    }
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
    mx *= p.scale_log2;                                   // scale > 0: the maximum commutes with it
    // raise the reference only when the row maximum has outgrown it by more than the step (or there is none yet)
    float alpha = 1.f;
    bool raise = false;
    if (mx > m) {
      if (m == -INFINITY) {
        m = mx;                                   // nothing accumulated for this row so far (its P were all zero)
      } else if (mx - m > kRescaleStep) {
        alpha = ex2(m - mx);
        m = mx;
        raise = true;
      }
    }
    const float m_use = (m == -INFINITY) ? 0.f : m;
    // the previous block's PV must have finished: it read the P buffer that is rewritten below, and it wrote the O
    // rows a rescale touches (issued long ago: this wait is normally already satisfied)
    if (j > 0 && !mbar_wait(pv_full, (j - 1) & 1, abort_flag, kWaitNs)) { ok = false; break; }
    if (__any_sync(0xffffffffu, raise)) {
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_pv + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st_32x32(tmem_pv + lane_off + c * 32, r);
      }
      tmem_st_wait();
      tc_fence_before_sync();
    }
    float sum = 0.f;
    // P row: 64 bf16 = eight 16-byte chunks, chunk c stored at (c ^ (row & 7)) (128-byte swizzle)
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = c8 * 8 + 2 * e;
        const float x0 = ex2(fmaf(__uint_as_float(c < 32 ? s0[c] : s1[c - 32]), p.scale_log2, -m_use));
        const float x1 = ex2(fmaf(__uint_as_float(c + 1 < 32 ? s0[c + 1] : s1[c + 1 - 32]), p.scale_log2, -m_use));
        sum += x0 + x1;
        pk[e] = pack_bf16x2(x0, x1);
      }
      *reinterpret_cast<uint4*>(prow + ((c8 ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
    l = l * alpha + sum;
    fence_proxy_async_smem();                     // P was written through the generic proxy, the MMA reads it through the async proxy
    mbar_arrive(p_full);
  }
  float o[kD];
#pragma unroll
  for (int i = 0; i < kD; ++i) o[i] = 0.f;
  if (ok && nblk > 0) {
    if (!mbar_wait(pv_full, (nblk - 1) & 1, abort_flag, kWaitNs)) {
      ok = false;
    } else {
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_pv + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = __uint_as_float(r[i]);
      }
      tc_fence_before_sync();
    }
  }
  if (!ok) *abort_flag = 1;
  if (ok && row_ok) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* orow = p.out + ((static_cast<int64_t>(q_begin) + row0 + row) * p.Hq + head) * kD;
#pragma unroll
    for (int c = 0; c < kD / 8; ++c) {
      uint4 v;
      v.x = pack_bf16x2(o[8 * c + 0] * inv, o[8 * c + 1] * inv);
      v.y = pack_bf16x2(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
      v.z = pack_bf16x2(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
      v.w = pack_bf16x2(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
      *reinterpret_cast<uint4*>(orow + 8 * c) = v;
    }
    if (p.lse != nullptr)
      p.lse[static_cast<int64_t>(head) * p.total_q + q_begin + row0 + row] =
          l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
}

template <int kStages, int kCtasPerSm>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
flash_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_vt, const FwdParams p) {
  // Two CTAs share an SM (one runs its exponentials while the other's products are on the tensor core), which leaves no
  // room for an alignment slack: the kernel has no static shared memory, so the dynamic window starts at offset 0 of the
  // CTA's allocation; the 1024-byte alignment the swizzled tiles need is checked, not assumed.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.error_flag != nullptr) *p.error_flag = 2;
    return;
  }
  using L = Lay<kStages>;
  constexpr int kOffK = L::kOffK, kOffV = L::kOffV, kOffP = L::kOffP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars;
  uint64_t* s_full = bars + 1;
  uint64_t* s_free = bars + 2;
  uint64_t* p_full = bars + 3;
  uint64_t* pv_full = bars + 4;
  uint64_t* kv_full = bars + 5;                 // [kStages]
  uint64_t* kv_empty = kv_full + kStages;       // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_empty + kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int b = blockIdx.z, head = blockIdx.y;
  const int q_begin = p.cu_seqlens_q[b], q_len = p.cu_seqlens_q[b + 1] - q_begin;
  // causal tiles get longer towards the end of a sequence: the long ones are scheduled first (the block scheduler hands
  // out blockIdx.x in increasing order), so the tail of the launch consists of short tiles
  const int row0 = (p.causal ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x)) * kBM;
  if (row0 >= q_len) return;                      // whole CTA, before any barrier or TMEM use
  const int kv_len = p.kv_lens[b];
  const int pos0 = p.q_pos0 ? p.q_pos0[b] : (kv_len - q_len);
  const int hkv = head / p.group;
  const int rows_here = min(q_len - row0, kBM);
  int kv_end = p.causal ? min(kv_len, pos0 + row0 + rows_here) : kv_len;
  if (kv_end < 0) kv_end = 0;
  const int nblk = (kv_end + kBN - 1) / kBN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 128);
    mbar_init(p_full, 128);
    mbar_init(pv_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 64;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_vt);
      mbar_arrive_expect_tx(q_full, kQBytes);
      tma_load_2d(smem, &tmap_q, q_full, head * kD, q_begin + row0);
      tma_load_2d(smem + kQBytes / 2, &tmap_q, q_full, head * kD + 64, q_begin + row0);
      const int z = b * p.Hkv + hkv;
      for (int j = 0; j < nblk; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, abort_flag, kWaitNs)) {
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[s], kKBytes + kVBytes);
        uint8_t* sk = smem + kOffK + s * kKBytes;
        tma_load_3d(sk, &tmap_k, &kv_full[s], 0, j * kBN, z);
        tma_load_3d(sk + kKBytes / 2, &tmap_k, &kv_full[s], 64, j * kBN, z);
        tma_load_3d(smem + kOffV + s * kVBytes, &tmap_vt, &kv_full[s], j * kBN, 0, z);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(1u, kBM, kBN);
      constexpr uint32_t idesc_pv = make_idesc(1u, kBM, kD);
      bool ok = mbar_wait(q_full, 0, abort_flag, kWaitNs);
      const uint32_t sq = smem_u32(smem);
      const uint32_t sp = smem_u32(smem + kOffP);
      auto issue_s = [&](int j) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(&kv_full[s], (j / kStages) & 1, abort_flag, kWaitNs)) return false;
        if (j > 0 && !mbar_wait(s_free, (j - 1) & 1, abort_flag, kWaitNs)) return false;
        tc_fence_after_sync();
        const uint32_t sk = smem_u32(smem + kOffK + s * kKBytes);
#pragma unroll
        for (int k = 0; k < kD / kUmmaK; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(sq + (k / 4) * (kQBytes / 2)) + 2 * (k % 4);
          const uint64_t bdesc = make_smem_desc_sw128(sk + (k / 4) * (kKBytes / 2)) + 2 * (k % 4);
          umma_f16(tmem_s, adesc, bdesc, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        return true;
      };
      if (ok && nblk > 0) ok = issue_s(0);
      for (int j = 0; j < nblk && ok; ++j) {
        // S of the next block goes out before this block's P is waited for: it only needs S of block j to have been read
        if (j + 1 < nblk) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(p_full, j & 1, abort_flag, kWaitNs)) { ok = false; break; }
        tc_fence_after_sync();
        const int s = j % kStages;
        const uint32_t sv = smem_u32(smem + kOffV + s * kVBytes);
#pragma unroll
        for (int k = 0; k < kBN / kUmmaK; ++k)
          umma_f16(tmem_pv, make_smem_desc_sw128(sp) + 2 * k, make_smem_desc_sw128(sv) + 2 * k, idesc_pv,
                   (j > 0 || k > 0) ? 1u : 0u);   // O accumulates over all blocks
        umma_commit(pv_full);
        umma_commit(&kv_empty[s]);      // K (read by S of this block) and Vt of this stage are free again
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ softmax + output (one thread per query row)
    TileCtx t;
    t.s_full = s_full; t.s_free = s_free; t.p_full = p_full; t.pv_full = pv_full;
    t.tmem_s = tmem_s; t.tmem_pv = tmem_pv;
    t.p_smem = smem + kOffP;
    t.row0 = row0; t.rows_here = rows_here; t.nblk = nblk;
    softmax_tile(p, t, warp, lane, q_begin, head, kv_len, pos0, abort_flag);
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.error_flag != nullptr) *p.error_flag = 1;
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Two-tile form: one CTA per SM handles 256 query rows as two 128-row tiles that share every K / Vt block (half the
// L2 -> shared-memory traffic per FLOP, and room for a three-stage ring, so a block is requested two blocks before it is
// needed).  320 threads: warp 0 TMA, warp 1 MMA, warps 2-5 softmax of tile 0, warps 6-9 softmax of tile 1; while one
// tile's rows are in their exponentials the other tile's products are on the tensor core.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kPPThreads = 320;
template <int STAGES>
struct LayPP {
  static constexpr int kOffK = 2 * kQBytes;
  static constexpr int kOffV = kOffK + STAGES * kKBytes;
  static constexpr int kOffP = kOffV + STAGES * kVBytes;
  static constexpr int kOffBar = kOffP + 2 * kPBytes;
  static constexpr int kSmem = kOffBar + (2 * STAGES + 12) * 8 + 64;
};
static_assert(LayPP<3>::kSmem + 1024 <= 227 * 1024, "the two-tile prefill kernel must fit one SM");

template <int kStages>
__global__ void __launch_bounds__(kPPThreads, 1)
flash_fwd_sm100_pp_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_vt, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = LayPP<kStages>;
  constexpr int kOffK = L::kOffK, kOffV = L::kOffV, kOffP = L::kOffP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars;
  uint64_t* s_full = bars + 1;        // [2] per tile
  uint64_t* s_free = bars + 3;
  uint64_t* p_full = bars + 5;
  uint64_t* pv_full = bars + 7;
  uint64_t* kv_full = bars + 9;                 // [kStages]
  uint64_t* kv_empty = kv_full + kStages;       // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_empty + kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int b = blockIdx.z, head = blockIdx.y;
  const int q_begin = p.cu_seqlens_q[b], q_len = p.cu_seqlens_q[b + 1] - q_begin;
  const int row0 = (p.causal ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x)) * (2 * kBM);
  if (row0 >= q_len) return;                      // whole CTA, before any barrier or TMEM use
  const int kv_len = p.kv_lens[b];
  const int pos0 = p.q_pos0 ? p.q_pos0[b] : (kv_len - q_len);
  const int hkv = head / p.group;
  int rows_t[2], nblk_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    rows_t[t] = max(0, min(q_len - (row0 + t * kBM), kBM));
    int kv_end = p.causal ? min(kv_len, pos0 + row0 + t * kBM + rows_t[t]) : kv_len;
    if (kv_end < 0) kv_end = 0;
    nblk_t[t] = rows_t[t] > 0 ? (kv_end + kBN - 1) / kBN : 0;
  }
  const int nblk = max(nblk_t[0], nblk_t[1]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&s_free[t], 128);
      mbar_init(&p_full[t], 128);
      mbar_init(&pv_full[t], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;          // tile t: S at columns [256 t, 256 t + 64), O at [256 t + 64, 256 t + 192)

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_vt);
      // both Q tiles (rows beyond the sequence or the tensor read other rows or zeros; they are never written out)
      mbar_arrive_expect_tx(q_full, 2 * kQBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_2d(smem + t * kQBytes, &tmap_q, q_full, head * kD, q_begin + row0 + t * kBM);
        tma_load_2d(smem + t * kQBytes + kQBytes / 2, &tmap_q, q_full, head * kD + 64, q_begin + row0 + t * kBM);
      }
      const int z = b * p.Hkv + hkv;
      for (int j = 0; j < nblk; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, abort_flag, kWaitNs)) {
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[s], kKBytes + kVBytes);
        uint8_t* sk = smem + kOffK + s * kKBytes;
        tma_load_3d(sk, &tmap_k, &kv_full[s], 0, j * kBN, z);
        tma_load_3d(sk + kKBytes / 2, &tmap_k, &kv_full[s], 64, j * kBN, z);
        tma_load_3d(smem + kOffV + s * kVBytes, &tmap_vt, &kv_full[s], j * kBN, 0, z);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(1u, kBM, kBN);
      constexpr uint32_t idesc_pv = make_idesc(1u, kBM, kD);
      bool ok = mbar_wait(q_full, 0, abort_flag, kWaitNs);
      auto issue_s = [&](int t, int j) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(&kv_full[s], (j / kStages) & 1, abort_flag, kWaitNs)) return false;
        if (j > 0 && !mbar_wait(&s_free[t], (j - 1) & 1, abort_flag, kWaitNs)) return false;
        tc_fence_after_sync();
        const uint32_t sq = smem_u32(smem + t * kQBytes);
        const uint32_t sk = smem_u32(smem + kOffK + s * kKBytes);
#pragma unroll
        for (int k = 0; k < kD / kUmmaK; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(sq + (k / 4) * (kQBytes / 2)) + 2 * (k % 4);
          const uint64_t bdesc = make_smem_desc_sw128(sk + (k / 4) * (kKBytes / 2)) + 2 * (k % 4);
          umma_f16(tmem_base + t * 256, adesc, bdesc, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        if (!mbar_wait(&p_full[t], j & 1, abort_flag, kWaitNs)) return false;
        tc_fence_after_sync();
        const uint32_t sp = smem_u32(smem + kOffP + t * kPBytes);
        const uint32_t sv = smem_u32(smem + kOffV + (j % kStages) * kVBytes);
#pragma unroll
        for (int k = 0; k < kBN / kUmmaK; ++k)
          umma_f16(tmem_base + t * 256 + 64, make_smem_desc_sw128(sp) + 2 * k, make_smem_desc_sw128(sv) + 2 * k, idesc_pv,
                   (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&pv_full[t]);
        return true;
      };
      for (int t = 0; t < 2 && ok; ++t)
        if (nblk_t[t] > 0) ok = issue_s(t, 0);
      for (int j = 0; j < nblk && ok; ++j) {
        // per tile: S of the next block as soon as this block's S has been read, then this block's P V
        for (int t = 0; t < 2 && ok; ++t) {
          if (j + 1 < nblk_t[t]) ok = issue_s(t, j + 1);
          if (ok && j < nblk_t[t]) ok = issue_pv(t, j);
        }
        if (ok) umma_commit(&kv_empty[j % kStages]);   // every product that reads this stage has been issued before
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int t = (warp - 2) >> 2;                 // warps 2-5: tile 0, warps 6-9: tile 1
    TileCtx c;
    c.s_full = &s_full[t]; c.s_free = &s_free[t]; c.p_full = &p_full[t]; c.pv_full = &pv_full[t];
    c.tmem_s = tmem_base + t * 256; c.tmem_pv = tmem_base + t * 256 + 64;
    c.p_smem = smem + kOffP + t * kPBytes;
    c.row0 = row0 + t * kBM; c.rows_here = rows_t[t]; c.nblk = nblk_t[t];
    softmax_tile(p, c, warp, lane, q_begin, head, kv_len, pos0, abort_flag);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.error_flag != nullptr) *p.error_flag = 1;
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

cudaError_t launch_flash_fwd_sm100(const FlashFwdSm100Args& a, cudaStream_t stream) {
  if (a.head_dim != kD || a.num_q_heads % a.num_kv_heads != 0 || a.Lp % kBN != 0 || a.Lp <= 0) return cudaErrorInvalidValue;
  if (!(a.scale > 0.f)) return cudaErrorInvalidValue;   // the row maximum is taken before scaling
  if (a.batch == 0 || a.max_q_len == 0) return cudaSuccess;
  PackParams pk;
  pk.k_cache = reinterpret_cast<const __nv_bfloat16*>(a.kv.k_cache);
  pk.v_cache = reinterpret_cast<const __nv_bfloat16*>(a.kv.v_cache);
  pk.block_table = a.kv.block_table;
  pk.kv_lens = a.kv_lens;
  pk.max_pages = a.kv.max_pages;
  pk.page_size = a.kv.page_size;
  pk.Hkv = a.num_kv_heads;
  pk.Lp = a.Lp;
  pk.k_out = reinterpret_cast<__nv_bfloat16*>(a.k_dense);
  pk.vt_out = reinterpret_cast<__nv_bfloat16*>(a.vt_dense);
  attn_pack_kv_kernel<<<dim3(a.Lp / kBN, a.num_kv_heads, a.batch), 256, 0, stream>>>(pk);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  TensorMap tq, tk, tv;
  const uint64_t bh = static_cast<uint64_t>(a.batch) * a.num_kv_heads;
  if (encode_tensor_map_2d(&tq, a.q, kBF16, static_cast<uint64_t>(a.total_q), static_cast<uint64_t>(a.num_q_heads) * kD,
                           static_cast<uint64_t>(a.num_q_heads) * kD * 2, kBM, 64, 128) != 0)
    return cudaErrorInvalidValue;
  if (encode_tensor_map_3d(&tk, a.k_dense, kBF16, bh, static_cast<uint64_t>(a.Lp), kD, kD * 2,
                           static_cast<uint64_t>(a.Lp) * kD * 2, kBN, 64, 128) != 0)
    return cudaErrorInvalidValue;
  if (encode_tensor_map_3d(&tv, a.vt_dense, kBF16, bh, kD, static_cast<uint64_t>(a.Lp), static_cast<uint64_t>(a.Lp) * 2,
                           static_cast<uint64_t>(a.Lp) * kD * 2, kD, 64, 128) != 0)
    return cudaErrorInvalidValue;
  FwdParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.lse = a.lse;
  p.cu_seqlens_q = a.cu_seqlens_q;
  p.q_pos0 = a.q_pos0;
  p.kv_lens = a.kv_lens;
  p.Hq = a.num_q_heads;
  p.Hkv = a.num_kv_heads;
  p.group = a.num_q_heads / a.num_kv_heads;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.total_q = a.total_q;
  p.error_flag = a.error_flag;
  dim3 grid((a.max_q_len + kBM - 1) / kBM, a.num_q_heads, a.batch);
  CUtensorMap mq, mk, mv;
  memcpy(&mq, tq.bytes, sizeof(mq));
  memcpy(&mk, tk.bytes, sizeof(mk));
  memcpy(&mv, tv.bytes, sizeof(mv));
  // Three forms: (2) two CTAs per SM with a two-stage KV ring (one CTA's exponentials overlap the other's products),
  // (1) one CTA per SM with a five-stage ring, (3) one CTA per SM with two query tiles sharing a three-stage ring.
  // TDB200_ATTN_FORM selects; default = the fastest measured.
  static const int form = [] {
    const char* e = std::getenv("TDB200_ATTN_FORM");
    return e != nullptr ? std::atoi(e) : 2;
  }();
  if (form == 3) {
    static SmemOptIn opt3;
    e = opt3.ensure(flash_fwd_sm100_pp_kernel<3>, LayPP<3>::kSmem + 1024);
    if (e != cudaSuccess) return e;
    dim3 grid2((a.max_q_len + 2 * kBM - 1) / (2 * kBM), a.num_q_heads, a.batch);
    flash_fwd_sm100_pp_kernel<3><<<grid2, kPPThreads, LayPP<3>::kSmem + 1024, stream>>>(mq, mk, mv, p);
  } else if (form == 1) {
    static SmemOptIn opt1;
    e = opt1.ensure(flash_fwd_sm100_kernel<5, 1>, Lay<5>::kSmem);
    if (e != cudaSuccess) return e;
    flash_fwd_sm100_kernel<5, 1><<<grid, kThreads, Lay<5>::kSmem, stream>>>(mq, mk, mv, p);
  } else {
    static SmemOptIn opt2;
    e = opt2.ensure(flash_fwd_sm100_kernel<2, 2>, Lay<2>::kSmem);
    if (e != cudaSuccess) return e;
    flash_fwd_sm100_kernel<2, 2><<<grid, kThreads, Lay<2>::kSmem, stream>>>(mq, mk, mv, p);
  }
  return cudaGetLastError();
}

}  // namespace tdb
