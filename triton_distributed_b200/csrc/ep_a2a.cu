// Expert-parallel all-to-all: dispatch (optionally quantising rows to fp8 e4m3 with one fp32 scale per 128 elements
// while they are sent) and combine (rows return to the token's owner, where the top-k weighted sum is taken in the same
// kernel); plus torch.distributed.all_to_all_single semantics with uneven splits, and stand-alone quant / dequant.
//
// Reference behaviour being matched (not its code):
//   low-latency all-to-all   kernels/nvidia/low_latency_all_to_all.py:36-279 (fixed-stride receive areas, split counts
//                            travel with the data, double buffering by call parity, monotonically increasing signal)
//   fused fp8 quantisation   tutorials/04-deepseek-infer-all2all.py:93-275 (scale = amax / 448 per 128 elements)
//   throughput dispatch      kernels/nvidia/ep_a2a.py:38-447 (slot ranges private to the source rank, so only LOCAL
//                            atomics are needed; slot remembered for combine), layers/nvidia/ep_a2a_layer.py:154-341
//   all_to_all_single_2d     kernels/nvidia/all_to_all_single_2d.py:41-171
// Differences by design: receive counts never travel through the CPU; the weighted top-k reduction of combine is fused;
// all waits are bounded.
#include <cuda_fp8.h>

#include "tdb/ep.h"
#include "tdb/launch.cuh"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kEpThreads = 256;
constexpr int kQuantBlock = 128;

TDB_DEVICE uint32_t quant4(float a, float b, float c, float d, float inv_scale) {
  const uint32_t q0 = __nv_cvt_float_to_fp8(a * inv_scale, __NV_SATFINITE, __NV_E4M3);
  const uint32_t q1 = __nv_cvt_float_to_fp8(b * inv_scale, __NV_SATFINITE, __NV_E4M3);
  const uint32_t q2 = __nv_cvt_float_to_fp8(c * inv_scale, __NV_SATFINITE, __NV_E4M3);
  const uint32_t q3 = __nv_cvt_float_to_fp8(d * inv_scale, __NV_SATFINITE, __NV_E4M3);
  return q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
}
TDB_DEVICE float fp8_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// One warp quantises one bf16 row of H elements (H % 128 == 0) into fp8 + H/128 scales and writes both.
// (blocks [b_begin, b_end) of the row when several warps share it)
TDB_DEVICE void warp_quant_row(const __nv_bfloat16* src, uint8_t* dst_q, float* dst_s, int H, int b_begin = 0, int b_end = -1) {
  const int lane = lane_id();
  const int nb = b_end < 0 ? H / kQuantBlock : b_end;
  // eight 128-value blocks per step: their loads are in flight together (a block per iteration would pay one memory
  // round trip per block, 56 in a row for a 7168-wide token)
  for (int b0 = b_begin; b0 < nb; b0 += 8) {
    uint2 u[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      u[j] = (b0 + j < nb) ? *reinterpret_cast<const uint2*>(src + (b0 + j) * kQuantBlock + lane * 4) : make_uint2(0u, 0u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (b0 + j >= nb) break;
      const float2 f0 = unpack_bf16x2(u[j].x), f1 = unpack_bf16x2(u[j].y);
      float amax = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
      amax = fmaxf(warp_max(amax), 1e-10f);
      const float scale = amax / 448.f;
      reinterpret_cast<uint32_t*>(dst_q + (b0 + j) * kQuantBlock)[lane] = quant4(f0.x, f0.y, f1.x, f1.y, 1.f / scale);
      if (lane == 0) dst_s[b0 + j] = scale;
    }
  }
}

struct DispatchParams {
  const __nv_bfloat16* x;        // [T, H] local tokens
  const int32_t* topk_ids;       // [T, k] global expert ids (>= E or < 0: dropped)
  int T, H, k, E, epr;
  int quant;                     // 1: send fp8 + scales
  int max_tokens;                // per-rank token capacity M
  // heap (symmetric) receive side, indexed [parity]
  uint8_t* recv_x;               // rows of row_bytes
  float* recv_scale;             // [rows][H/128]
  int32_t* recv_meta;            // [rows] source pair index t*k+j
  int32_t* recv_count;           // [epr][W]
  uint32_t* flags;               // [W] epoch per source
  uint64_t rows_per_parity;
  // slot layout
  const int32_t* base;           // [W dst][epr][W src] first row of (dst, local expert, src) on dst; null = fixed stride
  int32_t* cursor;               // local [E] (zero on entry)
  int32_t* sent_row;             // local [T*k] row each pair went to (-1 dropped)
  CtxDev* ctx;
  SymmInfo symm;
  int wait_recv;                 // the last CTA also waits for all sources' flags
  int parts;                     // warps per row: 1, 2, 4 or 8
};

__global__ void __launch_bounds__(kEpThreads) ep_dispatch_kernel(const DispatchParams p) {
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  const int par = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int warps = kEpThreads / 32;
  const int lane = threadIdx.x & 31;
  const int row_bytes = p.quant ? p.H : p.H * 2;
  const int nsc = p.H / kQuantBlock;
  uint8_t* rx = p.recv_x + par * p.rows_per_parity * row_bytes;
  float* rs = p.recv_scale + par * p.rows_per_parity * nsc;
  int32_t* rm = p.recv_meta + par * p.rows_per_parity;
  const int64_t pairs = static_cast<int64_t>(p.T) * p.k;
  // `parts` warps share a row (a row is a chain of dependent memory round trips: with few rows more warps per row cut
  // the latency).  The slot of a row comes from one atomic on the LOCAL cursor of its expert, taken by the row's first
  // warp and handed to the others through shared memory.
  __shared__ int64_t s_row[kEpThreads / 32];
  const int parts = p.parts, rpc = warps / parts;
  const int grp = (threadIdx.x >> 5) / parts, part = (threadIdx.x >> 5) % parts;
  const int nblk = p.H / kQuantBlock;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rpc; base < pairs; base += static_cast<int64_t>(gridDim.x) * rpc) {
    const int64_t pr = base + grp;
    int e = -1;
    if (pr < pairs) {
      e = p.topk_ids[pr];
      if (e < 0 || e >= p.E) e = -1;
    }
    if (part == 0 && lane == 0 && pr < pairs) {
      int64_t row = -1;
      if (e >= 0) {
        const int dst = e / p.epr, le = e - dst * p.epr;
        const int idx = atomicAdd(p.cursor + e, 1);
        const int64_t b = p.base ? p.base[(static_cast<int64_t>(dst) * p.epr + le) * W + rank]
                                 : (static_cast<int64_t>(le) * W + rank) * p.max_tokens;
        row = b + idx;
      }
      p.sent_row[pr] = static_cast<int32_t>(row);
      s_row[grp] = row;
    }
    __syncthreads();
    if (e >= 0) {
      const int dst = e / p.epr;
      const int64_t row = s_row[grp];
      const __nv_bfloat16* src = p.x + (pr / p.k) * p.H;
      uint8_t* drow = symm_at(p.symm, rx + row * row_bytes, dst);
      if (p.quant) {
        warp_quant_row(src, drow, symm_at(p.symm, rs + row * nsc, dst), p.H, part * nblk / parts, (part + 1) * nblk / parts);
      } else {
        const int nv = p.H >> 3;
        for (int i = part * nv / parts + lane; i < (part + 1) * nv / parts; i += 32) st_v4(drow + i * 16, ld_nc_v4(src + i * 8));
      }
      if (part == 0 && lane == 0) *symm_at(p.symm, rm + row, dst) = static_cast<int32_t>(pr);
    }
    __syncthreads();   // s_row is rewritten by the next iteration
  }
  // ---- completion: the last CTA of the grid publishes counts and flags
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&p.ctx->grid_bar, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    int32_t* rc = p.recv_count + par * p.epr * W;
    for (int i = threadIdx.x; i < p.E; i += kEpThreads) {
      const int dst = i / p.epr, le = i - dst * p.epr;
      *symm_at(p.symm, rc + le * W + rank, dst) = p.cursor[i];
      p.cursor[i] = 0;   // ready for the next call
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x < W) {
      fence_acq_rel_sys();
      st_release_sys(symm_at(p.symm, p.flags + rank, (rank + threadIdx.x) % W), epoch);
      if (p.wait_recv) ok = wait_until(p.symm, p.flags + threadIdx.x, epoch, kCmpGe, kKernelEpDispatch, 1, threadIdx.x, 0);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      p.ctx->grid_bar = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
    }
  }
}

// For every receive row of the previous dispatch (its parity): expert id of the row (local expert index) or `epr`
// (= "no token") so that the generic sort kernel can build the grouped-GEMM layout.
// Parity of the receive buffers the last finished dispatch of `dctx` wrote (it has already advanced the epoch).
TDB_DEVICE int last_parity(const CtxDev* dctx) { return static_cast<int>((ld_volatile(&dctx->epoch) + 1u) & 1u); }

__global__ void ep_recv_ids_kernel(const int32_t* __restrict__ recv_count_base, const int32_t* __restrict__ base_self,
                                   int32_t* __restrict__ row_expert, int epr, int W, int max_tokens, int64_t rows,
                                   const CtxDev* dctx) {
  const int32_t* recv_count = recv_count_base + last_parity(dctx) * epr * W;
  // fixed stride: row = (le * W + src) * max_tokens + i ; packed: rows of (le, src) start at base_self[le * W + src]
  for (int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; r < rows;
       r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int ex = epr;
    if (base_self == nullptr) {
      const int64_t blk = r / max_tokens;
      const int i = static_cast<int>(r - blk * max_tokens);
      if (blk < static_cast<int64_t>(epr) * W && i < recv_count[blk]) ex = static_cast<int>(blk / W);
    } else {
      // binary search over the (le, src) blocks
      int lo = 0, hi = epr * W - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (base_self[mid] <= r) lo = mid; else hi = mid - 1;
      }
      if (r - base_self[lo] < recv_count[lo]) ex = lo / W;
    }
    row_expert[r] = ex;
  }
}

// Exclusive offsets of the packed layout: base[d][le][s] = sum of counts[s'][d*epr+le'] over (le', s') before (le, s).
// counts_all [W src][E] (all-gathered).  One CTA per destination rank.
__global__ void ep_layout_kernel(const int32_t* __restrict__ counts_all, int32_t* __restrict__ base, int epr, int W, int E) {
  const int d = blockIdx.x;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int le = 0; le < epr; ++le) {
      for (int s = 0; s < W; ++s) {
        base[(static_cast<int64_t>(d) * epr + le) * W + s] = acc;
        acc += counts_all[static_cast<int64_t>(s) * E + d * epr + le];
      }
    }
  }
}

// counts[e] per expert of the local routing (for the throughput layout exchange)
__global__ void ep_count_kernel(const int32_t* __restrict__ ids, int64_t n, int E, int32_t* counts) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(counts + e, 1);
  }
}

// Gather receive rows into the expert-sorted layout, de-quantising fp8 rows on the way.
__global__ void ep_gather_rows_kernel(const uint8_t* __restrict__ recv_x_base, const float* __restrict__ recv_scale_base,
                                      const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ meta,
                                      __nv_bfloat16* __restrict__ out, int H, int quant, int64_t rows_per_parity,
                                      const CtxDev* dctx) {
  const int par = last_parity(dctx);
  const uint8_t* recv_x = recv_x_base + par * rows_per_parity * (quant ? H : 2 * H);
  const float* recv_scale = recv_scale_base + par * rows_per_parity * (H / kQuantBlock);
  // the grid is sized for the machine, not for the row capacity: most of the capacity is unused in a decode step
  const int64_t total = meta[0];
  for (int64_t r = blockIdx.x; r < total; r += gridDim.x) {
    const int id = sorted_ids[r];
    __nv_bfloat16* dst = out + r * H;
    if (id < 0) {
      for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
      continue;
    }
    if (!quant) {
      const uint4* s = reinterpret_cast<const uint4*>(recv_x + static_cast<int64_t>(id) * H * 2);
      for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = s[i];
      continue;
    }
    const uint8_t* q = recv_x + static_cast<int64_t>(id) * H;
    const float* sc = recv_scale + static_cast<int64_t>(id) * (H / kQuantBlock);
    for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
      const uint32_t w = reinterpret_cast<const uint32_t*>(q)[i];
      const float s = sc[(i * 4) / kQuantBlock];
      uint2 o;
      o.x = pack_bf16x2(fp8_to_float(w & 0xff) * s, fp8_to_float((w >> 8) & 0xff) * s);
      o.y = pack_bf16x2(fp8_to_float((w >> 16) & 0xff) * s, fp8_to_float(w >> 24) * s);
      reinterpret_cast<uint2*>(dst)[i] = o;
    }
  }
}

// ---------------------------------------------------------------------------
// Receive side in one launch: from the per-(local expert, source) counts alone, lay the received rows out for the
// grouped GEMM (rows sorted by local expert, every expert padded to 128 rows), de-quantising fp8 rows on the way.
// The receive areas are already grouped by (expert, source), so the place of every row follows from a prefix sum over
// at most epr * W counts that every CTA recomputes in shared memory; nothing scans the receive capacity.
// One warp moves one row.  Block 0 also writes the layout tensors (sorted_ids are receive-row indices, -1 = padding;
// padding rows of x_sorted are left as they are).
// ---------------------------------------------------------------------------
constexpr int kFinishMaxBlocks = 2048;    // epr * W
constexpr int kFinishMaxExperts = 256;    // epr

struct FinishParams {
  const uint8_t* recv_x;
  const float* recv_scale;
  const int32_t* recv_count;
  const int32_t* base_self;    // packed layout: first receive row of every (expert, source) block; null = fixed stride
  int epr, W, max_tokens, H, quant;
  int64_t rows_per_parity;
  const CtxDev* dctx;
  __nv_bfloat16* x_sorted;     // [cap, H]
  int32_t* sorted_ids;         // [cap]
  int32_t* tile_expert;        // [cap / 128]
  int32_t* offsets;            // [epr + 1]
  int32_t* counts;             // [epr]
  int32_t* meta;               // {padded rows, tiles}
  int32_t* real_rows;          // [cap + 1]: the sorted rows that carry a token, packed, and their number in the last slot
  int64_t cap;                 // multiple of 128
  int parts;                   // warps per token row
};

__global__ void __launch_bounds__(kEpThreads) ep_finish_kernel(const FinishParams p) {
  __shared__ int s_real[kFinishMaxExperts];      // tokens of the experts before this one
  __shared__ int s_cnt[kFinishMaxBlocks];        // tokens of (le, src)
  __shared__ int s_in[kFinishMaxBlocks];         // rows of the same expert from earlier sources
  __shared__ int s_tot[kFinishMaxExperts];       // tokens of the expert
  __shared__ int s_off[kFinishMaxExperts + 1];   // padded first row of the expert
  const int par = last_parity(p.dctx);
  const int epr = p.epr, W = p.W, nblk = epr * W;
  const int32_t* rc = p.recv_count + par * nblk;
  for (int i = threadIdx.x; i < nblk; i += kEpThreads) {
    int c = rc[i];
    s_cnt[i] = c < 0 ? 0 : c;
  }
  __syncthreads();
  for (int le = threadIdx.x; le < epr; le += kEpThreads) {
    int acc = 0;
    for (int sr = 0; sr < W; ++sr) {
      s_in[le * W + sr] = acc;
      acc += s_cnt[le * W + sr];
    }
    s_tot[le] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t acc = 0;
    int real = 0;
    for (int le = 0; le < epr; ++le) {
      s_off[le] = static_cast<int>(acc);
      int64_t nxt = acc + (static_cast<int64_t>(s_tot[le]) + 127) / 128 * 128;
      if (nxt > p.cap) {          // cannot happen with a capacity of min(receive rows, W * tokens * k) + epr * 127 rows;
        s_tot[le] = 0;            // an expert that would not fit is dropped rather than written out of bounds
        nxt = acc;
      }
      s_real[le] = real;
      real += s_tot[le];
      acc = nxt;
    }
    s_off[epr] = static_cast<int>(acc);
    if (blockIdx.x == 0) p.real_rows[p.cap] = real;
  }
  __syncthreads();
  const int R = s_off[epr];
  if (blockIdx.x == 0) {
    for (int le = threadIdx.x; le < epr; le += kEpThreads) {
      p.offsets[le] = s_off[le];
      p.counts[le] = s_tot[le];
    }
    if (threadIdx.x == 0) {
      p.offsets[epr] = R;
      p.meta[0] = R;
      p.meta[1] = R / 128;
    }
    const int max_tiles = static_cast<int>(p.cap / 128);
    for (int t = threadIdx.x; t < max_tiles; t += kEpThreads) {
      int ex = -1;
      if (t * 128 < R) {
        int lo = 0, hi = epr - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (s_off[mid] <= t * 128) lo = mid; else hi = mid - 1;
        }
        ex = lo;
      }
      p.tile_expert[t] = ex;
    }
  }
  const int row_bytes = p.quant ? p.H : 2 * p.H;
  const int nsc = p.H / kQuantBlock;
  const uint8_t* recv_x = p.recv_x + par * p.rows_per_parity * row_bytes;
  const float* recv_scale = p.recv_scale + par * p.rows_per_parity * nsc;
  const int warps = kEpThreads / 32, lane = threadIdx.x & 31;
  // padding rows of partly filled tiles: marked, not cleared.  A GEMM row depends on its own input row only and nothing
  // reads the output rows of padding, so clearing up to 127 rows per expert would be wasted traffic (with many
  // experts per rank far more bytes than the tokens themselves).
  for (int r = blockIdx.x * kEpThreads + threadIdx.x; r < R; r += gridDim.x * kEpThreads) {
    int lo = 0, hi = epr - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_off[mid] <= r) lo = mid; else hi = mid - 1;
    }
    if (r - s_off[lo] >= s_tot[lo]) p.sorted_ids[r] = -1;
  }
  // token rows: the j-th token row overall (experts in order, sources in order inside an expert) is handled by `parts`
  // warps; indexing by token row rather than by sorted row spreads the rows evenly over the warps (the token rows of an
  // expert are adjacent and 128-row aligned, a stride over sorted rows would give a few warps all of them)
  const int n_real = s_real[epr - 1] + s_tot[epr - 1];
  const int parts = p.parts;
  for (int wj = blockIdx.x * warps + (threadIdx.x >> 5); wj < n_real * parts; wj += gridDim.x * warps) {
    const int j = wj / parts, part = wj - j * parts;
    int lo = 0, hi = epr - 1;
    while (lo < hi) {      // last expert whose first token row is <= j: the one that owns row j (empty ones share starts)
      const int mid = (lo + hi + 1) >> 1;
      if (s_real[mid] <= j) lo = mid; else hi = mid - 1;
    }
    const int le = lo;
    const int jr = j - s_real[le];
    const int r = s_off[le] + jr;
    int sr = 0;
    while (sr + 1 < W && s_in[le * W + sr + 1] <= jr) ++sr;
    const int i_in = jr - s_in[le * W + sr];
    const int64_t id = p.base_self ? static_cast<int64_t>(p.base_self[le * W + sr]) + i_in
                                   : (static_cast<int64_t>(le) * W + sr) * p.max_tokens + i_in;
    uint4* dst = reinterpret_cast<uint4*>(p.x_sorted + static_cast<int64_t>(r) * p.H);
    if (part == 0 && lane == 0) {
      p.sorted_ids[r] = static_cast<int32_t>(id);
      p.real_rows[j] = r;
    }
    if (!p.quant) {
      const uint4* src = reinterpret_cast<const uint4*>(recv_x + id * row_bytes);
      const int nv = p.H >> 3;
      const int i1 = (part + 1) * nv / parts;
      int i = part * nv / parts + lane;
      for (; i + 96 < i1; i += 128) {
        const uint4 v0 = src[i], v1 = src[i + 32], v2 = src[i + 64], v3 = src[i + 96];
        dst[i] = v0; dst[i + 32] = v1; dst[i + 64] = v2; dst[i + 96] = v3;
      }
      for (; i < i1; i += 32) dst[i] = src[i];
      continue;
    }
    // fp8 row: a lane turns 16 values (one 16-byte load, inside one 128-value scale block) into two 16-byte stores
    const uint4* q = reinterpret_cast<const uint4*>(recv_x + id * row_bytes);
    const float* sc = recv_scale + id * nsc;
    const int nch = p.H >> 4;
    const int c1 = (part + 1) * nch / parts;
    for (int i0 = part * nch / parts; i0 < c1; i0 += 128) {
      uint4 w[4];
      float scl[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 32 + lane;
        const bool in = i < c1;
        w[u] = in ? q[i] : make_uint4(0u, 0u, 0u, 0u);
        scl[u] = in ? sc[i >> 3] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 32 + lane;
        if (i >= c1) break;
        const uint32_t ws[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
        uint32_t o[8];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          o[2 * c] = pack_bf16x2(fp8_to_float(ws[c] & 0xff) * scl[u], fp8_to_float((ws[c] >> 8) & 0xff) * scl[u]);
          o[2 * c + 1] = pack_bf16x2(fp8_to_float((ws[c] >> 16) & 0xff) * scl[u], fp8_to_float(ws[c] >> 24) * scl[u]);
        }
        dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Combine: y_sorted rows (expert outputs, bf16) go back to the source rank of their token, into ret[pair]; when all
// expert ranks have flagged, every CTA reduces its share of the local tokens: out[t] = sum_j w[t,j] * ret[t*k+j].
// ---------------------------------------------------------------------------
struct CombineParams {
  const __nv_bfloat16* y;        // [rows_sorted, H] expert outputs in the sorted layout
  const int32_t* pos_of;         // [recv rows] sorted row of every receive row (-1: no token); unused with sorted_ids
  const int32_t* sorted_ids;     // optional [sorted rows] receive row of every sorted row (-1: padding): the send loop
  const int32_t* sort_meta;      //   then walks the sort_meta[0] sorted rows instead of the whole receive capacity
  const int32_t* real_rows;      // optional (with sorted_ids) [cap + 1]: packed list of the sorted rows that carry a token,
  int64_t real_cap;              //   count in slot [real_cap]: `parts` warps per listed row, no scan at all
  int parts;
  const int32_t* recv_meta;      // [2][recv rows] pair index at the source (parity of the matching dispatch)
  const CtxDev* dctx;            // the dispatch context (gives that parity)
  const int32_t* base_self;      // packed layout: [epr*W] first row of block; null = fixed stride
  int epr, max_tokens;
  int64_t recv_rows;
  __nv_bfloat16* ret;            // heap [2][max_tokens*k][H]
  uint64_t ret_half;             // elements per parity
  uint32_t* flags;               // heap [W]
  // local reduction
  const int32_t* topk_ids;       // [T, k]
  const float* topk_w;           // [T, k] or null
  __nv_bfloat16* out;            // [T, H]
  int T, H, k, E;
  CtxDev* ctx;
  SymmInfo symm;
};

__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(const CombineParams p) {
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  const int par = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int warps = kEpThreads / 32, lane = threadIdx.x & 31;
  __nv_bfloat16* ret = p.ret + par * p.ret_half;
  const int32_t* recv_meta = p.recv_meta + last_parity(p.dctx) * p.recv_rows;
  // ---- send.  Receive rows that carry a token are sparse and clustered (the first few slots of every
  // (expert, source) block), so a fixed row-to-warp mapping leaves most warps idle.  Warps instead pull chunks of 32
  // consecutive rows from a shared counter, look at the 32 `pos_of` entries with one coalesced load, and copy the
  // rows that are there one after the other with several 16-byte loads in flight.
  const int blocks = p.epr * W;
  uint32_t* work = &p.ctx->pad[0];
  const int nvec = p.H >> 3;
  // copy of one expert-output row to its token's owner, several 16-byte loads in flight
  auto send_row = [&](int pos, int pair, int64_t r, int part, int parts) {
    int src;
    if (p.base_self == nullptr) {
      src = static_cast<int>((r / p.max_tokens) % W);
    } else {
      int lo = 0, hi = blocks - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (p.base_self[mid] <= r) lo = mid; else hi = mid - 1;
      }
      src = lo % W;
    }
    const uint4* sp = reinterpret_cast<const uint4*>(p.y + static_cast<int64_t>(pos) * p.H);
    uint4* d = reinterpret_cast<uint4*>(symm_at(p.symm, ret + static_cast<int64_t>(pair) * p.H, src));
    const int i1 = (part + 1) * nvec / parts;
    int i = part * nvec / parts + lane;
    for (; i + 96 < i1; i += 128) {
      const uint4 v0 = sp[i], v1 = sp[i + 32], v2 = sp[i + 64], v3 = sp[i + 96];
      st_v4(d + i, v0);
      st_v4(d + i + 32, v1);
      st_v4(d + i + 64, v2);
      st_v4(d + i + 96, v3);
    }
    for (; i < i1; i += 32) st_v4(d + i, sp[i]);
  };
  if (p.real_rows != nullptr) {
    // the receive side listed the rows that carry a token: one warp per row, rows spread evenly over all warps (the
    // rows of an expert are adjacent, so chunked scanning would leave the few warps that hit them with all the work)
    const int n_real = p.real_rows[p.real_cap];
    const int parts = p.parts;
    for (int wj = blockIdx.x * warps + (threadIdx.x >> 5); wj < n_real * parts; wj += gridDim.x * warps) {
      const int j = wj / parts;
      const int pos = p.real_rows[j];
      const int64_t r = p.sorted_ids[pos];
      if (r >= 0) send_row(pos, recv_meta[r], r, wj - j * parts, parts);
    }
  } else {
  while (true) {
    uint32_t chunk = 0;
    if (lane == 0) chunk = atomicAdd(work, 1u);
    chunk = __shfl_sync(0xffffffffu, chunk, 0);
    const int64_t r_base = static_cast<int64_t>(chunk) * 32;
    const int64_t domain = p.sorted_ids ? static_cast<int64_t>(p.sort_meta[0]) : p.recv_rows;
    if (r_base >= domain) break;
    const int64_t r_mine = r_base + lane;
    int pos_mine = -1;
    int64_t id_mine = r_mine;      // receive row
    if (p.sorted_ids) {
      id_mine = r_mine < domain ? p.sorted_ids[r_mine] : -1;
      pos_mine = id_mine >= 0 ? static_cast<int>(r_mine) : -1;
    } else if (r_mine < domain) {
      pos_mine = p.pos_of[r_mine];
    }
    const int pair_mine = pos_mine >= 0 ? recv_meta[id_mine] : 0;
    uint32_t valid = __ballot_sync(0xffffffffu, pos_mine >= 0);
    while (valid) {
      const int l = __ffs(valid) - 1;
      valid &= valid - 1;
      const int pos = __shfl_sync(0xffffffffu, pos_mine, l);
      const int pair = __shfl_sync(0xffffffffu, pair_mine, l);
      const int64_t r = __shfl_sync(0xffffffffu, id_mine, l);
      send_row(pos, pair, r, 0, 1);
    }
  }
  }
  __shared__ int s_last;
  __shared__ int s_ok;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&p.ctx->grid_bar, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    s_ok = 1;
  }
  __syncthreads();
  if (s_last && threadIdx.x < W) {
    __threadfence();
    fence_acq_rel_sys();
    st_release_sys(symm_at(p.symm, p.flags + rank, (rank + threadIdx.x) % W), epoch);
  }
  // ---- wait for every expert rank, then reduce
  if (threadIdx.x < W) {
    if (!wait_until(p.symm, p.flags + threadIdx.x, epoch, kCmpGe, kKernelEpCombine, 1, threadIdx.x, 0)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    // weighted sum of the k returned rows of every token: the (up to eight) row loads of a step are issued together
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
      for (int j0 = 0; j0 < p.k; j0 += 8) {
        float wj[8];
        bool okj[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int jj = j0 + j;
          const int e = jj < p.k ? p.topk_ids[t * p.k + jj] : -1;
          okj[j] = e >= 0 && e < p.E;
          wj[j] = okj[j] ? (p.topk_w ? p.topk_w[t * p.k + jj] : 1.f) : 0.f;
        }
        for (int i = threadIdx.x; i < (p.H >> 3); i += kEpThreads) {
          uint4 u[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            u[j] = okj[j] ? ld_relaxed_sys_v4(ret + (static_cast<int64_t>(t) * p.k + j0 + j) * p.H + i * 8)
                          : make_uint4(0u, 0u, 0u, 0u);
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          uint4* optr = reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(t) * p.H) + i;
          if (j0 > 0) {
            const uint4 prev = *optr;   // more than eight slots: continue from the partial sum of the earlier ones
            const float2 f0 = unpack_bf16x2(prev.x), f1 = unpack_bf16x2(prev.y), f2 = unpack_bf16x2(prev.z), f3 = unpack_bf16x2(prev.w);
            acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 f0 = unpack_bf16x2(u[j].x), f1 = unpack_bf16x2(u[j].y), f2 = unpack_bf16x2(u[j].z), f3 = unpack_bf16x2(u[j].w);
            acc[0] += wj[j] * f0.x; acc[1] += wj[j] * f0.y; acc[2] += wj[j] * f1.x; acc[3] += wj[j] * f1.y;
            acc[4] += wj[j] * f2.x; acc[5] += wj[j] * f2.y; acc[6] += wj[j] * f3.x; acc[7] += wj[j] * f3.y;
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
          *optr = o;
        }
      }
    }
  }
  // ---- last CTA out advances the epoch (second counter: `done`)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(&p.ctx->done, 1u);
    if (prev == gridDim.x - 1) {
      p.ctx->done = 0;
      p.ctx->grid_bar = 0;
      p.ctx->pad[0] = 0;   // work counter of the send phase
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
    }
  }
}

// ---------------------------------------------------------------------------
// all_to_all_single with uneven splits: rows [in_off[d], in_off[d+1]) of `in` go to rank d, which stores the rows of
// source s at out_off[d][s] = sum of splits[s'][d] for s' < s.  splits_all [W src][W dst] all-gathered beforehand.
// out lives in the heap; the kernel returns when all sources' rows have arrived.
// ---------------------------------------------------------------------------
struct A2AParams {
  const char* in;
  char* out;                    // heap
  const int32_t* splits_all;    // [W][W]
  int64_t row_bytes;
  uint32_t* flags;              // heap [W]
  CtxDev* ctx;
  SymmInfo symm;
};

__global__ void __launch_bounds__(kEpThreads) a2a_single_kernel(const A2AParams p) {
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  const int W = p.symm.world, rank = p.symm.rank;
  // CTA b serves destination b % W, part b / W of gridDim.x / W parts
  const int parts = gridDim.x / W;
  const int dst = blockIdx.x % W, part = blockIdx.x / W;
  if (part < parts) {
    int64_t in_row = 0;
    for (int d = 0; d < dst; ++d) in_row += p.splits_all[rank * W + d];
    int64_t out_row = 0;
    for (int s = 0; s < rank; ++s) out_row += p.splits_all[s * W + dst];
    const int64_t bytes = static_cast<int64_t>(p.splits_all[rank * W + dst]) * p.row_bytes;
    const int64_t per = ((bytes / 16 + parts - 1) / parts) * 16;
    const int64_t lo = min(bytes, per * part), hi = min(bytes, lo + per);
    const char* s = p.in + in_row * p.row_bytes;
    char* d = symm_at(p.symm, p.out + out_row * p.row_bytes, dst);
    for (int64_t i = lo + threadIdx.x * 16; i < hi; i += static_cast<int64_t>(kEpThreads) * 16) st_v4(d + i, ld_nc_v4(s + i));
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&p.ctx->grid_bar, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < W) {
      __threadfence();
      fence_acq_rel_sys();
      st_release_sys(symm_at(p.symm, p.flags + rank, (rank + threadIdx.x) % W), epoch);
      wait_until(p.symm, p.flags + threadIdx.x, epoch, kCmpGe, kKernelA2A, 1, threadIdx.x, 0);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      p.ctx->grid_bar = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
    }
  }
}

// ---------------------------------------------------------------------------
// Head-to-sequence exchange of Ulysses sequence parallelism: `in` holds all S = W * s_local positions restricted to this
// rank's head block ([S][row_bytes], pitch in_pitch).  The rows [d * s_local, (d + 1) * s_local) go to rank d, which
// assembles [s_local][W * row_bytes]: source rank r fills the column block [r * row_bytes, (r + 1) * row_bytes) of every
// row.  out: heap [s_local][W * row_bytes], ONE buffer (the result is at a fixed address, so a CUDA graph that
// captured a consumer of it stays valid).  A rank may only write into a peer's buffer when that peer has finished
// reading the previous result, i.e. when it has entered this call: CTA 0 of every rank announces its entry first
// thing, and every CTA waits for the announcement of its destination before it stores (a wait on a remote CTA 0,
// which is always scheduled).  The kernel returns when the blocks of all sources have arrived.
// flags: heap [2][W] = entry announcements, arrival flags; both carry the call epoch kept on the device.
// Reference: kernels/nvidia/sp_ulysess_o_all2all_gemm.py:299-392 (per-tile push of the attention output).
// ---------------------------------------------------------------------------
struct A2AColsParams {
  const char* in;
  char* out;                   // heap [s_local][W * row_bytes]
  int64_t in_pitch, row_bytes;
  int s_local;
  uint32_t* flags;             // heap [2][W]
  CtxDev* ctx;
  SymmInfo symm;
};

__global__ void __launch_bounds__(kEpThreads) a2a_cols_kernel(const A2AColsParams p) {
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  const int W = p.symm.world, rank = p.symm.rank;
  const int parts = gridDim.x / W;
  const int dst = blockIdx.x % W, part = blockIdx.x / W;
  __shared__ int s_go;
  if (blockIdx.x == 0 && threadIdx.x < W)
    st_release_sys(symm_at(p.symm, p.flags + rank, (rank + threadIdx.x) % W), epoch);
  if (threadIdx.x == 0)
    s_go = wait_until(p.symm, p.flags + dst, epoch, kCmpGe, kKernelA2A, 3, dst, 0) ? 1 : 0;
  __syncthreads();
  if (part < parts && s_go) {
    const int64_t out_pitch = static_cast<int64_t>(W) * p.row_bytes;
    char* obase = symm_at(p.symm, p.out, dst) + rank * p.row_bytes;
    const char* ibase = p.in + static_cast<int64_t>(dst) * p.s_local * p.in_pitch;
    const int nvec = static_cast<int>(p.row_bytes >> 4);
    const int warps = kEpThreads / 32, lane = threadIdx.x & 31;
    for (int r = part * warps + (threadIdx.x >> 5); r < p.s_local; r += parts * warps) {
      const char* s = ibase + r * p.in_pitch;
      char* d = obase + r * out_pitch;
      int i = lane;
      for (; i + 96 < nvec; i += 128) {
        const uint4 v0 = ld_nc_v4(s + (i << 4)), v1 = ld_nc_v4(s + ((i + 32) << 4)), v2 = ld_nc_v4(s + ((i + 64) << 4)),
                    v3 = ld_nc_v4(s + ((i + 96) << 4));
        st_v4(d + (i << 4), v0);
        st_v4(d + ((i + 32) << 4), v1);
        st_v4(d + ((i + 64) << 4), v2);
        st_v4(d + ((i + 96) << 4), v3);
      }
      for (; i < nvec; i += 32) st_v4(d + (i << 4), ld_nc_v4(s + (i << 4)));
    }
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&p.ctx->grid_bar, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < W) {
      __threadfence();
      fence_acq_rel_sys();
      st_release_sys(symm_at(p.symm, p.flags + W + rank, (rank + threadIdx.x) % W), epoch);
      wait_until(p.symm, p.flags + W + threadIdx.x, epoch, kCmpGe, kKernelA2A, 2, threadIdx.x, 0);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      p.ctx->grid_bar = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
    }
  }
}

// ---- stand-alone quantisation ---------------------------------------------------------------------------------
__global__ void fp8_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ s, int64_t T,
                                 int H) {
  const int warps = blockDim.x >> 5;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5); t < T;
       t += static_cast<int64_t>(gridDim.x) * warps)
    warp_quant_row(x + t * H, q + t * H, s + t * (H / kQuantBlock), H);
}
__global__ void fp8_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ s, __nv_bfloat16* __restrict__ out,
                                   int64_t T, int H) {
  const int64_t n4 = T * H / 4;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(q)[i];
    const int64_t el = i * 4;
    const float sc = s[(el / H) * (H / kQuantBlock) + (el % H) / kQuantBlock];
    uint2 o;
    o.x = pack_bf16x2(fp8_to_float(w & 0xff) * sc, fp8_to_float((w >> 8) & 0xff) * sc);
    o.y = pack_bf16x2(fp8_to_float((w >> 16) & 0xff) * sc, fp8_to_float(w >> 24) * sc);
    reinterpret_cast<uint2*>(out)[i] = o;
  }
}

SymmInfo to_dev(const SymmInfoHost& h) {
  SymmInfo s;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&s, &h, sizeof(s));
  return s;
}

int grid_1d(int64_t n, int threads, int cap) {
  int64_t g = (n + threads - 1) / threads;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

cudaError_t launch_ep_dispatch(const EpDispatchArgs& a, cudaStream_t s) {
  if (a.H % kQuantBlock != 0 || a.E % a.symm.world != 0) return cudaErrorInvalidValue;
  DispatchParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  p.topk_ids = a.topk_ids;
  p.T = a.T; p.H = a.H; p.k = a.k; p.E = a.E;
  p.epr = a.E / a.symm.world;
  p.quant = a.quant;
  p.max_tokens = a.max_tokens;
  p.recv_x = reinterpret_cast<uint8_t*>(a.recv_x);
  p.recv_scale = a.recv_scale;
  p.recv_meta = a.recv_meta;
  p.recv_count = a.recv_count;
  p.flags = a.flags;
  p.rows_per_parity = a.rows_per_parity;
  p.base = a.base;
  p.cursor = a.cursor;
  p.sent_row = a.sent_row;
  p.ctx = a.ctx;
  p.symm = to_dev(a.symm);
  p.wait_recv = 1;
  p.parts = (a.parts == 2 || a.parts == 4 || a.parts == 8) ? a.parts : 1;
  const int ctas = a.num_ctas > 0 ? a.num_ctas : 64;
  ep_dispatch_kernel<<<ctas, kEpThreads, 0, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_ep_count(const int32_t* ids, int64_t n, int E, int32_t* counts, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, s);
  if (e != cudaSuccess) return e;
  if (n > 0) ep_count_kernel<<<grid_1d(n, 256, 296), 256, 0, s>>>(ids, n, E, counts);
  return cudaGetLastError();
}

cudaError_t launch_ep_layout(const int32_t* counts_all, int32_t* base, int epr, int W, int E, cudaStream_t s) {
  ep_layout_kernel<<<W, 32, 0, s>>>(counts_all, base, epr, W, E);
  return cudaGetLastError();
}

cudaError_t launch_ep_recv_ids(const int32_t* recv_count, const int32_t* base_self, int32_t* row_expert, int epr, int W,
                               int max_tokens, int64_t rows, const CtxDev* dispatch_ctx, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  ep_recv_ids_kernel<<<grid_1d(rows, 256, 592), 256, 0, s>>>(recv_count, base_self, row_expert, epr, W, max_tokens, rows,
                                                             dispatch_ctx);
  return cudaGetLastError();
}

cudaError_t launch_ep_gather_rows(const void* recv_x, const float* recv_scale, const int32_t* sorted_ids, const int32_t* meta,
                                  void* out, int64_t rows_cap, int H, int quant, int64_t rows_per_parity,
                                  const CtxDev* dispatch_ctx, cudaStream_t s) {
  if (rows_cap == 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>(rows_cap < 148 * 16 ? rows_cap : 148 * 16);
  ep_gather_rows_kernel<<<grid, 128, 0, s>>>(reinterpret_cast<const uint8_t*>(recv_x), recv_scale,
                                                                       sorted_ids, meta, reinterpret_cast<__nv_bfloat16*>(out),
                                                                       H, quant, rows_per_parity, dispatch_ctx);
  return cudaGetLastError();
}

cudaError_t launch_ep_finish(const EpFinishArgs& a, cudaStream_t s) {
  if (a.H % 128 != 0 || a.cap % 128 != 0 || a.epr < 1 || a.epr > kFinishMaxExperts || a.epr * a.W > kFinishMaxBlocks)
    return cudaErrorInvalidValue;
  FinishParams p;
  p.recv_x = reinterpret_cast<const uint8_t*>(a.recv_x);
  p.recv_scale = a.recv_scale;
  p.recv_count = a.recv_count;
  p.base_self = a.base_self;
  p.epr = a.epr; p.W = a.W; p.max_tokens = a.max_tokens; p.H = a.H; p.quant = a.quant;
  p.rows_per_parity = a.rows_per_parity;
  p.dctx = a.dispatch_ctx;
  p.x_sorted = reinterpret_cast<__nv_bfloat16*>(a.x_sorted);
  p.sorted_ids = a.sorted_ids;
  p.tile_expert = a.tile_expert;
  p.offsets = a.offsets;
  p.counts = a.counts;
  p.meta = a.meta;
  p.real_rows = a.real_rows;
  p.cap = a.cap;
  p.parts = (a.parts == 2 || a.parts == 4 || a.parts == 8) ? a.parts : 1;
  const int ctas = a.num_ctas > 0 ? a.num_ctas : 64;
  ep_finish_kernel<<<ctas, kEpThreads, 0, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_ep_combine(const EpCombineArgs& a, cudaStream_t s) {
  if (a.H % 8 != 0) return cudaErrorInvalidValue;
  if (a.sorted_ids == nullptr && a.pos_of == nullptr) return cudaErrorInvalidValue;
  if (a.sorted_ids != nullptr && a.sort_meta == nullptr) return cudaErrorInvalidValue;
  CombineParams p;
  p.y = reinterpret_cast<const __nv_bfloat16*>(a.y);
  p.pos_of = a.pos_of;
  p.sorted_ids = a.sorted_ids;
  p.sort_meta = a.sort_meta;
  p.real_rows = a.sorted_ids != nullptr ? a.real_rows : nullptr;
  p.real_cap = a.real_cap;
  p.parts = (a.parts == 2 || a.parts == 4 || a.parts == 8) ? a.parts : 1;
  p.recv_meta = a.recv_meta;
  p.dctx = a.dispatch_ctx;
  p.base_self = a.base_self;
  p.epr = a.E / a.symm.world;
  p.max_tokens = a.max_tokens;
  p.recv_rows = a.recv_rows;
  p.ret = reinterpret_cast<__nv_bfloat16*>(a.ret);
  p.ret_half = a.ret_half;
  p.flags = a.flags;
  p.topk_ids = a.topk_ids;
  p.topk_w = a.topk_w;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.T = a.T; p.H = a.H; p.k = a.k; p.E = a.E;
  p.ctx = a.ctx;
  p.symm = to_dev(a.symm);
  int ctas = a.num_ctas > 0 ? a.num_ctas : 64;
  // every CTA waits on remote flags that the last CTA of each rank raises: the whole grid must be resident at once,
  // so it is clamped to what the occupancy calculator says fits this device
  static int resident = 0;
  if (resident == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ep_combine_kernel, kEpThreads, 0) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    resident = sms * per_sm;
  }
  if (ctas > resident) ctas = resident;
  // cooperative: every CTA waits for flags that only the LAST CTA of each rank raises, so all CTAs of a rank must run
  return launch_coop(ep_combine_kernel, dim3(ctas), dim3(kEpThreads), static_cast<size_t>(0), s, p);
}

cudaError_t launch_a2a_single(const void* in, void* out, const int32_t* splits_all, int64_t row_bytes, uint32_t* flags,
                              CtxDev* ctx, const SymmInfoHost& symm, int parts, cudaStream_t s) {
  if (row_bytes % 16 != 0) return cudaErrorInvalidValue;
  A2AParams p;
  p.in = reinterpret_cast<const char*>(in);
  p.out = reinterpret_cast<char*>(out);
  p.splits_all = splits_all;
  p.row_bytes = row_bytes;
  p.flags = flags;
  p.ctx = ctx;
  p.symm = to_dev(symm);
  if (parts < 1) parts = 1;
  a2a_single_kernel<<<symm.world * parts, kEpThreads, 0, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_a2a_cols(const void* in, int64_t in_pitch, void* out, uint64_t out_bytes, int64_t row_bytes, int s_local,
                            uint32_t* flags, CtxDev* ctx, const SymmInfoHost& symm, int parts, cudaStream_t s) {
  if (row_bytes % 16 != 0 || in_pitch % 16 != 0 || s_local < 0) return cudaErrorInvalidValue;
  if (static_cast<uint64_t>(s_local) * symm.world * row_bytes > out_bytes) return cudaErrorInvalidValue;
  A2AColsParams p;
  p.in = reinterpret_cast<const char*>(in);
  p.out = reinterpret_cast<char*>(out);
  p.in_pitch = in_pitch;
  p.row_bytes = row_bytes;
  p.s_local = s_local;
  p.flags = flags;
  p.ctx = ctx;
  p.symm = to_dev(symm);
  if (parts < 1) parts = 1;
  a2a_cols_kernel<<<symm.world * parts, kEpThreads, 0, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_fp8_quant(const void* x, void* q, float* scales, int64_t T, int H, cudaStream_t s) {
  if (H % kQuantBlock != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  fp8_quant_kernel<<<grid_1d(T, 8, 592), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q),
                                                      scales, T, H);
  return cudaGetLastError();
}

cudaError_t launch_fp8_dequant(const void* q, const float* scales, void* out, int64_t T, int H, cudaStream_t s) {
  if (H % kQuantBlock != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  fp8_dequant_kernel<<<grid_1d(T * H / 4, 256, 1184), 256, 0, s>>>(reinterpret_cast<const uint8_t*>(q), scales,
                                                                  reinterpret_cast<__nv_bfloat16*>(out), T, H);
  return cudaGetLastError();
}

}  // namespace tdb
