// Fused tensor-parallel MoE kernels for sm_100a: one launch each for
//
//   all-gather -> grouped GEMM         y[pair, :] = x_gathered[token(pair), :] @ w1[expert(pair)]^T
//   grouped GEMM -> top-k reduce -> reduce-scatter / all-reduce
//                                      out[t, :] = sum over ranks, slots j of weight[t, j] * (h[pair(t, j), :] @ w2[e_j]^T)
//
// Both run the same persistent grouped tcgen05 GEMM over rows sorted by expert (128-row tiles, one expert per tile,
// the per-tile expert selects the weight slice through the third coordinate of the B tensor map).  What differs from a
// dense GEMM is the A operand: the rows of a tile are scattered over the token buffer, so four "gather" warps copy them
// with 16-byte cp.async into the 128-byte-swizzled stage (a padding row is zero-filled), fence the stage for the async
// proxy and arrive on its barrier; B comes by TMA; one thread issues tcgen05.mma; accumulators are double-buffered in
// TMEM; four epilogue warps write rows straight to global memory (one thread owns a row).
//
// all-gather mode: comm CTAs of the launch push the local token rows into every rank's workspace in 128-row chunks
// with one epoch flag per chunk (nearest consumer first).  A gather thread waits for the flag of exactly the chunk its
// row lives in, and tiles are visited in the order of moe_tile_schedule (by arrival stage), so the GEMM starts on the
// local tokens while the remote ones are still in flight.
//
// reduce mode: the epilogue multiplies every row by its routing weight; tiles are visited N-chunk by N-chunk and a
// counter per chunk tells the reducer CTAs of the same launch when a chunk of the sorted output is complete.  The
// reducers sum the k rows of every token, store the sum into the owner rank's slot over NVLink (reduce-scatter) or
// into every rank's slot (all-reduce), raise a flag per (chunk, source), wait for the other ranks' flags and add the
// W slots into the output - while the GEMM CTAs work on the next chunk.
//
// Reference behaviour being matched (not its code):
//   python/triton_dist/kernels/nvidia/allgather_group_gemm.py:535-608 (gathered A rows, wait per segment, tiles by
//   arrival), moe_reduce_rs.py:167-244, 404-487 (weight in the epilogue, N-chunk counters, reducer storing into the
//   peer's slot), moe_reduce_ar.py:274, 400-479.
// TMA loads read local memory only; every wait is bounded and reports through the status page.
#include <cuda.h>

#include "tdb/api.h"
#include "tdb/launch.cuh"
#include "tdb/moe.h"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kBN = 256;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;    // 16 KB
constexpr int kBBytes = kBN * kBK * 2;    // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kBarOffset = kStages * kStageBytes;
constexpr int kSmemTotal = kBarOffset + (2 * kStages + 4) * 8 + 16;
constexpr int kThreads = 320;             // warp 0 B producer, 1 MMA, 2-5 epilogue, 6-9 A gather

constexpr int kPushPiece = 32 * 1024;
constexpr int kPushSlots = 6;
constexpr int kPushAhead = 4;
static_assert(kPushSlots * kPushPiece + kPushSlots * 8 <= kSmemTotal, "push ring must fit the kernel's shared memory");

struct MoeParams {
  int mode;                    // MoeFusedMode
  int K, N;                    // reduction length, output columns of this rank
  int k_top;                   // slots per token
  const __nv_bfloat16* x;      // A source rows: [tokens or pairs, K]; all-gather mode: the local shard [t_local, K]
  int64_t ldx;
  int a_row_div;               // source row of sorted row r: sorted_ids[r] / a_row_div (k for token rows, 1 for pair rows)
  const int32_t* sorted_ids;   // [cap] flat pair index per sorted row, -1 = padding
  const int32_t* tile_expert;  // [cap / 128]
  const int32_t* order;        // tile visiting order or null (identity)
  const int32_t* meta;         // {padded rows, tiles}
  int max_tiles;
  __nv_bfloat16* y;            // output rows
  int64_t ldy;
  int scatter_out;             // 1: row r goes to y[sorted_ids[r]] ((token, slot) order), 0: y[r] (sorted layout)
  const float* row_weight;     // optional [pairs] routing weight applied in the epilogue
  int tiles_n;
  // all-gather
  int t_local;                 // tokens per rank
  int n_comm;
  __nv_bfloat16* ag_ws;        // heap [2][world * max_t_local][K]
  uint64_t ag_buf_elems;
  uint32_t* ag_flags;          // heap [2][world][max_chunks]
  int max_chunks;
  // reduce
  int n_chunks, tiles_n_chunk; // N chunks and n-tiles per chunk
  int n_red;                   // reducer CTAs
  int T;                       // tokens (all ranks)
  const int32_t* pos_of;       // [T * k] sorted row of every pair (-1: dropped)
  uint32_t* chunk_done;        // device [2][n_chunks] tile counters (epoch parity)
  __nv_bfloat16* red_slots;    // heap [2][world][rows][N]: reduce-scatter rows = T / world, all-reduce rows = T
  uint64_t red_slot_elems;
  uint32_t* red_flags;         // heap [2][world][n_chunks * n_red]
  __nv_bfloat16* out;          // [T / world, N] or [T, N]
  int64_t ld_out;
  CtxDev* ctx;
  SymmInfo symm;
  uint64_t mbar_timeout_ns;
};

TDB_DEVICE void cp_async_16(uint32_t smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 16 : 0;   // src-size 0: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(sz) : "memory");
}
TDB_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// One (deferred) arrival on an mbarrier that happens when all cp.async copies this thread has issued so far have
// landed; the thread does not wait.  The barrier's count must include the arrival (.noinc).
TDB_DEVICE void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int N>
TDB_DEVICE void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
TDB_DEVICE void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// ---------------------------------------------------------------------------
// All-gather push of a comm CTA (one thread drives a ring of bulk copies local -> shared -> peer workspace).
// ---------------------------------------------------------------------------
__device__ void ag_push(const MoeParams& p, uint32_t epoch, uint8_t* smem) {
  if (threadIdx.x != 0) return;
  const int buf = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int chunks = (p.t_local + kBM - 1) / kBM;
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * 2;
  char* ws_local = reinterpret_cast<char*>(p.ag_ws + buf * p.ag_buf_elems);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPushSlots * kPushPiece);
  for (int i = 0; i < kPushSlots; ++i) mbar_init(&bars[i], 1);
  fence_mbar_init();
  const int my_chunks = chunks > static_cast<int>(blockIdx.x) ? (chunks - blockIdx.x + p.n_comm - 1) / p.n_comm : 0;
  auto chunk_bytes = [&](int ordinal) -> uint64_t {
    const int c = blockIdx.x + ordinal * p.n_comm;
    return static_cast<uint64_t>(min(kBM, p.t_local - c * kBM)) * row_bytes;
  };
  uint64_t total_pieces = 0;
  for (int o = 0; o < my_chunks; ++o) total_pieces += (chunk_bytes(o) + kPushPiece - 1) / kPushPiece;
  total_pieces *= (W - 1);
  uint32_t ld_i = 0, st_i = 0;
  int ld_d = 1, ld_c = 0, st_d = 1, st_c = 0;
  uint64_t ld_off = 0, st_off = 0;
  constexpr int kPend = 4;
  uint32_t pend_group[kPend];
  int pend_peer[kPend], pend_chunk[kPend];
  int pend_n = 0;
  auto raise_flag = [&](int peer, int c) {
    fence_proxy_async();
    fence_acq_rel_sys();
    uint32_t* flag = p.ag_flags + (static_cast<uint64_t>(buf) * W + rank) * p.max_chunks + c;
    st_release_sys(symm_at(p.symm, flag, peer), epoch);
  };
  bool ok = true;
  for (uint64_t step = 0; step < total_pieces + kPushAhead && ok; ++step) {
    if (step < total_pieces) {
      const int slot = ld_i % kPushSlots;
      bulk_wait_read<kPushSlots - kPushAhead - 1>();
      const int c = blockIdx.x + ld_c * p.n_comm;
      const uint64_t cb = chunk_bytes(ld_c);
      const uint32_t bytes = static_cast<uint32_t>((cb - ld_off) < (uint64_t)kPushPiece ? (cb - ld_off) : (uint64_t)kPushPiece);
      const char* src = reinterpret_cast<const char*>(p.x) + static_cast<uint64_t>(c) * kBM * row_bytes + ld_off;
      mbar_arrive_expect_tx(&bars[slot], bytes);
      bulk_load(smem + slot * kPushPiece, src, bytes, &bars[slot]);
      ++ld_i;
      ld_off += bytes;
      if (ld_off >= cb) {
        ld_off = 0;
        if (++ld_c >= my_chunks) {
          ld_c = 0;
          ++ld_d;
        }
      }
    }
    if (step >= kPushAhead) {
      const int slot = st_i % kPushSlots;
      if (!mbar_wait(&bars[slot], (st_i / kPushSlots) & 1, nullptr, p.mbar_timeout_ns)) {
        report(p.symm, kTimeoutMbarrier, kKernelGroupGemm, 40, -1, slot, 0, static_cast<int>(st_i));
        ok = false;
        break;
      }
      const int c = blockIdx.x + st_c * p.n_comm;
      const uint64_t cb = chunk_bytes(st_c);
      const uint32_t bytes = static_cast<uint32_t>((cb - st_off) < (uint64_t)kPushPiece ? (cb - st_off) : (uint64_t)kPushPiece);
      const int peer = (rank - st_d + W) % W;
      char* dst_local = ws_local + (static_cast<uint64_t>(rank) * p.t_local + static_cast<uint64_t>(c) * kBM) * row_bytes + st_off;
      bulk_store(symm_at(p.symm, dst_local, peer), smem + slot * kPushPiece, bytes);
      bulk_commit();
      ++st_i;
      st_off += bytes;
      if (st_off >= cb) {
        if (pend_n == kPend) {
          bulk_wait<0>();
          for (int j = 0; j < pend_n; ++j) raise_flag(pend_peer[j], pend_chunk[j]);
          pend_n = 0;
        }
        pend_group[pend_n] = st_i - 1;
        pend_peer[pend_n] = peer;
        pend_chunk[pend_n] = c;
        ++pend_n;
        st_off = 0;
        if (++st_c >= my_chunks) {
          st_c = 0;
          ++st_d;
        }
      }
      if (pend_n > 0 && (st_i - 1) - pend_group[0] >= 2) {
        bulk_wait<2>();
        int keep = 0;
        for (int j = 0; j < pend_n; ++j) {
          if ((st_i - 1) - pend_group[j] >= 2) {
            raise_flag(pend_peer[j], pend_chunk[j]);
          } else {
            pend_group[keep] = pend_group[j];
            pend_peer[keep] = pend_peer[j];
            pend_chunk[keep] = pend_chunk[j];
            ++keep;
          }
        }
        pend_n = keep;
      }
    }
  }
  bulk_wait<0>();
  for (int j = 0; j < pend_n; ++j) raise_flag(pend_peer[j], pend_chunk[j]);
}

// ---------------------------------------------------------------------------
// Reducer CTA of the reduce mode.  Chunk by chunk: wait until the GEMM CTAs have finished the chunk's tiles, sum the
// k weighted rows of every token (this CTA's share of the tokens) and store the sum into the slot of this rank on the
// token's owner (reduce-scatter) or on every rank (all-reduce); raise this CTA's flag for the chunk on the
// destinations; wait for the same CTA index of every other rank; add the W slots of this CTA's output rows.
// ---------------------------------------------------------------------------
__device__ void moe_reducer(const MoeParams& p, uint32_t epoch) {
  const int buf = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const bool rs = p.mode == kMoeReduceRS;
  const int rows_out = rs ? p.T / W : p.T;          // rows of a slot / of the output
  const int num_m = min(p.meta[1], p.max_tiles);
  const int chunk_cols = p.tiles_n_chunk * kBN;
  const uint32_t tiles_in_chunk = static_cast<uint32_t>(num_m) * p.tiles_n_chunk;
  const int r_idx = blockIdx.x, n_red = p.n_red;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kThreads / 32;
  __shared__ int s_ok;
  for (int c = 0; c < p.n_chunks; ++c) {
    const int c0 = c * chunk_cols;
    const int ccols = min(chunk_cols, p.N - c0);
    const int vecs = ccols >> 3;
    // ---- the chunk's tiles are complete (counter bumped by the GEMM epilogues of this launch)
    if (threadIdx.x == 0) {
      const uint32_t* ctr = p.chunk_done + buf * p.n_chunks + c;
      const uint64_t t0 = globaltimer_ns();
      bool ok = true;
      uint32_t it = 0;
      while (ld_acquire_gpu(ctr) < tiles_in_chunk) {
        if ((++it & 63u) == 0u && (globaltimer_ns() - t0 > p.symm.timeout_ns || abort_requested(p.symm))) {
          report(p.symm, kTimeoutFlag, kKernelMoeReduce, 1, -1, c, (int)tiles_in_chunk, (int)ld_acquire_gpu(ctr));
          ok = false;
          break;
        }
      }
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (s_ok == 0) return;
    // ---- top-k sum of this CTA's tokens, stored into the destination slots [buf][rank]
    for (int t = r_idx * nwarps + warp; t < p.T; t += n_red * nwarps) {
      const int owner = rs ? t / rows_out : -1;
      const int row_dst = rs ? t - owner * rows_out : t;
      int pos[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pos[j] = (j < p.k_top) ? p.pos_of[static_cast<int64_t>(t) * p.k_top + j] : -1;
      // two 16-byte column groups per lane and pass: sixteen row loads in flight per lane
      for (int v0 = lane; v0 < vecs; v0 += 64) {
        const int v1 = v0 + 32;
        const bool has1 = v1 < vecs;
        float acc0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float acc1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 u0[8], u1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const __nv_bfloat16* rowp = p.y + static_cast<int64_t>(pos[j] >= 0 ? pos[j] : 0) * p.ldy + c0;
          u0[j] = pos[j] >= 0 ? ld_v4(rowp + 8 * v0) : make_uint4(0u, 0u, 0u, 0u);
          u1[j] = (pos[j] >= 0 && has1) ? ld_v4(rowp + 8 * v1) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 a0 = unpack_bf16x2(u0[j].x), a1 = unpack_bf16x2(u0[j].y), a2 = unpack_bf16x2(u0[j].z),
                       a3 = unpack_bf16x2(u0[j].w);
          acc0[0] += a0.x; acc0[1] += a0.y; acc0[2] += a1.x; acc0[3] += a1.y;
          acc0[4] += a2.x; acc0[5] += a2.y; acc0[6] += a3.x; acc0[7] += a3.y;
          const float2 b0 = unpack_bf16x2(u1[j].x), b1 = unpack_bf16x2(u1[j].y), b2 = unpack_bf16x2(u1[j].z),
                       b3 = unpack_bf16x2(u1[j].w);
          acc1[0] += b0.x; acc1[1] += b0.y; acc1[2] += b1.x; acc1[3] += b1.y;
          acc1[4] += b2.x; acc1[5] += b2.y; acc1[6] += b3.x; acc1[7] += b3.y;
        }
        // more than eight slots per token: the remaining ones one at a time
        for (int j = 8; j < p.k_top; ++j) {
          const int pj = p.pos_of[static_cast<int64_t>(t) * p.k_top + j];
          if (pj < 0) continue;
          const __nv_bfloat16* rowp = p.y + static_cast<int64_t>(pj) * p.ldy + c0;
          const uint4 w0 = ld_v4(rowp + 8 * v0);
          const float2 a0 = unpack_bf16x2(w0.x), a1 = unpack_bf16x2(w0.y), a2 = unpack_bf16x2(w0.z), a3 = unpack_bf16x2(w0.w);
          acc0[0] += a0.x; acc0[1] += a0.y; acc0[2] += a1.x; acc0[3] += a1.y;
          acc0[4] += a2.x; acc0[5] += a2.y; acc0[6] += a3.x; acc0[7] += a3.y;
          if (has1) {
            const uint4 w1 = ld_v4(rowp + 8 * v1);
            const float2 b0 = unpack_bf16x2(w1.x), b1 = unpack_bf16x2(w1.y), b2 = unpack_bf16x2(w1.z), b3 = unpack_bf16x2(w1.w);
            acc1[0] += b0.x; acc1[1] += b0.y; acc1[2] += b1.x; acc1[3] += b1.y;
            acc1[4] += b2.x; acc1[5] += b2.y; acc1[6] += b3.x; acc1[7] += b3.y;
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (half == 1 && !has1) break;
          const float* acc = half ? acc1 : acc0;
          const int v = half ? v1 : v0;
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
          __nv_bfloat16* slot = p.red_slots + (static_cast<uint64_t>(buf) * W + rank) * p.red_slot_elems +
                                static_cast<uint64_t>(row_dst) * p.N + c0 + 8 * v;
          if (rs) {
            st_v4(symm_at(p.symm, slot, owner), o);
          } else {
            for (int d = 0; d < W; ++d) st_v4(symm_at(p.symm, slot, (rank + d) % W), o);
          }
        }
      }
    }
    // ---- flags: this CTA's part of chunk c is in place on every destination
    __syncthreads();
    if (threadIdx.x < W) {
      fence_acq_rel_sys();
      uint32_t* flag = p.red_flags + (static_cast<uint64_t>(buf) * W + rank) * (p.n_chunks * n_red) + c * n_red + r_idx;
      st_release_sys(symm_at(p.symm, flag, (rank + threadIdx.x) % W), epoch);
    }
    // ---- final sum of the rows this CTA is responsible for on the receiving side.  A destination row (d) receives
    //      its partials from CTA index ((token) / nwarps) % n_red of every source, the token being global: rows are
    //      assigned to summing CTAs by the same rule, so one flag per source covers everything this CTA reads.
    bool ok = true;
    if (threadIdx.x < W) {
      const uint32_t* flag = p.red_flags + (static_cast<uint64_t>(buf) * W + threadIdx.x) * (p.n_chunks * n_red) + c * n_red + r_idx;
      ok = wait_until(p.symm, flag, epoch, kCmpGe, kKernelMoeReduce, 2, threadIdx.x, c * n_red + r_idx);
    }
    ok = __syncthreads_and(ok);
    if (!ok) return;
    const int t_base = rs ? rank * rows_out : 0;    // global token of output row 0
    for (int t = r_idx * nwarps + warp; t < p.T; t += n_red * nwarps) {
      if (t < t_base || t >= t_base + rows_out) continue;
      const int row = t - t_base;
      for (int v = lane; v < vecs; v += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 u[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s)
          if (s < W)
            u[s] = ld_relaxed_sys_v4(p.red_slots + (static_cast<uint64_t>(buf) * W + s) * p.red_slot_elems +
                                     static_cast<uint64_t>(row) * p.N + c0 + 8 * v);
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < W) {
            const float2 f0 = unpack_bf16x2(u[s].x), f1 = unpack_bf16x2(u[s].y), f2 = unpack_bf16x2(u[s].z),
                         f3 = unpack_bf16x2(u[s].w);
            acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
            acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        st_v4(p.out + static_cast<uint64_t>(row) * p.ld_out + c0 + 8 * v, o);
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
moe_fused_kernel(const __grid_constant__ CUtensorMap tmap_b, const MoeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int buf = epoch & 1;
  const int n_aux = p.mode == kMoeAllGather ? p.n_comm : (p.mode == kMoePlain ? 0 : p.n_red);

  if (static_cast<int>(blockIdx.x) < n_aux) {
    if (p.mode == kMoeAllGather) {
      ag_push(p, epoch, smem);
    } else {
      moe_reducer(p, epoch);
    }
  } else {
    if (threadIdx.x == 0) {
      for (int i = 0; i < kStages; ++i) {
        mbar_init(&full_bar[i], 129);    // 128 gather threads (deferred arrivals) + the B producer's expect_tx arrival
        mbar_init(&empty_bar[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&tmem_full[i], 1);
        mbar_init(&tmem_empty[i], 128);
      }
      *abort_flag = 0;
      fence_mbar_init();
      tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
      tmem_alloc(tmem_base_smem, 2 * kBN);
      tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_smem;

    const int n_gemm = gridDim.x - n_aux;
    const int g_idx = blockIdx.x - n_aux;
    const int num_m = min(p.meta[1], p.max_tiles);
    const int num_kb = (p.K + kBK - 1) / kBK;
    // work item w -> (N chunk, position in the tile order, n-tile inside the chunk); chunk-major so that a chunk's
    // tiles finish together, n-tile innermost so that consecutive items of a CTA reuse the gathered rows from L2
    const int n_chunks = p.mode == kMoePlain || p.mode == kMoeAllGather ? 1 : p.n_chunks;
    const int tnc = n_chunks == 1 ? p.tiles_n : p.tiles_n_chunk;
    const int items_per_chunk = num_m * tnc;
    const int num_items = items_per_chunk * n_chunks;
    auto decode = [&](int w, int* m_tile, int* n_tile, int* chunk) {
      const int c = w / items_per_chunk;
      const int r = w - c * items_per_chunk;
      const int mi = r / tnc;
      *chunk = c;
      *n_tile = c * tnc + (r - mi * tnc);
      *m_tile = p.order != nullptr ? p.order[mi] : mi;
    };

    if (warp == 0) {
      // ------------------------------------------------------------ B producer (TMA)
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int w = g_idx; w < num_items && ok; w += n_gemm) {
          int mt, nt, ch;
          decode(w, &mt, &nt, &ch);
          if (nt >= p.tiles_n) continue;
          const int expert = p.tile_expert[mt];
          if (expert < 0) continue;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.mbar_timeout_ns)) {
              ok = false;
              report(p.symm, kTimeoutMbarrier, kKernelGroupGemm, 10, -1, s, (int)ph, w);
              break;
            }
            mbar_arrive_expect_tx(&full_bar[s], kBBytes);
            tma_load_3d(smem + s * kStageBytes + kABytes, &tmap_b, &full_bar[s], kb * kBK, nt * kBN, expert);
          }
        }
        if (!ok) *abort_flag = 1;
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc(1u, kBM, kBN);
        uint32_t it = 0;
        int local = 0;
        bool ok = true;
        for (int w = g_idx; w < num_items && ok; w += n_gemm) {
          int mt, nt, ch;
          decode(w, &mt, &nt, &ch);
          if (nt >= p.tiles_n || p.tile_expert[mt] < 0) continue;
          const int b = local & 1;
          const uint32_t aph = (local >> 1) & 1;
          ++local;
          if (!mbar_wait(&tmem_empty[b], aph ^ 1, abort_flag, p.mbar_timeout_ns)) {
            ok = false;
            report(p.symm, kTimeoutMbarrier, kKernelGroupGemm, 20, -1, b, (int)aph, w);
            break;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + b * kBN;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_wait(&full_bar[s], ph, abort_flag, p.mbar_timeout_ns)) {
              ok = false;
              report(p.symm, kTimeoutMbarrier, kKernelGroupGemm, 21, -1, s, (int)ph, w);
              break;
            }
            // the A rows were written by cp.async of the gather threads (generic proxy), whose completion this thread
            // has just observed through the barrier: order them before the tensor core's (async proxy) reads
            fence_proxy_async_smem();
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + s * kStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + kABytes);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k)
              umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit(&empty_bar[s]);
          }
          if (ok) umma_commit(&tmem_full[b]);
        }
        if (!ok) *abort_flag = 1;
      }
    } else if (warp < 6) {
      // ------------------------------------------------------------ epilogue (warps 2..5)
      const int q = warp & 3;
      const bool leader = (warp == 2 && lane == 0);
      const int row_in_tile = q * 32 + lane;
      int local = 0;
      bool ok = true;
      for (int w = g_idx; w < num_items && ok; w += n_gemm) {
        int mt, nt, ch;
        decode(w, &mt, &nt, &ch);
        if (nt >= p.tiles_n || p.tile_expert[mt] < 0) {
          // a tile that is skipped still counts towards its chunk
          if (p.chunk_done != nullptr && leader) red_release_gpu_add(p.chunk_done + buf * p.n_chunks + ch, 1u);
          continue;
        }
        const int b = local & 1;
        const uint32_t aph = (local >> 1) & 1;
        ++local;
        if (!mbar_wait(&tmem_full[b], aph, abort_flag, p.mbar_timeout_ns)) {
          ok = false;
          if (lane == 0) report(p.symm, kTimeoutMbarrier, kKernelGroupGemm, 30, -1, b, (int)aph, w);
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_acc = tmem_base + b * kBN + (static_cast<uint32_t>(q * 32) << 16);
        const int srow = mt * kBM + row_in_tile;
        const int id = p.sorted_ids[srow];
        const float wgt = (p.row_weight != nullptr && id >= 0) ? p.row_weight[id] : 1.f;
        __nv_bfloat16* dst = nullptr;
        if (p.scatter_out) {
          if (id >= 0) dst = p.y + static_cast<int64_t>(id) * p.ldy;
        } else {
          dst = p.y + static_cast<int64_t>(srow) * p.ldy;   // padding rows are written too (zeros): the layout stays dense
        }
        const int n0 = nt * kBN;
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (c == kBN / 32 - 1) {
            tc_fence_before_sync();
            mbar_arrive(&tmem_empty[b]);
          }
          const int col0 = n0 + c * 32;
          if (dst != nullptr && col0 < p.N) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col0 + 8 * j + 8 <= p.N) {
                uint4 o;
                o.x = pack_bf16x2(wgt * __uint_as_float(r[8 * j + 0]), wgt * __uint_as_float(r[8 * j + 1]));
                o.y = pack_bf16x2(wgt * __uint_as_float(r[8 * j + 2]), wgt * __uint_as_float(r[8 * j + 3]));
                o.z = pack_bf16x2(wgt * __uint_as_float(r[8 * j + 4]), wgt * __uint_as_float(r[8 * j + 5]));
                o.w = pack_bf16x2(wgt * __uint_as_float(r[8 * j + 6]), wgt * __uint_as_float(r[8 * j + 7]));
                st_v4(dst + col0 + 8 * j, o);
              }
            }
          }
        }
        if (p.chunk_done != nullptr) {
          // all 128 rows of the tile are stored before the chunk counter moves
          epi_bar();
          if (leader) {
            __threadfence();
            red_release_gpu_add(p.chunk_done + buf * p.n_chunks + ch, 1u);
          }
        }
      }
      if (!ok) *abort_flag = 1;
    } else {
      // ------------------------------------------------------------ A gather (warps 6..9)
      // Eight consecutive lanes copy the eight 16-byte pieces of one 128-byte row segment, so a warp instruction
      // fetches four whole 128-byte lines (a lane per row would touch 32 half-used sectors); a thread owns piece
      // g % 8 of the eight rows g / 8 + 16 i.
      const int g = threadIdx.x - 192;
      const int piece = g & 7;
      const int row0 = g >> 3;
      // A thread never waits for its copies: after the eight copies of a k-block it leaves a deferred arrival on the
      // stage's barrier (cp.async.mbarrier.arrive.noinc), which fires when they have landed.  So every free stage of the
      // ring is in flight, and a stage is handed to the tensor core the moment its last copy lands (tying the hand-off to
      // the issue of a later stage made every MMA wait for the completion of its predecessor).
      uint32_t it = 0;          // k-blocks issued (stage ring position)
      bool ok = true;
      for (int w = g_idx; w < num_items && ok; w += n_gemm) {
        int mt, nt, ch;
        decode(w, &mt, &nt, &ch);
        if (nt >= p.tiles_n || p.tile_expert[mt] < 0) continue;
        const char* src[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = row0 + 16 * i;
          const int id = p.sorted_ids[mt * kBM + r];
          src[i] = nullptr;
          if (id >= 0) {
            const int64_t srow = id / p.a_row_div;
            if (p.mode == kMoeAllGather) {
              const int owner = static_cast<int>(srow / p.t_local);
              const int lrow = static_cast<int>(srow - static_cast<int64_t>(owner) * p.t_local);
              if (owner == p.symm.rank) {
                src[i] = reinterpret_cast<const char*>(p.x + static_cast<int64_t>(lrow) * p.ldx);
              } else {
                // wait for exactly the chunk this row lives in
                const uint32_t* flag = p.ag_flags + (static_cast<uint64_t>(buf) * p.symm.world + owner) * p.max_chunks + lrow / kBM;
                if (!wait_until(p.symm, flag, epoch, kCmpGe, kKernelGroupGemm, 1, owner, lrow / kBM)) *abort_flag = 1;
                src[i] = reinterpret_cast<const char*>(p.ag_ws + buf * p.ag_buf_elems +
                                                       (static_cast<uint64_t>(owner) * p.t_local + lrow) * p.K);
              }
            } else {
              src[i] = reinterpret_cast<const char*>(p.x + srow * p.ldx);
            }
          }
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.mbar_timeout_ns)) {
            ok = false;
            if (g == 0) report(p.symm, kTimeoutMbarrier, kKernelGroupGemm, 50, -1, s, (int)ph, w);
            break;
          }
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const int kcol = kb * kBK + 8 * piece;            // first element of this thread's piece
          const bool k_ok = kcol + 8 <= p.K;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = row0 + 16 * i;
            const bool valid = src[i] != nullptr && k_ok;
            cp_async_16(sa + r * 128 + ((piece ^ (r & 7)) << 4),
                        valid ? src[i] + static_cast<int64_t>(kcol) * 2 : reinterpret_cast<const char*>(p.x), valid);
          }
          cp_async_arrive_noinc(&full_bar[s]);
        }
      }
      cp_async_commit();
      cp_async_wait<0>();       // nothing of this thread is in flight when the CTA winds down
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, 2 * kBN);
    }
  }

  // last CTA out advances the call epoch and clears the chunk counters of the parity the next-but-one call will use
  if (p.ctx != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t prev = atomicAdd(&p.ctx->done, 1u);
      if (prev == gridDim.x - 1) {
        if (p.chunk_done != nullptr)
          for (int c = 0; c < p.n_chunks; ++c) p.chunk_done[buf * p.n_chunks + c] = 0;
        p.ctx->done = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(&p.ctx->epoch) = epoch + 1;
      }
    }
  }
}

}  // namespace

cudaError_t launch_moe_fused(const MoeFusedArgs& a, cudaStream_t stream) {
  static_assert(kSmemTotal + 1024 <= 227 * 1024, "fused MoE kernel exceeds the shared memory of an SM");
  const int smem = kSmemTotal + 1024;
  {
    static SmemOptIn opt_in;
    cudaError_t e = opt_in.ensure(moe_fused_kernel, smem);
    if (e != cudaSuccess) return e;
  }
  if (a.K % 8 != 0 || a.N % 8 != 0 || a.ldx % 8 != 0 || a.ldy % 8 != 0) return cudaErrorInvalidValue;
  if (a.k_top < 1) return cudaErrorInvalidValue;
  MoeParams p;
  memset(&p, 0, sizeof(p));
  p.mode = a.mode;
  p.K = a.K; p.N = a.N; p.k_top = a.k_top;
  p.x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  p.ldx = a.ldx;
  p.a_row_div = a.a_row_div;
  p.sorted_ids = a.sorted_ids;
  p.tile_expert = a.tile_expert;
  p.order = a.order;
  p.meta = a.meta;
  p.max_tiles = a.max_tiles;
  p.y = reinterpret_cast<__nv_bfloat16*>(a.y);
  p.ldy = a.ldy;
  p.scatter_out = a.scatter_out;
  p.row_weight = a.row_weight;
  p.tiles_n = (a.N + kBN - 1) / kBN;
  p.t_local = a.t_local;
  p.n_comm = a.n_comm;
  p.ag_ws = reinterpret_cast<__nv_bfloat16*>(a.ag_ws);
  p.ag_buf_elems = static_cast<uint64_t>(a.symm.world) * a.max_t_local * static_cast<uint64_t>(a.K);
  p.ag_flags = a.ag_flags;
  p.max_chunks = a.max_chunks;
  p.n_chunks = a.n_chunks > 0 ? a.n_chunks : 1;
  p.tiles_n_chunk = (p.tiles_n + p.n_chunks - 1) / p.n_chunks;
  p.n_red = a.n_red;
  p.T = a.T;
  p.pos_of = a.pos_of;
  p.chunk_done = a.chunk_done;
  p.red_slots = reinterpret_cast<__nv_bfloat16*>(a.red_slots);
  p.red_slot_elems = a.red_slot_elems;
  p.red_flags = a.red_flags;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.ld_out = a.ld_out;
  p.ctx = a.ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &a.symm, sizeof(SymmInfo));
  p.mbar_timeout_ns = a.symm.timeout_ns > 0 ? a.symm.timeout_ns : 4000000000ull;
  int n_aux = 0;
  if (a.mode == kMoeAllGather) {
    if (a.n_comm < 1 || a.t_local < 1 || (a.t_local + kBM - 1) / kBM > a.max_chunks || a.t_local > a.max_t_local)
      return cudaErrorInvalidValue;
    // the token rows pushed by bulk copies: 16-byte multiples
    if ((static_cast<uint64_t>(a.K) * 2) % 16 != 0) return cudaErrorInvalidValue;
    n_aux = a.n_comm;
  } else if (a.mode == kMoeReduceRS || a.mode == kMoeReduceAR) {
    if (a.n_red < 1 || a.T < 1 || a.chunk_done == nullptr || a.pos_of == nullptr) return cudaErrorInvalidValue;
    if (a.mode == kMoeReduceRS && a.T % a.symm.world != 0) return cudaErrorInvalidValue;
    // chunk boundaries fall on tile boundaries, so every chunk but the last is a multiple of 8 columns wide
    n_aux = a.n_red;
  }
  if (a.num_ctas - n_aux < 1) return cudaErrorInvalidValue;
  CUtensorMap tb;
  memcpy(&tb, a.tmap_b.bytes, sizeof(CUtensorMap));
  if (a.mode == kMoeReduceRS || a.mode == kMoeReduceAR) {
    // the reducer CTAs wait for chunk counters that the GEMM CTAs of the same launch bump: all CTAs must be resident
    return launch_coop(moe_fused_kernel, dim3(a.num_ctas), dim3(kThreads), static_cast<size_t>(smem), stream, tb, p);
  }
  moe_fused_kernel<<<a.num_ctas, kThreads, smem, stream>>>(tb, p);
  return cudaGetLastError();
}

}  // namespace tdb
