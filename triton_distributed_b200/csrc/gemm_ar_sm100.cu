// Small-M ("decode") GEMM with split-K and an optional fused all-reduce:
//
//     out[M, N] = sum over ranks ( X[M, K_local] * W[N, K_local]^T ),   M <= 256
//
// The problem is swapped so that the weight rows fill the 128-row dimension of tcgen05.mma: the A operand is a
// 128 x 64 weight tile, the B operand the M_pad x 64 activation tile, and the accumulator in TMEM is
// [128 lanes = output columns] x [M_pad columns = tokens].  The weights are read exactly once through a deep TMA ring,
// which is what bounds decode GEMMs.  Two kernels share this core:
//
//   cluster form (skinny_cluster_kernel, the default): the S <= 8 CTAs of a thread-block cluster share one tile of
//     128 * NT columns and split its K range evenly; their fp32 parts meet through distributed shared memory
//     (no global scratch, no atomics, a result that does not depend on arrival order).  Launched with programmatic
//     dependent launch: weight tiles are requested before griddepcontrol.wait.
//   stream-K form (skinny_gemm_kernel; more column tiles than SMs, explicit split counts, unsplit tiles): the work is
//     the flattened list of (column tile, k-block) units; every CTA takes one contiguous, equally long range of it, so
//     all SMs stream the same number of weight bytes whatever the tile count is.  A range covers pieces of one to three
//     tiles.  A piece that spans a tile's whole K is stored directly; other pieces are added with
//     red.global.add.v4.f32 into a column-major accumulation buffer, and the CTA that arrives last on a column tile
//     converts it and clears the buffer again (self-cleaning, CUDA-graph safe).
//
// In all-reduce mode the CTA that completes a column tile (the last arriver, or the first CTA of the cluster) runs the
// cross-rank sum for that tile right away:
//     NVLS:  store the bf16 partial tile to the heap, flag all ranks, wait for all ranks' flags of this tile,
//            multimem.ld_reduce the tile (summed inside the switch) -> out
//     push:  store the partial tile into slot [rank] on every peer, flag, wait, sum the W slots -> out
// so there is one launch per layer op, and in the stream-K form the all-reduce of early tiles overlaps the GEMM of
// later ones.
//
// Reference behaviour being matched (not its code): python/triton_dist/kernels/nvidia/gemm_allreduce.py:124-315
// (per-tile flags, consumer CTAs reduce with multimem.ld_reduce, double-buffered phases :74-92), layer wrapper
// layers/nvidia/gemm_allreduce_layer.py:32-116.
#include <cuda.h>

#include <cstdlib>

#include "tdb/api.h"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kTN = 128;    // output columns per tile (MMA M)
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
// shared-memory barrier waits follow the configured wait limit of the launch (symm.timeout_ns, TDB200_WAIT_TIMEOUT_S;
// four seconds when the caller passes none)
#define kMbarTimeoutNs (p.symm.timeout_ns != 0 ? p.symm.timeout_ns : 4000000000ull)

template <int MPAD>
struct Layout {
  static constexpr int kWBytes = kTN * kBK * 2;        // 16 KB
  static constexpr int kXBytesRaw = MPAD * kBK * 2;
  static constexpr int kXBytes = (kXBytesRaw + 1023) / 1024 * 1024;   // keep every operand 1024-byte aligned
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes > 12 ? 12 : (200 * 1024) / kStageBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 32;
  static constexpr int kTmemCols = (2 * MPAD) < 32 ? 32 : 2 * MPAD;
};

struct KP {
  int M, N, K;
  int tiles_n, kb_total;
  int per_cta;               // (tile, k-block) units per CTA (stream-K form)
  int cluster_s;             // CTAs per column tile (cluster form)
  int bulk_exchange;         // cluster form: parts travel as bulk copies into the reducing CTA's shared memory
  __nv_bfloat16* out;        // [M, N]
  int64_t ld_out;
  float* acc;                // [tiles_n * 128, M_pad] fp32 split-K accumulation (all zero between calls)
  uint32_t* counters;        // [tiles_n] arrivals per tile (zero between calls)
  int mode;                  // 0 plain, 1 all-reduce
  int use_mc;
  __nv_bfloat16* partial;    // heap: NVLS [2][M_cap][N]; push [2][W][M_cap][N]
  uint64_t partial_half;     // elements per parity buffer
  uint32_t* flags;           // heap [W][max_tiles] epochs
  int max_tiles;
  int m_cap;
  CtxDev* ctx;
  SymmInfo symm;
};

TDB_DEVICE void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
TDB_DEVICE void red_add_v4_f32(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// The pieces of this CTA's unit range, in order: (column tile, [kb0, kb1)).
struct PieceIter {
  int u, u1, kb_total;
  int nt, kb0, kb1;
  TDB_DEVICE PieceIter(const KP& p) : kb_total(p.kb_total) {
    const int total = p.tiles_n * p.kb_total;
    u = min(total, static_cast<int>(blockIdx.x) * p.per_cta);
    u1 = min(total, u + p.per_cta);
  }
  TDB_DEVICE bool next() {
    if (u >= u1) return false;
    nt = u / kb_total;
    kb0 = u - nt * kb_total;
    kb1 = min(kb_total, kb0 + (u1 - u));
    u += kb1 - kb0;
    return true;
  }
};
// number of CTAs whose ranges touch tile nt
TDB_DEVICE int pieces_of_tile(const KP& p, int nt) {
  return ((nt + 1) * p.kb_total - 1) / p.per_cta - (nt * p.kb_total) / p.per_cta + 1;
}

// Cross-rank sum of column tile nt, run by the 128 epilogue threads of one CTA after the rank's bf16 partial of the tile
// is complete in `dst` (the heap partial of this parity): push or NVLS form.  False when a peer's flag did not arrive
// within the wait limit.
TDB_DEVICE bool tile_exchange(const KP& p, int nt, __nv_bfloat16* dst, int par, uint32_t epoch) {
  const int W = p.symm.world, rank = p.symm.rank;
  // ---- cross-rank sum of this tile
  const int tn = min(kTN, p.N - nt * kTN);   // valid columns of the tile (multiple of 8)
  if (!p.use_mc) {
    // push the tile into slot [rank] of every peer
    epi_bar();
    const int vec_per_row = tn / 8;
    const int et = threadIdx.x - 64;
    for (int v = et; v < p.M * vec_per_row; v += 128) {
      const int m = v / vec_per_row, cv = v - m * vec_per_row;
      __nv_bfloat16* src = dst + static_cast<int64_t>(m) * p.N + nt * kTN + cv * 8;
      const uint4 u = ld_v4(src);
      for (int j = 1; j < W; ++j) st_v4(symm_at(p.symm, src, (rank + j) % W), u);
    }
  }
  epi_bar();
  const int et = threadIdx.x - 64;   // 0..127 within the epilogue warps
  bool wok = true;
  if (et < W) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(p.symm, p.flags + static_cast<int64_t>(rank) * p.max_tiles + nt, (rank + et) % W), epoch);
    wok = wait_until(p.symm, p.flags + static_cast<int64_t>(et) * p.max_tiles + nt, epoch, kCmpGe, kKernelGemmAr, 40,
                     et, nt);
  }
  // combine the per-thread results without leaving the named barrier unbalanced
  __shared__ int s_wok;
  if (et == 0) s_wok = 1;
  epi_bar();
  if (!wok) s_wok = 0;
  epi_bar();
  if (s_wok == 0) return false;
  const int vec_per_row = tn / 8;
  const int total_vec = p.M * vec_per_row;
  if (p.use_mc) {
    // the switch returns the sum over all ranks; eight requests per thread are in flight at a time (one NVLS
    // round trip costs microseconds, and a tile of 128 tokens has sixteen 16-byte vectors per thread)
    constexpr int kInFlight = 8;
    for (int v0 = et; v0 < total_vec; v0 += 128 * kInFlight) {
      uint4 o[kInFlight];
#pragma unroll
      for (int i = 0; i < kInFlight; ++i) {
        const int v = v0 + i * 128;
        if (v < total_vec) {
          const int m = v / vec_per_row, cv = v - m * vec_per_row;
          const __nv_bfloat16* src = p.partial + par * p.partial_half + static_cast<int64_t>(m) * p.N + nt * kTN + cv * 8;
          o[i] = multimem_ld_reduce_bf16x8(mc_ptr(p.symm, src));
        }
      }
#pragma unroll
      for (int i = 0; i < kInFlight; ++i) {
        const int v = v0 + i * 128;
        if (v < total_vec) {
          const int m = v / vec_per_row, cv = v - m * vec_per_row;
          st_v4(p.out + static_cast<int64_t>(m) * p.ld_out + nt * kTN + cv * 8, o[i]);
        }
      }
    }
  } else {
    for (int v = et; v < total_vec; v += 128) {
      const int m = v / vec_per_row, cv = v - m * vec_per_row;
      const int col = nt * kTN + cv * 8;
      uint4 u[kMaxRanks];
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)
        if (s < W)
          u[s] = ld_relaxed_sys_v4(p.partial + par * p.partial_half + (static_cast<uint64_t>(s) * p.m_cap + m) * p.N + col);
      float accv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < W) {
          const float2 f0 = unpack_bf16x2(u[s].x), f1 = unpack_bf16x2(u[s].y), f2 = unpack_bf16x2(u[s].z),
                       f3 = unpack_bf16x2(u[s].w);
          accv[0] += f0.x; accv[1] += f0.y; accv[2] += f1.x; accv[3] += f1.y;
          accv[4] += f2.x; accv[5] += f2.y; accv[6] += f3.x; accv[7] += f3.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(accv[0], accv[1]); o.y = pack_bf16x2(accv[2], accv[3]);
      o.z = pack_bf16x2(accv[4], accv[5]); o.w = pack_bf16x2(accv[6], accv[7]);
      st_v4(p.out + static_cast<int64_t>(m) * p.ld_out + col, o);
    }
  }
  return true;
}

template <int MPAD>
__global__ void __launch_bounds__(kThreads, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const KP p) {
  using L = Layout<MPAD>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);
  volatile int* is_last = reinterpret_cast<volatile int*>(tmem_base_smem + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int par = epoch & 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_smem, L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_smem;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0, issued = 0;
      bool ok = true;
      for (PieceIter pc(p); ok && pc.next();) {
        const int nt = pc.nt, kb0 = pc.kb0, kb1 = pc.kb1;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, kMbarTimeoutNs)) {
            ok = false;
            report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 10, -1, s, (int)ph, nt);
            break;
          }
          uint8_t* sw = smem + s * L::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[s], L::kWBytes + L::kXBytesRaw);
          tma_load_2d(sw, &tmap_w, &full_bar[s], kb * kBK, nt * kTN);
          tma_load_2d(sw + L::kWBytes, &tmap_x, &full_bar[s], kb * kBK, 0);
          ++issued;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        const uint32_t first = issued > (uint32_t)kStages ? issued - kStages : 0;
        for (uint32_t j = first; j < issued; ++j) mbar_wait(&full_bar[j % kStages], (j / kStages) & 1, nullptr, 200000000ull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1u, kTN, MPAD);
      uint32_t it = 0;
      int local = 0;
      bool ok = true;
      for (PieceIter pc(p); ok && pc.next(); ++local) {
        const int kb0 = pc.kb0, kb1 = pc.kb1;
        const int b = local & 1;
        const uint32_t aph = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[b], aph ^ 1, abort_flag, kMbarTimeoutNs)) {
          ok = false;
          report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 20, -1, b, (int)aph, pc.nt);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + b * MPAD;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, kMbarTimeoutNs)) {
            ok = false;
            report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 21, -1, s, (int)ph, pc.nt);
            break;
          }
          tc_fence_after_sync();
          const uint32_t sw = smem_u32(smem + s * L::kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sw);
          const uint64_t bdesc = make_smem_desc_sw128(sw + L::kWBytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tmem_full[b]);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int q = warp & 3;
    const bool leader = (warp == 2 && lane == 0);
    const int rank = p.symm.rank;
    int local = 0;
    bool ok = true;
    for (PieceIter pc(p); ok && pc.next(); ++local) {
      const int nt = pc.nt;
      const int b = local & 1;
      const uint32_t aph = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[b], aph, abort_flag, kMbarTimeoutNs)) {
        ok = false;
        if (lane == 0) report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 30, -1, b, (int)aph, nt);
        break;
      }
      tc_fence_after_sync();
      const int n = nt * kTN + q * 32 + lane;   // this thread's output column
      const bool n_ok = n < p.N;
      const int pieces = pieces_of_tile(p, nt);
      // A piece that covers the tile's whole K needs no split accumulation: its values go straight to their bf16
      // destination (the output, or the heap partial of the all-reduce).
      const bool single = pieces == 1;
      const bool direct = single && p.mode == 0;
      __nv_bfloat16* dst;
      int64_t ld_dst;
      if (p.mode == 0) {
        dst = p.out;
        ld_dst = p.ld_out;
      } else if (p.use_mc) {
        dst = p.partial + par * p.partial_half;
        ld_dst = p.N;
      } else {
        dst = p.partial + par * p.partial_half + static_cast<uint64_t>(rank) * p.m_cap * p.N;
        ld_dst = p.N;
      }
      // split accumulation buffer: [column][M_pad] fp32, so that a thread's sixteen consecutive tokens of its column
      // are contiguous and go out as four 16-byte vector reductions
      float* acc_col = p.acc + static_cast<int64_t>(nt * kTN + q * 32 + lane) * MPAD;
#pragma unroll 1
      for (int c = 0; c < MPAD / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x16(tmem_base + b * MPAD + c * 16 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (!n_ok) continue;
        if (single) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c * 16 + j;
            if (m < p.M) dst[static_cast<int64_t>(m) * ld_dst + n] = __float2bfloat16(__uint_as_float(r[j]));
          }
        } else {
          // rows at or beyond M are zero (the activation tile is zero-filled there), so whole quads are added
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            if (c * 16 + j < p.M)
              red_add_v4_f32(acc_col + c * 16 + j, __uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                             __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[b]);
      if (direct) continue;
      if (!single) {
        // ---- tile arrival: the last split to finish owns the tile's finalisation
        __threadfence();
        epi_bar();
        if (leader) {
          const uint32_t prev = atomicAdd(p.counters + nt, 1u);
          *is_last = (prev == static_cast<uint32_t>(pieces) - 1) ? 1 : 0;
          if (*is_last) p.counters[nt] = 0;
        }
        epi_bar();
        if (*is_last == 0) continue;
        __threadfence();
        // finalise: fp32 accumulation -> bf16 (out, or the heap partial for the all-reduce); clear the accumulator
        if (n_ok) {
          // batches of independent 16-byte loads: one L2 round trip per batch
          constexpr int kBatch = MPAD < 32 ? MPAD : 32;
          for (int m0 = 0; m0 < p.M; m0 += kBatch) {
            float4 v[kBatch / 4];
#pragma unroll
            for (int j = 0; j < kBatch / 4; ++j)
              v[j] = (m0 + 4 * j < p.M) ? __ldcg(reinterpret_cast<const float4*>(acc_col + m0 + 4 * j))
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kBatch / 4; ++j) {
              if (m0 + 4 * j < p.M) {
                *reinterpret_cast<float4*>(acc_col + m0 + 4 * j) = make_float4(0.f, 0.f, 0.f, 0.f);
                const float f[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (m0 + 4 * j + e < p.M)
                    dst[static_cast<int64_t>(m0 + 4 * j + e) * ld_dst + n] = __float2bfloat16(f[e]);
              }
            }
          }
        }
      }
      if (p.mode == 0) continue;
      if (!tile_exchange(p, nt, dst, par, epoch)) {
        ok = false;
        break;
      }
    }
    if (!ok) *abort_flag = 1;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
  if (p.ctx != nullptr) {
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
}

TDB_DEVICE float4 ld_dsmem_v4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
// shared::cta -> shared::cluster bulk copy; completes `bytes` on the destination CTA's mbarrier.  Addresses 16-byte
// aligned, size a multiple of 16.
TDB_DEVICE void bulk_copy_to_cluster(uint32_t dst_cluster_addr, const void* src, uint32_t bytes, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster_addr),
               "r"(smem_u32(src)), "r"(bytes), "r"(bar_cluster_addr)
               : "memory");
}
TDB_DEVICE void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
TDB_DEVICE void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }

// Cluster form of the same GEMM: the S CTAs of a thread-block cluster share ONE column tile (128 * NT columns) and
// split its K range evenly.  Every CTA accumulates its part in TMEM (NT accumulators that share each activation tile),
// parks it as fp32 in its own shared memory (the drained TMA ring), and after a cluster barrier CTA r sums rows
// [r * M / S, (r + 1) * M / S) over all S parts through distributed shared memory and stores them as bf16 rows.  No
// global accumulation buffer, no atomics, no arrival counters; the result does not depend on arrival order.  In
// all-reduce mode CTA 0 of the cluster then runs the cross-rank sum of the tile's NT column blocks.
constexpr int cluster_stage_bytes(int mpad, int nt) { return nt * kTN * kBK * 2 + (mpad * kBK * 2 + 1023) / 1024 * 1024; }
constexpr int cluster_stages(int mpad, int nt) {
  return (200 * 1024) / cluster_stage_bytes(mpad, nt) > 12 ? 12 : (200 * 1024) / cluster_stage_bytes(mpad, nt);
}
constexpr int pow2_at_least(int v) { return v <= 32 ? 32 : v <= 64 ? 64 : v <= 128 ? 128 : v <= 256 ? 256 : 512; }
// a (token pad, tile width) pair can run when its accumulators fit TMEM, its fp32 part fits the drained ring and the
// ring keeps at least three stages
constexpr bool cluster_form_ok(int mpad, int nt) {
  return nt * mpad <= 512 && cluster_stages(mpad, nt) >= 3 &&
         nt * mpad * kTN * 4 <= cluster_stages(mpad, nt) * cluster_stage_bytes(mpad, nt);
}

template <int MPAD, int NT>
struct ClusterLayout {
  static constexpr int kWBytes = NT * kTN * kBK * 2;   // NT weight boxes of 16 KB
  static constexpr int kXBytesRaw = MPAD * kBK * 2;
  static constexpr int kXBytes = (kXBytesRaw + 1023) / 1024 * 1024;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = cluster_stages(MPAD, NT);
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 32;
  static constexpr int kTmemCols = pow2_at_least(NT * MPAD);
  static constexpr int kPartBytes = NT * MPAD * kTN * 4;
  // room for the part and, behind it, the slices received from up to seven peers (at most the part's size plus one
  // row per peer)
  static constexpr bool kBulkOk = 2 * kPartBytes + 8 * NT * kTN * 4 <= kBarOffset;
  static_assert(cluster_form_ok(MPAD, NT), "invalid cluster form");
};

template <int MPAD, int NT>
__global__ void __launch_bounds__(kThreads, 1)
skinny_cluster_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const KP p) {
  using L = ClusterLayout<MPAD, NT>;
  constexpr int kStages = L::kStages;
  constexpr int kCols = NT * kTN;                 // columns of the CTA tile
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_full + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.cluster_s;
  const int r = static_cast<int>(cluster_ctarank());
  const int ct = static_cast<int>(blockIdx.x) / S;   // CTA tile: columns [ct * kCols, (ct + 1) * kCols)
  const int kb0 = static_cast<int>(static_cast<int64_t>(p.kb_total) * r / S);
  const int kb1 = static_cast<int>(static_cast<int64_t>(p.kb_total) * (r + 1) / S);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);   // arrival of the peers' slices (bulk exchange)
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_smem, L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_smem;
  float* part = reinterpret_cast<float*>(smem);   // [M][kCols] fp32, written once the ring has drained
  uint64_t* recv_bar = &tmem_full[1];
  const bool bulk = L::kBulkOk && p.bulk_exchange != 0 && S > 1;
  const int rows_per = (p.M + S - 1) / S;         // rows of the tile that one CTA of the cluster reduces
  float* recv = part + MPAD * kCols;              // [S - 1][rows_per][kCols] fp32: the peers' rows of this CTA's slice
  // Programmatic dependent launch: the successor may be scheduled from here on, and this kernel may itself be running
  // before its predecessor has finished.  The weights are constant, so the producer fills the ring with weight tiles
  // first; everything the predecessor may write (activations, the epoch, flags, outputs) is touched after pdl_wait().
  pdl_launch_dependents();
  const int pre = (warp == 0 && lane == 0) ? min(kb1 - kb0, kStages) : 0;
  for (int i = 0; i < pre; ++i) {
    uint8_t* sw = smem + i * L::kStageBytes;
    mbar_arrive_expect_tx(&full_bar[i], L::kWBytes + L::kXBytesRaw);
#pragma unroll
    for (int j = 0; j < NT; ++j)
      tma_load_2d(sw + j * (kTN * kBK * 2), &tmap_w, &full_bar[i], (kb0 + i) * kBK, ct * kCols + j * kTN);
  }
  pdl_wait();
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int par = epoch & 1;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t issued = 0;
      bool ok = true;
      for (; issued < static_cast<uint32_t>(pre); ++issued)
        tma_load_2d(smem + issued * L::kStageBytes + L::kWBytes, &tmap_x, &full_bar[issued], (kb0 + issued) * kBK, 0);
      for (int kb = kb0 + pre; kb < kb1; ++kb, ++issued) {
        const int s = issued % kStages;
        const uint32_t ph = (issued / kStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, kMbarTimeoutNs)) {
          ok = false;
          report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 50, -1, s, (int)ph, ct);
          break;
        }
        uint8_t* sw = smem + s * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], L::kWBytes + L::kXBytesRaw);
#pragma unroll
        for (int j = 0; j < NT; ++j)
          tma_load_2d(sw + j * (kTN * kBK * 2), &tmap_w, &full_bar[s], kb * kBK, ct * kCols + j * kTN);
        tma_load_2d(sw + L::kWBytes, &tmap_x, &full_bar[s], kb * kBK, 0);
      }
      if (!ok) {
        *abort_flag = 1;
        const uint32_t first = issued > (uint32_t)kStages ? issued - kStages : 0;
        for (uint32_t j = first; j < issued; ++j) mbar_wait(&full_bar[j % kStages], (j / kStages) & 1, nullptr, 200000000ull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1u, kTN, MPAD);
      uint32_t it = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(&full_bar[s], ph, abort_flag, kMbarTimeoutNs)) {
          ok = false;
          report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 51, -1, s, (int)ph, ct);
          break;
        }
        tc_fence_after_sync();
        const uint32_t sw = smem_u32(smem + s * L::kStageBytes);
        const uint64_t bdesc = make_smem_desc_sw128(sw + L::kWBytes);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const uint64_t adesc = make_smem_desc_sw128(sw + j * (kTN * kBK * 2));
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_f16(tmem_base + j * MPAD, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(&tmem_full[0]);
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int q = warp & 3;
    if (mbar_wait(&tmem_full[0], 0, abort_flag, kMbarTimeoutNs)) {
      tc_fence_after_sync();
      // all MMAs are complete, so every stage of the ring has been consumed and the fp32 part may overwrite it
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float* mine = part + j * kTN + q * 32 + lane;
        if constexpr (MPAD >= 32) {
#pragma unroll 1
          for (int c = 0; c < MPAD / 32; ++c) {
            if (c * 32 >= p.M) break;
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + j * MPAD + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) mine[(c * 32 + i) * kCols] = __uint_as_float(v[i]);
          }
        } else {
          uint32_t v[16];
          tmem_ld_32x16(tmem_base + j * MPAD + (static_cast<uint32_t>(q * 32) << 16), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) mine[i * kCols] = __uint_as_float(v[i]);
        }
      }
      tc_fence_before_sync();
      if (bulk) fence_proxy_async_smem();   // the copy engine reads the part
    } else {
      if (lane == 0) report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 52, -1, 0, 0, ct);
      *abort_flag = 1;
    }
    if (bulk && threadIdx.x == 64) {
      const int mine_rows = max(0, min(p.M, (r + 1) * rows_per) - r * rows_per);
      mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>((S - 1) * mine_rows * kCols * 4));
    }
  }

  // ---- every part of the tile is parked: CTA r reduces its share of the rows (each thread arrives after its own
  // writes, and the barrier completes only when all threads of all CTAs have arrived)
  cluster_arrive_release();
  cluster_wait_acquire();
  __nv_bfloat16* dst;
  int64_t ld_dst;
  if (p.mode == 0) {
    dst = p.out;
    ld_dst = p.ld_out;
  } else if (p.use_mc) {
    dst = p.partial + par * p.partial_half;
    ld_dst = p.N;
  } else {
    dst = p.partial + par * p.partial_half + static_cast<uint64_t>(p.symm.rank) * p.m_cap * p.N;
    ld_dst = p.N;
  }
  if (warp >= 2) {
    const int et = threadIdx.x - 64;
    constexpr int kVecRow = kCols / 4;              // float4 per row of the part: 32, 64, 96 or 128
    constexpr int kRowsPerPass = 128 / kVecRow;     // 4, 2, 1 (32 threads idle) or 1
    const int c4 = et % kVecRow;                    // columns [4 * c4, 4 * c4 + 4) of the CTA tile
    const int m_lo = r * rows_per;
    const int m_hi = et < kRowsPerPass * kVecRow ? min(p.M, (r + 1) * rows_per) : 0;
    const bool col_ok = ct * kCols + c4 * 4 < p.N;  // N is a multiple of 4
    bool recv_ok = true;
    if (bulk) {
      // push form: every CTA sends each peer the rows that peer reduces (one bulk copy per peer, into the slot of this
      // CTA in the peer's receive area), then sums its own rows from local shared memory only
      if (et == 0) {
        for (int j = 1; j < S; ++j) {
          const int d = (r + j) % S;
          const int lo = d * rows_per, hi = min(p.M, (d + 1) * rows_per);
          if (hi <= lo) continue;
          const int slot = r < d ? r : r - 1;
          bulk_copy_to_cluster(mapa_u32(smem_u32(recv + static_cast<size_t>(slot) * rows_per * kCols), d),
                               part + static_cast<size_t>(lo) * kCols, static_cast<uint32_t>((hi - lo) * kCols * 4),
                               mapa_u32(smem_u32(recv_bar), d));
        }
      }
      recv_ok = mbar_wait(recv_bar, 0, abort_flag, kMbarTimeoutNs);
      if (!recv_ok) {
        if (et == 0) report(p.symm, kTimeoutMbarrier, kKernelGemmAr, 53, -1, r, S, ct);
        *abort_flag = 1;
      }
    }
    for (int m = m_lo + et / kVecRow; recv_ok && m < m_hi; m += kRowsPerPass) {
      float4 v[8];
      v[0] = *reinterpret_cast<const float4*>(part + m * kCols + c4 * 4);   // the own part: a plain shared load
      if (bulk) {
#pragma unroll
        for (int j = 1; j < 8; ++j)
          if (j < S)
            v[j] = *reinterpret_cast<const float4*>(recv + (static_cast<size_t>(j - 1) * rows_per + (m - m_lo)) * kCols + c4 * 4);
      } else {
        const uint32_t local = smem_u32(part + m * kCols + c4 * 4);
#pragma unroll
        for (int j = 1; j < 8; ++j)
          if (j < S) v[j] = ld_dsmem_v4(mapa_u32(local, static_cast<uint32_t>((r + j) % S)));
      }
      float4 a = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j)
        if (j < S) {
          a.x += v[j].x; a.y += v[j].y; a.z += v[j].z; a.w += v[j].w;
        }
      if (col_ok) {
        uint2 o;
        o.x = pack_bf16x2(a.x, a.y);
        o.y = pack_bf16x2(a.z, a.w);
        *reinterpret_cast<uint2*>(dst + static_cast<int64_t>(m) * ld_dst + ct * kCols + c4 * 4) = o;
      }
    }
    if (p.mode == 1) __threadfence();   // CTA 0 of the cluster reads these rows back for the cross-rank sum
  }
  // no CTA may leave (or reuse its shared memory) while a peer still reads its part
  cluster_arrive_release();
  cluster_wait_acquire();
  if (p.mode == 1 && r == 0 && warp >= 2) {
    bool ok = true;
    for (int j = 0; ok && j < NT; ++j)
      if ((ct * NT + j) * kTN < p.N) ok = tile_exchange(p, ct * NT + j, dst, par, epoch);
    if (!ok) *abort_flag = 1;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
  if (p.ctx != nullptr) {
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
}

// Cluster launches of one (M_pad, NT) instantiation: the largest cluster size <= want_s whose clusters all fit into one
// wave (asked from the occupancy API once per process and size), and the launch itself.
template <int MPAD, int NT>
struct ClusterForm {
  using L = ClusterLayout<MPAD, NT>;
  static constexpr int kSmem = L::kTotal + 1024;

  static void fill(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int tiles, int s, cudaStream_t stream) {
    static const bool pdl = [] {
      const char* e = std::getenv("TDB200_PDL");
      return e == nullptr || std::atoi(e) != 0;
    }();
    cfg = cudaLaunchConfig_t{};
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = stream;
    cfg.gridDim = dim3(tiles * s);
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = s;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
  }

  // whether `tiles` clusters of s CTAs are co-resident (asked from the occupancy API once per process and size)
  static bool fits(int tiles, int s) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(skinny_cluster_kernel<MPAD, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
          cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      set = true;
    }
    static int max_clusters[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (s < 1 || s > 8) return false;
    if (max_clusters[s] == 0) {
      cudaLaunchConfig_t cfg;
      cudaLaunchAttribute attr[2];
      fill(cfg, attr, tiles, s, nullptr);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, skinny_cluster_kernel<MPAD, NT>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = -1;
      }
      max_clusters[s] = n > 0 ? n : -1;
    }
    return max_clusters[s] >= tiles;   // one wave
  }

  static cudaError_t launch(const SkinnyGemmArgs& a, KP& p, int tiles, int s, cudaStream_t stream) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    fill(cfg, attr, tiles, s, stream);
    p.cluster_s = s;
    CUtensorMap tw, tx;
    memcpy(&tw, a.tmap_w.bytes, sizeof(CUtensorMap));
    memcpy(&tx, a.tmap_x.bytes, sizeof(CUtensorMap));
    return cudaLaunchKernelEx(&cfg, skinny_cluster_kernel<MPAD, NT>, tw, tx, p);
  }
};

// One (tile width, cluster size) candidate of the cluster form: its cost in bytes one CTA has to move.  Streaming a
// byte of weights or activations into shared memory is the unit; a byte of the fp32 exchange through distributed shared
// memory costs about 2.5 of them (measured: the exchange of a 64 KB part takes as long as streaming 160 KB), and every
// CTA pays a fixed cost worth about 96 KB.
template <int MPAD, int NT>
void cluster_candidates(const SkinnyGemmArgs& a, const KP& p, int num_ctas, int force_s, double* best_cost, int* best_nt,
                        int* best_s, int* best_tiles) {
  if constexpr (cluster_form_ok(MPAD, NT)) {
    const int tiles = (a.N + NT * kTN - 1) / (NT * kTN);
    if (tiles > num_ctas) return;
    int s_max = num_ctas / tiles;
    if (s_max > 8) s_max = 8;
    if (s_max > p.kb_total) s_max = p.kb_total;
    const double unit = NT * kTN * kBK * 2 + MPAD * kBK * 2;
    const double part = static_cast<double>(NT) * MPAD * kTN * 4;
    for (int s = s_max; s >= 1; --s) {
      if (force_s >= 1 && s != force_s) continue;
      if (s > 1 && p.kb_total / s < 4 && force_s < 1) continue;
      if (!ClusterForm<MPAD, NT>::fits(tiles, s)) continue;
      const double kb = (p.kb_total + s - 1) / s;
      const double cost = kb * unit + (s > 1 ? 2.5 * part * (s - 1) / s : 0.0) + 96.0 * 1024;
      if (cost < *best_cost) {
        *best_cost = cost;
        *best_nt = NT;
        *best_s = s;
        *best_tiles = tiles;
      }
    }
  }
}

template <int MPAD, int NT>
cudaError_t cluster_launch_if(const SkinnyGemmArgs& a, KP& p, int tiles, int s, cudaStream_t stream) {
  if constexpr (cluster_form_ok(MPAD, NT)) {
    return ClusterForm<MPAD, NT>::launch(a, p, tiles, s, stream);
  } else {
    return cudaErrorInvalidValue;
  }
}

// Chooses the CTA tile width (128 to 512 columns: a wider tile reads every activation tile less often, but has a larger
// part to exchange and leaves fewer tiles to spread over the SMs) and the cluster size, and launches.  Measured on the
// Qwen3-32B shapes at TP 2 / 4 / 8: from 64 tokens on the 128-column tile with the largest cluster that fits always
// won, so only that is considered there; below, the byte-cost model decides.  A choice that ends at one CTA per tile
// is left to the stream-K kernel, whose unsplit tiles go from TMEM straight to their destination (`whole_tiles`).
// `launched` stays false when no cluster form fits or is wanted; the caller then runs the stream-K form.
template <int MPAD>
cudaError_t launch_cluster_form(const SkinnyGemmArgs& a, KP& p, int num_ctas, int force_s, int force_nt,
                                bool explicit_cfg, cudaStream_t stream, bool* launched, bool* whole_tiles) {
  *launched = false;
  int nt = 0, s = 0, tiles = 0;
  double cost = 1e30;
  // all-reduce mode: one 128-column block per cluster, so that the cross-rank exchanges of all blocks run side by side
  // (the blocks of a wider tile would be exchanged one after the other by the cluster's first CTA)
  const bool narrow_only = (MPAD >= 64 || a.all_reduce != 0) && force_nt == 0;
  if (force_nt == 0 || force_nt == 1) cluster_candidates<MPAD, 1>(a, p, num_ctas, force_s, &cost, &nt, &s, &tiles);
  if (!narrow_only) {
    if (force_nt == 0 || force_nt == 2) cluster_candidates<MPAD, 2>(a, p, num_ctas, force_s, &cost, &nt, &s, &tiles);
    if (force_nt == 0 || force_nt == 3) cluster_candidates<MPAD, 3>(a, p, num_ctas, force_s, &cost, &nt, &s, &tiles);
    if (force_nt == 0 || force_nt == 4) cluster_candidates<MPAD, 4>(a, p, num_ctas, force_s, &cost, &nt, &s, &tiles);
  }
  if (nt == 0) return cudaSuccess;
  if (s == 1 && !explicit_cfg && force_s == 0) {
    *whole_tiles = true;
    return cudaSuccess;
  }
  *launched = true;
  switch (nt) {
    case 1: return cluster_launch_if<MPAD, 1>(a, p, tiles, s, stream);
    case 2: return cluster_launch_if<MPAD, 2>(a, p, tiles, s, stream);
    case 3: return cluster_launch_if<MPAD, 3>(a, p, tiles, s, stream);
    default: return cluster_launch_if<MPAD, 4>(a, p, tiles, s, stream);
  }
}

template <int MPAD>
cudaError_t launch_t(const SkinnyGemmArgs& a, const KP& p, int grid, cudaStream_t stream) {
  using L = Layout<MPAD>;
  const int smem = L::kTotal + 1024;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    set = true;
  }
  CUtensorMap tw, tx;
  memcpy(&tw, a.tmap_w.bytes, sizeof(CUtensorMap));
  memcpy(&tx, a.tmap_x.bytes, sizeof(CUtensorMap));
  skinny_gemm_kernel<MPAD><<<grid, kThreads, smem, stream>>>(tw, tx, p);
  return cudaGetLastError();
}

}  // namespace

int skinny_gemm_mpad(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : M <= 256 ? 256 : -1; }

int skinny_gemm_pick_splits(int N, int K, int num_sms, int M) {
  // A work item is (128 columns, one K split); items run in rounds of `num_sms`.  Pick the split count that
  // minimises rounds x (time of one item), keeping at least 6 k-blocks per item so that the
  // pipeline fill does not dominate; the fp32 accumulation traffic of the splits (M x N x 8 bytes per split against
  // N x K x 2 bytes of weights) is charged too.
  const int tiles = (N + kTN - 1) / kTN;
  const int kb = (K + kBK - 1) / kBK;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && kb / s < 6) break;
    const int items = tiles * s;
    const int rounds = (items + num_sms - 1) / num_sms;
    // time of one item in k-block units: its share of K, a fixed fill / drain / hand-over cost, and the atomics of
    // a split accumulation (M x 128 fp32 per item)
    const double item = (kb + s - 1) / s + 6.0 + (s > 1 ? M / 16.0 : 0.0);
    const double cost = rounds * item;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

cudaError_t launch_skinny_gemm(const SkinnyGemmArgs& a, cudaStream_t stream) {
  if (a.M < 1 || a.M > 256 || a.K % 8 != 0) return cudaErrorInvalidValue;
  if (a.all_reduce && a.N % 8 != 0) return cudaErrorInvalidValue;
  KP p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_n = (a.N + kTN - 1) / kTN;
  p.kb_total = (a.K + kBK - 1) / kBK;
  // stream-K partition: equal unit ranges over the CTAs.  splits == 0 keeps at least `min_units` k-blocks per CTA
  // (a shorter range does not pay for the pipeline fill and the split accumulation); splits >= 1 asks for about that
  // many pieces per tile.
  const int total_units = p.tiles_n * p.kb_total;
  const int num_ctas = a.num_ctas < 1 ? 1 : a.num_ctas;
  const int even = (total_units + num_ctas - 1) / num_ctas;
  static const int min_units = [] {
    const char* e = std::getenv("TDB200_SKINNY_MIN_UNITS");
    const int v = e ? std::atoi(e) : 8;
    return v < 1 ? 1 : v;
  }();
  const int want = a.splits >= 1 ? (p.kb_total + a.splits - 1) / a.splits : min_units;
  p.per_cta = even > want ? even : want;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.ld_out = a.ld_out;
  p.acc = a.acc;
  p.counters = a.counters;
  p.mode = a.all_reduce ? 1 : 0;
  p.use_mc = (a.use_multimem && a.symm.mc_base != 0) ? 1 : 0;
  p.partial = reinterpret_cast<__nv_bfloat16*>(a.partial);
  p.m_cap = a.m_cap;
  p.partial_half = p.use_mc ? static_cast<uint64_t>(a.m_cap) * a.N : static_cast<uint64_t>(a.symm.world) * a.m_cap * a.N;
  p.flags = a.flags;
  p.max_tiles = a.max_tiles;
  p.ctx = a.ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &a.symm, sizeof(SymmInfo));
  if ((p.per_cta < p.kb_total || p.per_cta % p.kb_total != 0 || p.mode == 1) && (a.acc == nullptr || a.counters == nullptr))
    return cudaErrorInvalidValue;
  if (p.mode == 1 && (p.tiles_n > a.max_tiles || a.M > a.m_cap || a.ctx == nullptr)) return cudaErrorInvalidValue;
  // form: without an explicit split count, the cluster kernel when the column tiles fit into one wave of clusters
  // (every CTA of a cluster gets at least four k-blocks); else, with splits >= 1 or with TDB200_SKINNY_FORM=1, the
  // stream-K kernel.  TDB200_SKINNY_CLUSTER_S fixes the cluster size, TDB200_SKINNY_CLUSTER_NT the tile width in
  // units of 128 columns (1 to 4).
  static const int form = [] {
    const char* e = std::getenv("TDB200_SKINNY_FORM");
    return e ? std::atoi(e) : 0;
  }();
  static const int env_s = [] {
    const char* e = std::getenv("TDB200_SKINNY_CLUSTER_S");
    return e ? std::atoi(e) : 0;
  }();
  static const int env_nt = [] {
    const char* e = std::getenv("TDB200_SKINNY_CLUSTER_NT");
    return e ? std::atoi(e) : 0;
  }();
  // an explicit (tile width, cluster size) of the caller, e.g. from the tuned table, comes before the environment; when
  // it cannot run (clusters not co-resident, accumulators or part too large), the launch fails instead of silently
  // running another form
  const bool explicit_cfg = a.cluster_nt >= 1 && a.cluster_s >= 1;
  const int force_nt = explicit_cfg ? a.cluster_nt : env_nt;
  const int force_s = explicit_cfg ? a.cluster_s : env_s;
  p.cluster_s = 0;
  p.bulk_exchange = a.bulk_exchange;
  if (form != 1 && a.splits < 1 && a.N % 4 == 0) {
    bool launched = false, whole_tiles = false;
    cudaError_t e;
    switch (skinny_gemm_mpad(a.M)) {
      case 16: e = launch_cluster_form<16>(a, p, num_ctas, force_s, force_nt, explicit_cfg, stream, &launched, &whole_tiles); break;
      case 32: e = launch_cluster_form<32>(a, p, num_ctas, force_s, force_nt, explicit_cfg, stream, &launched, &whole_tiles); break;
      case 64: e = launch_cluster_form<64>(a, p, num_ctas, force_s, force_nt, explicit_cfg, stream, &launched, &whole_tiles); break;
      case 128: e = launch_cluster_form<128>(a, p, num_ctas, force_s, force_nt, explicit_cfg, stream, &launched, &whole_tiles); break;
      case 256: e = launch_cluster_form<256>(a, p, num_ctas, force_s, force_nt, explicit_cfg, stream, &launched, &whole_tiles); break;
      default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess || launched) return e;
    if (explicit_cfg) return cudaErrorInvalidConfiguration;
    // one CTA per tile was the best the cluster form could offer: the stream-K kernel with unsplit tiles does the same
    // work with a shorter epilogue
    if (whole_tiles && skinny_gemm_mpad(a.M) >= 64) p.per_cta = even > p.kb_total ? even : p.kb_total;
  }
  const int grid = (total_units + p.per_cta - 1) / p.per_cta;
  switch (skinny_gemm_mpad(a.M)) {
    case 16: return launch_t<16>(a, p, grid, stream);
    case 32: return launch_t<32>(a, p, grid, stream);
    case 64: return launch_t<64>(a, p, grid, stream);
    case 128: return launch_t<128>(a, p, grid, stream);
    case 256: return launch_t<256>(a, p, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace tdb
