// Block-scaled fp8 (e4m3) GEMM for sm_100a on CTA pairs, with the same two fused tensor-parallel forms as the bf16
// kernel:
//
//   C[m, n] = sum over 128-wide K blocks kb of  a_s[m, kb] * b_s[n / 128, kb] * sum_k A8[m, k] * B8[n, k]
//
// A8 [M, K] e4m3 with one fp32 scale per row and 128-wide K block (1 x 128), B8 [N, K] e4m3 with one scale per
// 128 x 128 block - the recipe of the reference's fp8 payloads (tutorials/04-deepseek-infer-all2all.py:185-215:
// scale = amax / 448, group size 128).  Accumulation order: every K block is multiplied on the tensor core into a
// fresh fp32 accumulator in TMEM (tcgen05.mma.kind::f8f6f4, cta_group::2, 256 x 256 x 32 per instruction, four per
// block), and promoted by CUDA cores: eight epilogue warps per CTA read the block's partial sums with tcgen05.ld,
// multiply by the two scales and add them to the tile's accumulators, which live in registers (128 per thread).
// Two partial buffers of 256 TMEM columns alternate, so the tensor core works on block kb + 1 while block kb is
// promoted.
//
// Roles inside a CTA (384 threads = three warp groups): warp 0 = TMA producer, warp 1 = MMA issuer (CTA 0 of the
// pair) and TMEM owner, warps 2-3 idle; warps 4-11 = promotion + epilogue; warp w owns TMEM lanes 32 (w % 4) .. +32,
// warps 4-7 the tile's columns 0-127 and warps 8-11 columns 128-255.  setmaxnreg moves registers from the first warp
// group (40 per thread) to the epilogue groups (232 per thread).  Barriers:
//   full[s]        in CTA 0, count 1 (+ 64 KB of transactions from both CTAs' loads)
//   empty[s]       in each CTA, count 1: committed by CTA 0 after the MMAs that read stage s
//   part_full[b]   in each CTA, count 1: committed by CTA 0 after the four MMAs of a K block
//   part_empty[b]  in CTA 0, count 16: one arrival per epilogue warp of both CTAs once it has read buffer b
//
// all-gather mode: A and its scales are sharded by rows; comm CTAs of the launch push the local fp8 rows and their
// scales into every rank's workspace (half the NVLink bytes of the bf16 op) and raise one flag per 128-row chunk.
// reduce-scatter mode: bf16 partial tiles go straight into the owner rank's slot with per 128 x 128 unit flags; the
// own segment (computed last) adds the arrived partials to its register accumulators and writes the output.
// TMA loads read local memory only and carry no multicast qualifier; every wait is bounded.
#include <cuda.h>

#include "tdb/api.h"
#include "tdb/launch.cuh"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kBM = 128;
constexpr int kBKB = 128;       // K per stage: 128 e4m3 values = 128 bytes = one swizzle row = one scale block
constexpr int kUmmaKB = 32;     // K of one tcgen05.mma kind::f8f6f4
constexpr int kBN = 256;
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = 32 * kEpiWarps;
constexpr int kThreads = 128 + kEpiThreads;  // 384: warp group 0 = producer, MMA issuer and two idle warps
constexpr int kRegsControl = 40;             // registers per thread of warp group 0 after setmaxnreg
constexpr int kRegsEpilogue = 232;           // ... of the two epilogue warp groups (128 accumulators + a chunk)
constexpr int kGroupM = 8;
constexpr int kStages = 5;
constexpr int kABytes = kBM * kBKB;          // 16 KB: this CTA's 128 rows of A
constexpr int kBBytes = 128 * kBKB;          // 16 KB: this CTA's half of the 256-row B tile
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStgBoxBytes = kBM * 64 * 2;   // one TMA-store box: 128 rows x 64 bf16 columns, 128-byte swizzle
constexpr int kStgOffset = kStages * kStageBytes;          // staging of a whole 128 x 256 bf16 tile (four boxes)
constexpr int kBarOffset = kStgOffset + 4 * kStgBoxBytes;
constexpr int kSmemTotal = kBarOffset + (2 * kStages + 4) * 8 + 16;

// comm CTA ring (same dynamic shared memory)
constexpr int kPushPiece = 32 * 1024;
constexpr int kPushSlots = 6;
constexpr int kPushAhead = 4;
static_assert(kPushSlots * kPushPiece + kPushSlots * 8 <= kSmemTotal, "push ring must fit the kernel's shared memory");

enum StatSlot : int { kStatProdFlagWait = 0, kStatProdEmptyWait = 1, kStatMmaFullWait = 2, kStatMmaTmemWait = 3,
                      kStatEpiTmemWait = 4, kStatEpiFlagWait = 5, kStatEpiStoreWait = 6, kStatTotal = 7, kStatSlots = 8 };

struct PeerMaps {
  CUtensorMap m[kMaxRanks];
};

struct F8Params {
  int mode;
  int M, N, K;
  int num_kb;            // K / 128
  int n_blocks;          // ceil(N / 128): rows of b_scales
  __nv_bfloat16* c;
  int64_t ldc;
  const float* a_scales;   // [M, num_kb] (plain / reduce-scatter)
  const float* b_scales;   // [n_blocks, num_kb]
  int tiles_m_seg, tiles_n, num_seg, seg_first, seg_rows, n_comm;
  // all-gather
  const uint8_t* a_local;
  const float* a_scales_local;
  uint8_t* ag_ws;            // heap [2][world * max_seg_rows][K] e4m3
  float* ag_ws_scales;       // heap [2][world * max_seg_rows][num_kb]
  uint64_t ag_buf_rows;      // world * max_seg_rows
  uint32_t* ag_flags;        // heap [2][world][max_chunks]
  int max_chunks;
  // reduce-scatter
  __nv_bfloat16* rs_slots;   // heap [2][world][max_seg_rows][N]
  uint64_t rs_slot_elems;
  uint32_t* rs_flags;        // heap [2][world][max_tiles], one per 128 x 128 unit
  int max_tiles;
  __nv_bfloat16* rs_out;
  int64_t ld_out;
  CtxDev* ctx;
  SymmInfo symm;
  uint64_t mbar_timeout_ns;
  unsigned long long* stats;
};

struct StallTimer {
  long long t0;
  bool on;
  TDB_DEVICE explicit StallTimer(const F8Params& p) : t0(0), on(p.stats != nullptr) {
    if (on) t0 = clock64();
  }
  TDB_DEVICE void stop(long long& acc) {
    if (on) acc += clock64() - t0;
  }
};
TDB_DEVICE void stat_flush(const F8Params& p, int slot, long long v) {
  if (p.stats != nullptr && v != 0)
    atomicAdd(p.stats + static_cast<uint64_t>(blockIdx.x) * kStatSlots + slot, static_cast<unsigned long long>(v));
}

struct PairTile {
  int seg, mt, nt, n0;
};
// Tile order: segments starting at seg_first, inside a segment groups of kGroupM pair rows swept over all columns
// (the same order as the bf16 pair kernel); r.mt is the pair-row index (256 rows).
__device__ __forceinline__ PairTile decode_tile(const F8Params& p, int t, int tiles_m_pair) {
  PairTile r;
  const int per_seg = tiles_m_pair * p.tiles_n;
  const int si = t / per_seg;
  const int rem = t - si * per_seg;
  r.seg = (p.seg_first + si) % p.num_seg;
  const int group_sz = kGroupM * p.tiles_n;
  const int g = rem / group_sz;
  const int first_m = g * kGroupM;
  const int gm = min(tiles_m_pair - first_m, kGroupM);
  const int in_g = rem - g * group_sz;
  r.mt = first_m + in_g % gm;
  r.nt = in_g / gm;
  r.n0 = r.nt * kBN;
  return r;
}

TDB_DEVICE void epi_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// ---------------------------------------------------------------------------
// All-gather push of a comm CTA: one thread drives a ring of shared-memory slots (bulk load local -> shared, bulk
// store shared -> the peer's workspace).  A chunk is 128 rows and has two extents, the fp8 rows and their scales;
// its flag on the destination follows once the store group of its last piece has completed.  Destinations are
// visited nearest consumer first.
// ---------------------------------------------------------------------------
__device__ void ag_push(const F8Params& p, uint32_t epoch, uint8_t* smem) {
  if (threadIdx.x != 0) return;
  const int buf = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int chunks = (p.seg_rows + kBM - 1) / kBM;
  const uint64_t ext_row_bytes[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.num_kb) * 4};
  const char* ext_src[2] = {reinterpret_cast<const char*>(p.a_local), reinterpret_cast<const char*>(p.a_scales_local)};
  char* ext_dst[2] = {
      reinterpret_cast<char*>(p.ag_ws) + (static_cast<uint64_t>(buf) * p.ag_buf_rows + static_cast<uint64_t>(rank) * p.seg_rows) * ext_row_bytes[0],
      reinterpret_cast<char*>(p.ag_ws_scales) + (static_cast<uint64_t>(buf) * p.ag_buf_rows + static_cast<uint64_t>(rank) * p.seg_rows) * ext_row_bytes[1]};
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPushSlots * kPushPiece);
  for (int i = 0; i < kPushSlots; ++i) mbar_init(&bars[i], 1);
  fence_mbar_init();

  const int my_chunks = chunks > static_cast<int>(blockIdx.x) ? (chunks - blockIdx.x + p.n_comm - 1) / p.n_comm : 0;
  auto ext_bytes = [&](int ordinal, int e) -> uint64_t {
    const int c = blockIdx.x + ordinal * p.n_comm;
    return static_cast<uint64_t>(min(kBM, p.seg_rows - c * kBM)) * ext_row_bytes[e];
  };
  uint64_t total_pieces = 0;
  for (int o = 0; o < my_chunks; ++o)
    for (int e = 0; e < 2; ++e) total_pieces += (ext_bytes(o, e) + kPushPiece - 1) / kPushPiece;
  total_pieces *= (W - 1);

  struct Cursor {
    int d, c, e;
    uint64_t off;
  };
  Cursor ld = {1, 0, 0, 0}, st = {1, 0, 0, 0};
  // returns true when the piece just consumed was the last one of its chunk
  auto advance = [&](Cursor& cu, uint32_t bytes) -> bool {
    cu.off += bytes;
    if (cu.off < ext_bytes(cu.c, cu.e)) return false;
    cu.off = 0;
    if (++cu.e < 2) return false;
    cu.e = 0;
    if (++cu.c >= my_chunks) {
      cu.c = 0;
      ++cu.d;
    }
    return true;
  };
  auto piece_bytes = [&](const Cursor& cu) -> uint32_t {
    const uint64_t left = ext_bytes(cu.c, cu.e) - cu.off;
    return static_cast<uint32_t>(left < static_cast<uint64_t>(kPushPiece) ? left : static_cast<uint64_t>(kPushPiece));
  };
  uint32_t ld_i = 0, st_i = 0;
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
      const int c = blockIdx.x + ld.c * p.n_comm;
      const uint32_t bytes = piece_bytes(ld);
      const char* src = ext_src[ld.e] + static_cast<uint64_t>(c) * kBM * ext_row_bytes[ld.e] + ld.off;
      mbar_arrive_expect_tx(&bars[slot], bytes);
      bulk_load(smem + slot * kPushPiece, src, bytes, &bars[slot]);
      ++ld_i;
      advance(ld, bytes);
    }
    if (step >= kPushAhead) {
      const int slot = st_i % kPushSlots;
      if (!mbar_wait(&bars[slot], (st_i / kPushSlots) & 1, nullptr, p.mbar_timeout_ns)) {
        report(p.symm, kTimeoutMbarrier, kKernelAgGemm, 41, -1, slot, 0, static_cast<int>(st_i));
        ok = false;
        break;
      }
      const int c = blockIdx.x + st.c * p.n_comm;
      const uint32_t bytes = piece_bytes(st);
      const int peer = (rank - st.d + W) % W;
      char* dst_local = ext_dst[st.e] + static_cast<uint64_t>(c) * kBM * ext_row_bytes[st.e] + st.off;
      bulk_store(symm_at(p.symm, dst_local, peer), smem + slot * kPushPiece, bytes);
      bulk_commit();
      ++st_i;
      if (advance(st, bytes)) {
        if (pend_n == kPend) {
          bulk_wait<0>();
          for (int j = 0; j < pend_n; ++j) raise_flag(pend_peer[j], pend_chunk[j]);
          pend_n = 0;
        }
        pend_group[pend_n] = st_i - 1;
        pend_peer[pend_n] = peer;
        pend_chunk[pend_n] = c;
        ++pend_n;
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_a_local, const __grid_constant__ PeerMaps peer_maps,
                     const F8Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* part_full = empty_bar + kStages;
  uint64_t* part_empty = part_full + 2;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(part_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int buf = epoch & 1;
  const long long cta_t0 = p.stats != nullptr ? clock64() : 0;

  const bool is_comm = (p.mode == kGemmAllGather) && (static_cast<int>(blockIdx.x) < p.n_comm);
  if (is_comm) {
    ag_push(p, epoch, smem);
  } else {
    if (threadIdx.x == 0) {
      for (int i = 0; i < kStages; ++i) {
        mbar_init(&full_bar[i], 1);
        mbar_init(&empty_bar[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&part_full[i], 1);
        mbar_init(&part_empty[i], 2 * kEpiWarps);
      }
      *abort_flag = 0;
      fence_mbar_init();
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      if (p.mode == kGemmAllGather) tma_prefetch_desc(&tmap_a_local);
    }
    if (warp == 1) {
      tmem_alloc_pair(tmem_base_smem, 2 * kBN);
      tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_smem;
    const int n_pairs = (gridDim.x - p.n_comm) / 2;
    const int pair_idx = (blockIdx.x - p.n_comm) / 2;
    const int tiles_m_pair = (p.tiles_m_seg + 1) / 2;
    const int num_tiles = p.num_seg * tiles_m_pair * p.tiles_n;
    const int num_kb = p.num_kb;
    const int tiles_n128 = (p.N + 127) / 128;

    if (warp < 4) {
      // warp group 0 gives registers away; the two epilogue warp groups take them (each branch starts with its own
      // setmaxnreg so the compiler allocates every role against its own limit)
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer (both CTAs, own operand halves)
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        long long w_flag = 0, w_empty = 0;
        for (int t = pair_idx; t < num_tiles && ok; t += n_pairs) {
          const PairTile tl = decode_tile(p, t, tiles_m_pair);
          const int mt = 2 * tl.mt + static_cast<int>(cr);
          const bool valid_m = mt < p.tiles_m_seg;
          const bool local_seg = (p.mode == kGemmAllGather) && tl.seg == p.symm.rank;
          if (p.mode == kGemmAllGather && !local_seg && valid_m) {
            StallTimer st(p);
            const uint32_t* flag = p.ag_flags + (static_cast<uint64_t>(buf) * p.symm.world + tl.seg) * p.max_chunks + mt;
            ok = wait_until(p.symm, flag, epoch, kCmpGe, kKernelAgGemm, 5, tl.seg, mt);
            st.stop(w_flag);
            if (!ok) break;
            fence_proxy_async();
          }
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_try_wait(&empty_bar[s], ph ^ 1)) {
              StallTimer st(p);
              const bool got = mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.mbar_timeout_ns);
              st.stop(w_empty);
              if (!got) {
                ok = false;
                report(p.symm, kTimeoutMbarrier, kKernelGemm, 210, -1, s, (int)ph, t);
                break;
              }
            }
            uint8_t* sa = smem + s * kStageBytes;
            uint8_t* sb = sa + kABytes;
            const uint32_t full0 = mapa_u32(smem_u32(&full_bar[s]), 0);
            if (cr == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * kStageBytes);
            if (local_seg) {
              tma_load_3d_pair(sa, &tmap_a_local, full0, kb * kBKB, mt * kBM, 0);
            } else {
              tma_load_3d_pair(sa, &tmap_a, full0, kb * kBKB, tl.seg * p.seg_rows + mt * kBM,
                               (p.mode == kGemmAllGather) ? buf : 0);
            }
            tma_load_3d_pair(sb, &tmap_b, full0, kb * kBKB, tl.n0 + static_cast<int>(cr) * 128, 0);
          }
        }
        stat_flush(p, kStatProdFlagWait, w_flag);
        stat_flush(p, kStatProdEmptyWait, w_empty);
        if (!ok) {
          *abort_flag = 1;
          const uint64_t t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 2000000ull) nanosleep(1000);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (CTA 0 of the pair only)
      if (lane == 0 && cr == 0) {
        constexpr uint32_t idesc = make_idesc(0u, 2 * kBM, kBN);   // e4m3 x e4m3 -> fp32
        uint32_t it = 0, pc = 0;
        bool ok = true;
        long long w_full = 0, w_part = 0;
        for (int t = pair_idx; t < num_tiles && ok; t += n_pairs) {
          for (int kb = 0; kb < num_kb; ++kb, ++it, ++pc) {
            const int b = pc & 1;
            const uint32_t pph = (pc >> 1) & 1;
            if (!mbar_try_wait(&part_empty[b], pph ^ 1)) {
              StallTimer st(p);
              const bool got = mbar_wait(&part_empty[b], pph ^ 1, abort_flag, p.mbar_timeout_ns);
              st.stop(w_part);
              if (!got) {
                ok = false;
                report(p.symm, kTimeoutMbarrier, kKernelGemm, 220, -1, b, (int)pph, t);
                break;
              }
            }
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_try_wait(&full_bar[s], ph)) {
              StallTimer st(p);
              const bool got = mbar_wait(&full_bar[s], ph, abort_flag, p.mbar_timeout_ns);
              st.stop(w_full);
              if (!got) {
                ok = false;
                report(p.symm, kTimeoutMbarrier, kKernelGemm, 221, -1, s, (int)ph, t);
                break;
              }
            }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + b * kBN;
            const uint32_t sa = smem_u32(smem + s * kStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + kABytes);
#pragma unroll
            for (int k = 0; k < kBKB / kUmmaKB; ++k)
              umma_f8_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
            umma_commit_pair_mask(&empty_bar[s], 3);
            umma_commit_pair_mask(&part_full[b], 3);

          }
        }
        stat_flush(p, kStatMmaFullWait, w_full);
        stat_flush(p, kStatMmaTmemWait, w_part);
        if (!ok) *abort_flag = 1;
      }
    }
    } else {
      // ------------------------------------------------------------ promotion + epilogue (warps 4..11 of both CTAs)
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
      const int q = warp & 3;                 // TMEM lane quarter this warp may access
      const int half = (warp - 4) >> 2;       // which 128 columns of the tile
      const int et = threadIdx.x - 128;       // 0 .. 255
      const int row_in_tile = q * 32 + lane;
      const uint32_t part_empty0 = mapa_u32(smem_u32(&part_empty[0]), 0);
      const uint32_t part_empty1 = mapa_u32(smem_u32(&part_empty[1]), 0);
      uint32_t pc = 0;
      bool ok = true;
      long long w_part = 0, w_flag = 0;
      for (int t = pair_idx; t < num_tiles && ok; t += n_pairs) {
        const PairTile tl = decode_tile(p, t, tiles_m_pair);
        const int mt = 2 * tl.mt + static_cast<int>(cr);
        const bool valid_m = mt < p.tiles_m_seg;
        const int seg_row = mt * kBM + row_in_tile;
        const bool row_ok = valid_m && seg_row < p.seg_rows;
        const int col0 = tl.n0 + half * 128;              // first column this thread owns
        const int nblk = col0 >> 7;
        const bool col_ok = col0 < p.N;
        // scale rows of this thread
        const float* as_row = nullptr;
        if (row_ok) {
          if (p.mode == kGemmAllGather) {
            as_row = (tl.seg == p.symm.rank)
                         ? p.a_scales_local + static_cast<uint64_t>(seg_row) * num_kb
                         : p.ag_ws_scales + (static_cast<uint64_t>(buf) * p.ag_buf_rows +
                                             static_cast<uint64_t>(tl.seg) * p.seg_rows + seg_row) * num_kb;
          } else {
            as_row = p.a_scales + (static_cast<uint64_t>(tl.seg) * p.seg_rows + seg_row) * num_kb;
          }
        }
        const float* bs_row = col_ok ? p.b_scales + static_cast<uint64_t>(nblk) * num_kb : nullptr;

        float acc[128];
#pragma unroll
        for (int j = 0; j < 128; ++j) acc[j] = 0.f;
        const bool scaled = as_row != nullptr && bs_row != nullptr;
        float scale_next = 0.f;

        for (int kb = 0; kb < num_kb; ++kb, ++pc) {
          const int b = pc & 1;
          const uint32_t pph = (pc >> 1) & 1;
          {
            StallTimer st(p);
            const bool got = mbar_wait(&part_full[b], pph, abort_flag, p.mbar_timeout_ns);
            if (et == 0) st.stop(w_part);
            if (!got) {
              ok = false;
              if (lane == 0) report(p.symm, kTimeoutMbarrier, kKernelGemm, 230, -1, b, (int)pph, t);
              break;
            }
          }
          tc_fence_after_sync();
          // The scales of a remote segment were written by a peer before the chunk's flag.  Loads issued from here on
          // are ordered after that flag (producer's acquire -> TMA / MMA completion barriers -> the wait above), so
          // block 0's scales are read now and every later block's one iteration ahead, never before the first wait.
          const float scale = kb == 0 ? (scaled ? as_row[0] * bs_row[0] : 0.f) : scale_next;
          if (scaled && kb + 1 < num_kb) scale_next = as_row[kb + 1] * bs_row[kb + 1];
          const uint32_t t_part = tmem_base + b * kBN + half * 128 + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_part + c * 32, r);
            tmem_ld_wait();
            if (c == 3) {
              // This warp has read its share of the partial buffer: hand it back to the tensor core.  The ordering
              // that matters (TMEM reads before the next MMA overwrites them) is carried by the tcgen05 fence, so the
              // arrival is relaxed: a release at cluster scope would make the warp wait for all of its outstanding
              // memory operations once per K block.
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster_relaxed(b ? part_empty1 : part_empty0);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(r[j]), scale, acc[c * 32 + j]);
          }
        }
        if (!ok) break;

        // ------------------------------------------------------------ tile output
        const bool own_seg = (p.mode == kGemmReduceScatter) && tl.seg == p.symm.rank;
        const int unit0 = mt * tiles_n128 + (tl.n0 >> 7);
        const int n_units = min(2, tiles_n128 - (tl.n0 >> 7));
        if (own_seg) {
          // partial tiles of the other ranks for these rows must have arrived
          bool wok = true;
          if (valid_m && et < p.symm.world && et != p.symm.rank) {
            StallTimer st(p);
            const uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * p.symm.world + et) * p.max_tiles + unit0;
            for (int u = 0; u < n_units && wok; ++u)
              wok = wait_until(p.symm, flag + u, epoch, kCmpGe, kKernelGemmRs, 6, et, unit0 + u);
            if (et == (p.symm.rank + 1) % p.symm.world) st.stop(w_flag);
          }
          if (!wok) *abort_flag = 1;
          epi_bar();
          if (*abort_flag != 0) {
            ok = false;
            break;
          }
          if (row_ok && col_ok) {
            // 16 columns at a time: the 32-byte pieces of all other ranks' partials are requested together
            const int W = p.symm.world;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int cc = col0 + c * 16;
              uint4 u[kMaxRanks - 1][2];
#pragma unroll
              for (int i = 0; i < kMaxRanks - 1; ++i) {
                if (i < W - 1) {
                  const int src_rank = (p.symm.rank + 1 + i) % W;
                  const __nv_bfloat16* src = p.rs_slots + (static_cast<uint64_t>(buf) * W + src_rank) * p.rs_slot_elems +
                                             static_cast<uint64_t>(seg_row) * p.N + cc;
#pragma unroll
                  for (int j = 0; j < 2; ++j)
                    u[i][j] = (cc + 8 * j + 8 <= p.N) ? ld_relaxed_sys_v4(src + 8 * j) : make_uint4(0u, 0u, 0u, 0u);
                }
              }
#pragma unroll
              for (int i = 0; i < kMaxRanks - 1; ++i) {
                if (i < W - 1) {
#pragma unroll
                  for (int j = 0; j < 2; ++j) {
                    const float2 f0 = unpack_bf16x2(u[i][j].x), f1 = unpack_bf16x2(u[i][j].y),
                                 f2 = unpack_bf16x2(u[i][j].z), f3 = unpack_bf16x2(u[i][j].w);
                    float* a8 = &acc[c * 16 + 8 * j];
                    a8[0] += f0.x; a8[1] += f0.y; a8[2] += f1.x; a8[3] += f1.y;
                    a8[4] += f2.x; a8[5] += f2.y; a8[6] += f3.x; a8[7] += f3.y;
                  }
                }
              }
            }
          }
        }
        if (p.mode == kGemmReduceScatter && !own_seg) {
          // Partial tile for another rank: staged in shared memory in the 128-byte-swizzled box layout and written
          // into the owner's slot with four TMA stores (whole 128-byte lines over NVLink; 16-byte stores from
          // registers would cross the link as half-used sectors), then the tile's two unit flags.
          epi_bar();   // the leader is past the completion wait of the previous staged tile: the staging is free
          uint8_t* stg = smem + kStgOffset;
          const int sw = row_in_tile & 7;
#pragma unroll
          for (int cb = 0; cb < 2; ++cb) {
            uint8_t* srow = stg + (half * 2 + cb) * kStgBoxBytes + row_in_tile * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float* a8 = &acc[cb * 64 + 8 * j];
              uint4 o;
              o.x = pack_bf16x2(a8[0], a8[1]);
              o.y = pack_bf16x2(a8[2], a8[3]);
              o.z = pack_bf16x2(a8[4], a8[5]);
              o.w = pack_bf16x2(a8[6], a8[7]);
              *reinterpret_cast<uint4*>(srow + ((j ^ sw) << 4)) = o;
            }
          }
          fence_proxy_async_smem();
          epi_bar();
          if (et == 0 && valid_m) {
            const int c2 = buf * p.symm.world + p.symm.rank;
#pragma unroll
            for (int bx = 0; bx < 4; ++bx) {
              const int col = tl.n0 + bx * 64;
              if (col < p.N) tma_store_3d(&peer_maps.m[tl.seg], stg + bx * kStgBoxBytes, col, mt * kBM, c2);
            }
            bulk_commit();
            bulk_wait<0>();
            fence_proxy_async();
            fence_acq_rel_sys();
            uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * p.symm.world + p.symm.rank) * p.max_tiles + unit0;
            uint32_t* dst = symm_at(p.symm, flag, tl.seg);
            if (n_units == 2 && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
              st_release_sys_u64(reinterpret_cast<uint64_t*>(dst), (static_cast<uint64_t>(epoch) << 32) | epoch);
            } else {
              for (int u = 0; u < n_units; ++u) st_release_sys(dst + u, epoch);
            }
          }
        } else {
          // output rows of this rank (plain / all-gather result, or the reduce-scatter's own segment)
          __nv_bfloat16* dst_row = nullptr;
          if (row_ok && col_ok) {
            dst_row = own_seg ? p.rs_out + static_cast<uint64_t>(seg_row) * p.ld_out
                              : p.c + (static_cast<uint64_t>(tl.seg) * p.seg_rows + seg_row) * p.ldc;
          }
          if (dst_row != nullptr) {
            const bool vec_ok = (reinterpret_cast<uintptr_t>(dst_row + col0) & 15u) == 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int cc = col0 + 8 * j;
              if (cc + 8 <= p.N && vec_ok) {
                uint4 o;
                o.x = pack_bf16x2(acc[8 * j + 0], acc[8 * j + 1]);
                o.y = pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]);
                o.z = pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]);
                o.w = pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]);
                st_v4(dst_row + cc, o);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  if (cc + e < p.N) dst_row[cc + e] = __float2bfloat16(acc[8 * j + e]);
              }
            }
          }
        }
      }
      if (et == 0) stat_flush(p, kStatEpiTmemWait, w_part);
   // here: latency of the first pair of TMEM loads of every block
      stat_flush(p, kStatEpiFlagWait, w_flag);
      if (!ok) *abort_flag = 1;
      if (et == 0) bulk_wait<0>();   // shared memory stays valid until the last TMA store has read it
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, 2 * kBN);
    }
  }
  if (threadIdx.x == 0 && p.stats != nullptr) stat_flush(p, kStatTotal, clock64() - cta_t0);

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

}  // namespace

cudaError_t launch_gemm_fp8(const GemmFp8Args& a, cudaStream_t stream) {
  static_assert(kSmemTotal + 1024 <= 227 * 1024, "fp8 pair kernel exceeds the shared memory of an SM");
  const int smem = kSmemTotal + 1024;
  {
    static SmemOptIn opt_in;
    cudaError_t e = opt_in.ensure(gemm_fp8_pair_kernel, smem);
    if (e != cudaSuccess) return e;
  }
  if (a.K < kBKB || a.K % kBKB != 0) return cudaErrorInvalidValue;
  F8Params p;
  memset(&p, 0, sizeof(p));
  p.mode = a.mode;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.num_kb = a.K / kBKB;
  p.n_blocks = (a.N + 127) / 128;
  p.c = reinterpret_cast<__nv_bfloat16*>(a.c);
  p.ldc = a.ldc;
  p.a_scales = a.a_scales;
  p.b_scales = a.b_scales;
  const bool fused = a.mode != kGemmPlain;
  p.num_seg = fused ? a.symm.world : 1;
  p.seg_rows = fused ? a.seg_rows : a.M;
  p.tiles_m_seg = (p.seg_rows + kBM - 1) / kBM;
  p.tiles_n = (a.N + kBN - 1) / kBN;
  p.seg_first = a.mode == kGemmAllGather ? a.symm.rank
               : a.mode == kGemmReduceScatter ? (a.symm.rank + 1) % a.symm.world : 0;
  p.n_comm = a.mode == kGemmAllGather ? a.n_comm_ctas : 0;
  p.a_local = reinterpret_cast<const uint8_t*>(a.a_local);
  p.a_scales_local = a.a_scales_local;
  p.ag_ws = reinterpret_cast<uint8_t*>(a.ag_ws);
  p.ag_ws_scales = a.ag_ws_scales;
  p.ag_buf_rows = static_cast<uint64_t>(a.symm.world) * a.max_seg_rows;
  p.ag_flags = a.ag_flags;
  p.max_chunks = a.max_chunks;
  p.rs_slots = reinterpret_cast<__nv_bfloat16*>(a.rs_slots);
  p.rs_slot_elems = static_cast<uint64_t>(a.max_seg_rows) * a.N;
  p.rs_flags = a.rs_flags;
  p.max_tiles = a.max_tiles;
  p.rs_out = reinterpret_cast<__nv_bfloat16*>(a.rs_out);
  p.ld_out = a.ld_out;
  p.ctx = a.ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &a.symm, sizeof(SymmInfo));
  p.mbar_timeout_ns = a.symm.timeout_ns > 0 ? a.symm.timeout_ns : 4000000000ull;
  p.stats = reinterpret_cast<unsigned long long*>(a.stats);
  if (a.mode == kGemmAllGather) {
    if (p.tiles_m_seg > a.max_chunks) return cudaErrorInvalidValue;
    if ((p.n_comm & 1) != 0 || p.n_comm < 2 || p.n_comm > a.num_ctas - 2) return cudaErrorInvalidValue;
    // bulk copies move multiples of 16 bytes: the scale extent of the last (ragged) chunk must be one
    if ((static_cast<uint64_t>(p.seg_rows % kBM) * p.num_kb * 4) % 16 != 0) return cudaErrorInvalidValue;
  }
  if (a.mode == kGemmReduceScatter && p.tiles_m_seg * ((a.N + 127) / 128) > a.max_tiles) return cudaErrorInvalidValue;
  const int grid = a.num_ctas & ~1;
  if (grid - p.n_comm < 2) return cudaErrorInvalidValue;
  CUtensorMap ta, tb, tl;
  memcpy(&ta, a.tmap_a.bytes, sizeof(CUtensorMap));
  memcpy(&tb, a.tmap_b.bytes, sizeof(CUtensorMap));
  memcpy(&tl, a.tmap_a_local.bytes, sizeof(CUtensorMap));
  PeerMaps pm;
  memcpy(&pm, a.tmap_peer_c, sizeof(PeerMaps));
  gemm_fp8_pair_kernel<<<grid, kThreads, smem, stream>>>(ta, tb, tl, pm, p);
  return cudaGetLastError();
}

}  // namespace tdb
