// Persistent, warp-specialised tcgen05 GEMM for sm_100a and its two fused
// tensor-parallel forms:
//
//   plain           C[M,N] = A[M,K] * B[N,K]^T
//   all-gather      A is sharded by rows over the ranks; "comm" CTAs of the same
//                   launch push the local shard into every rank's workspace with
//                   bulk-TMA copies (local memory -> shared memory -> peer memory,
//                   nearest consumer first) or NVLS multimem.st, and set a
//                   per-chunk epoch flag; GEMM CTAs wait for exactly the chunk a
//                   tile needs, then TMA-load it from LOCAL memory.
//   reduce-scatter  every rank computes a partial C; the epilogue TMA-stores each
//                   tile straight into the owner rank's slot over NVLink and sets
//                   a per-tile epoch flag there; after its last tile every CTA
//                   joins the owner-side reduction of the arrived slots (single-CTA
//                   kernel), or the own segment's epilogue sums the arrived partials
//                   into its accumulators (CTA-pair kernel).
//
// Roles inside a CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer
// (one elected lane) and TMEM owner, warps 2-5 = epilogue: TMEM -> registers ->
// bf16 -> swizzled shared-memory staging -> TMA store (local or peer memory).
// Accumulators are double-buffered in TMEM (2 x BLOCK_N fp32 columns) so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Reference behaviour being matched (not its code):
//   AG+GEMM   python/triton_dist/kernels/nvidia/allgather_gemm.py:159-264 (consumer GEMM waits per rank
//             segment, local segment first) and allgather.py:106-137 (producer + ready flags)
//   GEMM+RS   python/triton_dist/kernels/nvidia/gemm_reduce_scatter.py:122-250 (tile order starts at the
//             next rank's segment, `fuse_scatter` epilogue writes into the owner's buffer :235-248)
//             and reduce_scatter.py:674-815 (local reduction over the W slots)
// Flags hold the call epoch (kept in device memory and bumped by the last CTA),
// buffers alternate by epoch parity, so nothing is reset and no barrier is needed
// between calls; every wait is bounded and reports through the status page.
#include <cuda.h>

#include "tdb/api.h"
#include "tdb/launch.cuh"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kGroupM = 8;
constexpr int kEpiCols = 64;      // columns per epilogue staging buffer (128-byte rows)
constexpr int kEpiBytes = kBM * kEpiCols * 2;
// Slots of the optional per-CTA stall counters (KParams::stats, SM clock cycles).
enum StatSlot : int {
  kStatProdFlagWait = 0,   // producer: all-gather chunk flags
  kStatProdEmptyWait = 1,  // producer: ring slots held by the tensor core
  kStatMmaFullWait = 2,    // MMA issuer: operands not yet in shared memory
  kStatMmaTmemWait = 3,    // MMA issuer: accumulator buffer still owned by the epilogue
  kStatEpiTmemWait = 4,    // epilogue: accumulator not finished
  kStatEpiFlagWait = 5,    // epilogue: partial tiles of the other ranks (reduce-scatter, own segment)
  kStatEpiStoreWait = 6,   // epilogue: TMA stores in flight (staging reuse / completion before a flag)
  kStatTotal = 7,          // CTA lifetime
  kStatSlots = 8,
};

template <int BN>
struct SmemLayout {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;          // 2 staging buffers, 1024-aligned
  static constexpr int kBarOffset = kEpiOffset + 2 * kEpiBytes;
  // full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], tmem_base, abort
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 16;
};

// ring used by the comm CTAs of the all-gather mode (same dynamic shared memory)
constexpr int kPushPiece = 32 * 1024;
constexpr int kPushSlots = 7;
constexpr int kPushAhead = 5;

struct PeerMaps {
  CUtensorMap m[kMaxRanks];
};

struct KParams {
  int mode;
  int M, N, K;
  __nv_bfloat16* c;
  int64_t ldc;
  int tiles_m_seg;   // M tiles per segment
  int tiles_n;
  int num_seg;
  int seg_first;     // first segment in this rank's tile order
  int seg_rows;
  int n_comm;
  int tma_store;     // epilogue through shared memory + TMA store
  // all-gather
  const __nv_bfloat16* a_local;
  __nv_bfloat16* ag_ws;
  uint64_t ag_buf_elems;   // elements between the two workspace buffers
  uint32_t* ag_flags;
  int max_chunks;
  int use_mc;
  // reduce-scatter
  __nv_bfloat16* rs_slots;
  uint64_t rs_slot_elems;  // elements per (buffer, source) slot
  uint32_t* rs_flags;
  int max_tiles;
  __nv_bfloat16* rs_out;
  int64_t ld_out;
  const int32_t* tile_expert;   // grouped GEMM: expert (third coordinate of B) of every M tile, < 0 = skip the tile
  CtxDev* ctx;
  SymmInfo symm;
  uint64_t mbar_timeout_ns;     // limit of every shared-memory barrier wait
  uint32_t epi_sleep_ns;        // pair kernel: sleep between polls of an epilogue warp waiting for its accumulator
  int pair_group_m;             // pair kernel: M tiles (of 256 rows) swept together over all columns
  int split_tail;               // pair kernel: tiles of an incomplete last wave are computed as two 128-column halves
  unsigned long long* stats;    // optional [grid][kStatSlots] stall counters (cycles), null = off
};

// Accumulates the cycles spent between construction and stop() into a stall counter (no-op when stats are off).
struct StallTimer {
  long long t0;
  bool on;
  TDB_DEVICE explicit StallTimer(const KParams& p) : t0(0), on(p.stats != nullptr) {
    if (on) t0 = clock64();
  }
  TDB_DEVICE void stop(long long& acc) {
    if (on) acc += clock64() - t0;
  }
};
TDB_DEVICE void stat_flush(const KParams& p, int slot, long long v) {
  if (p.stats != nullptr && v != 0)
    atomicAdd(p.stats + static_cast<uint64_t>(blockIdx.x) * kStatSlots + slot, static_cast<unsigned long long>(v));
}

struct Tile {
  int seg, mt, nt, m0, n0, m_end;
};

__device__ __forceinline__ Tile decode_tile(const KParams& p, int t, int BN) {
  Tile r;
  const int per_seg = p.tiles_m_seg * p.tiles_n;
  const int si = t / per_seg;
  const int rem = t - si * per_seg;
  r.seg = (p.seg_first + si) % p.num_seg;
  const int group_sz = kGroupM * p.tiles_n;
  const int g = rem / group_sz;
  const int first_m = g * kGroupM;
  const int gm = min(p.tiles_m_seg - first_m, kGroupM);
  const int in_g = rem - g * group_sz;
  r.mt = first_m + in_g % gm;
  r.nt = in_g / gm;
  r.m0 = r.seg * p.seg_rows + r.mt * kBM;
  r.n0 = r.nt * BN;
  r.m_end = min(p.M, (r.seg + 1) * p.seg_rows);
  return r;
}

// ---------------------------------------------------------------------------
// All-gather push, NVLS flavour: SM-issued multimem.st (one store reaches all ranks).
// ---------------------------------------------------------------------------
__device__ void ag_push_multimem(const KParams& p, uint32_t epoch) {
  const int buf = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int chunks = (p.seg_rows + kBM - 1) / kBM;
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * 2;
  char* ws_local = reinterpret_cast<char*>(p.ag_ws + buf * p.ag_buf_elems);
  for (int c = blockIdx.x; c < chunks; c += p.n_comm) {
    const int r0 = c * kBM;
    const int rows = min(kBM, p.seg_rows - r0);
    const uint64_t nvec = (rows * row_bytes) >> 4;
    const char* src = reinterpret_cast<const char*>(p.a_local) + r0 * row_bytes;
    char* dst = mc_ptr(p.symm, ws_local + (static_cast<uint64_t>(rank) * p.seg_rows + r0) * row_bytes);
    uint64_t i = threadIdx.x;
    for (; i + 3ull * kThreads < nvec; i += 4ull * kThreads) {
      uint4 v0 = ld_nc_v4(src + (i << 4));
      uint4 v1 = ld_nc_v4(src + ((i + kThreads) << 4));
      uint4 v2 = ld_nc_v4(src + ((i + 2 * kThreads) << 4));
      uint4 v3 = ld_nc_v4(src + ((i + 3 * kThreads) << 4));
      multimem_st_v4(dst + (i << 4), v0);
      multimem_st_v4(dst + ((i + kThreads) << 4), v1);
      multimem_st_v4(dst + ((i + 2 * kThreads) << 4), v2);
      multimem_st_v4(dst + ((i + 3 * kThreads) << 4), v3);
    }
    for (; i < nvec; i += kThreads) multimem_st_v4(dst + (i << 4), ld_nc_v4(src + (i << 4)));
    __syncthreads();
    if (threadIdx.x < W) {
      // every lane orders the CTA's stores (made visible to it by the barrier) before its own flag store
      fence_acq_rel_sys();
      uint32_t* flag = p.ag_flags + (static_cast<uint64_t>(buf) * W + rank) * p.max_chunks + c;
      st_release_sys(symm_at(p.symm, flag, (rank + threadIdx.x) % W), epoch);
    }
  }
}

// ---------------------------------------------------------------------------
// All-gather push, bulk-TMA flavour: one thread drives a ring of shared-memory
// slots: bulk load (local A -> smem), bulk store (smem -> the peer's workspace).
// Destinations are visited nearest consumer first: rank r's shard is the d-th
// segment rank (r - d) computes, so it goes to (r - 1), (r - 2), ... in turn and
// every receiver takes in one source at full link rate at a time.
// ---------------------------------------------------------------------------
__device__ void ag_push_bulk(const KParams& p, uint32_t epoch, uint8_t* smem) {
  if (threadIdx.x != 0) return;
  const int buf = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int chunks = (p.seg_rows + kBM - 1) / kBM;
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * 2;
  char* ws_local = reinterpret_cast<char*>(p.ag_ws + buf * p.ag_buf_elems);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPushSlots * kPushPiece);
  for (int i = 0; i < kPushSlots; ++i) mbar_init(&bars[i], 1);
  fence_mbar_init();

  // work list of this CTA: for d in 1..W-1 (the GEMM reads the local shard in place), for its chunks, for the
  // pieces of a chunk
  const int my_chunks = chunks > static_cast<int>(blockIdx.x) ? (chunks - blockIdx.x + p.n_comm - 1) / p.n_comm : 0;
  uint32_t ld_i = 0, st_i = 0;                 // pieces loaded / stored so far (global counters over the ring)
  int ld_d = 1, ld_c = 0;
  uint64_t ld_off = 0;                          // load cursor: (distance, chunk ordinal, byte offset in chunk)
  int st_d = 1, st_c = 0;
  uint64_t st_off = 0;                          // store cursor
  // flags whose chunk has been committed but not yet confirmed complete (raised two groups later, so the
  // pipeline never drains in the middle)
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
  auto chunk_bytes = [&](int ordinal) -> uint64_t {
    const int c = blockIdx.x + ordinal * p.n_comm;
    return static_cast<uint64_t>(min(kBM, p.seg_rows - c * kBM)) * row_bytes;
  };
  const uint64_t total_pieces = [&]() {
    uint64_t n = 0;
    for (int o = 0; o < my_chunks; ++o) n += (chunk_bytes(o) + kPushPiece - 1) / kPushPiece;
    return n * (W - 1);
  }();
  for (uint64_t step = 0; step < total_pieces + kPushAhead && ok; ++step) {
    if (step < total_pieces) {
      // ---- issue the load of piece `ld_i`
      const int slot = ld_i % kPushSlots;
      // the store that last read this slot is at most (kPushSlots - kPushAhead - 1) groups behind the newest
      bulk_wait_read<kPushSlots - kPushAhead - 1>();
      const int c = blockIdx.x + ld_c * p.n_comm;
      const uint64_t cb = chunk_bytes(ld_c);
      const uint32_t bytes = static_cast<uint32_t>((cb - ld_off) < (uint64_t)kPushPiece ? (cb - ld_off) : (uint64_t)kPushPiece);
      const char* src = reinterpret_cast<const char*>(p.a_local) + static_cast<uint64_t>(c) * kBM * row_bytes + ld_off;
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
      // ---- store piece `st_i`
      const int slot = st_i % kPushSlots;
      if (!mbar_wait(&bars[slot], (st_i / kPushSlots) & 1, nullptr, p.mbar_timeout_ns)) {
        report(p.symm, kTimeoutMbarrier, kKernelAgGemm, 40, -1, slot, 0, static_cast<int>(st_i));
        ok = false;
        break;
      }
      const int c = blockIdx.x + st_c * p.n_comm;
      const uint64_t cb = chunk_bytes(st_c);
      const uint32_t bytes = static_cast<uint32_t>((cb - st_off) < (uint64_t)kPushPiece ? (cb - st_off) : (uint64_t)kPushPiece);
      const int peer = (rank - st_d + W) % W;
      char* dst_local = ws_local + (static_cast<uint64_t>(rank) * p.seg_rows + static_cast<uint64_t>(c) * kBM) * row_bytes + st_off;
      bulk_store(symm_at(p.symm, dst_local, peer), smem + slot * kPushPiece, bytes);
      bulk_commit();
      ++st_i;
      st_off += bytes;
      if (st_off >= cb) {
        // last piece of this chunk for `peer` committed as group st_i - 1: its flag follows once that group is done
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
      // groups older than the two newest are complete after wait_group 2
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
// All-gather push, NVLS ring flavour (CTA-pair kernel): every byte leaves this GPU once and the switch replicates it to
// all ranks, so a few comm CTAs are enough.  The comm CTAs work on the shard chunk by chunk TOGETHER: CTA i owns rows
// [i, i + 1) * 128 / n_comm of every 128-row chunk, so chunk c is complete everywhere before chunk c + 1 starts and the
// GEMM (which visits remote tiles chunk-major in this mode) never waits for the tail of a shard.  One thread streams
// the rows local memory -> shared memory with bulk copies through a ring of slots; all threads move a landed slot to
// the multicast address with multimem.st.  Flag (chunk, comm CTA) is raised on every rank after the CTA's rows.
// ---------------------------------------------------------------------------
__device__ void ag_push_mc_ring(const KParams& p, uint32_t epoch, uint8_t* smem) {
  const int buf = epoch & 1;
  const int W = p.symm.world, rank = p.symm.rank;
  const int tid = threadIdx.x;
  const int bi = blockIdx.x;
  const int chunks = (p.seg_rows + kBM - 1) / kBM;
  const int rows_per_cta = kBM / p.n_comm;          // n_comm divides 128 (checked on the host)
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * 2;
  char* ws_local = reinterpret_cast<char*>(p.ag_ws + buf * p.ag_buf_elems);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPushSlots * kPushPiece);
  __shared__ int s_ok;
  if (tid == 0) {
    for (int i = 0; i < kPushSlots; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
    s_ok = 1;
  }
  __syncthreads();
  // this CTA's byte range of chunk c: [lo, hi) relative to the chunk's first byte
  auto range = [&](int c, uint64_t* lo, uint64_t* hi) {
    const int rows_c = min(kBM, p.seg_rows - c * kBM);
    *lo = static_cast<uint64_t>(min(rows_c, bi * rows_per_cta)) * row_bytes;
    *hi = static_cast<uint64_t>(min(rows_c, (bi + 1) * rows_per_cta)) * row_bytes;
  };
  // piece cursor for loads (thread 0) and for the copy (all threads)
  struct Cur {
    int c;
    uint64_t off;
  };
  auto piece_of = [&](const Cur& cu, uint64_t* src_off, uint32_t* bytes) -> bool {   // false: past the end
    if (cu.c >= chunks) return false;
    uint64_t lo, hi;
    range(cu.c, &lo, &hi);
    const uint64_t left = hi - lo - cu.off;
    *bytes = static_cast<uint32_t>(left < static_cast<uint64_t>(kPushPiece) ? left : static_cast<uint64_t>(kPushPiece));
    *src_off = static_cast<uint64_t>(cu.c) * kBM * row_bytes + lo + cu.off;
    return true;
  };
  auto advance = [&](Cur& cu, uint32_t bytes) -> bool {   // true: that was the chunk's last piece
    uint64_t lo, hi;
    range(cu.c, &lo, &hi);
    cu.off += bytes;
    if (cu.off < hi - lo) return false;
    cu.off = 0;
    ++cu.c;
    return true;
  };
  auto skip_empty = [&](Cur& cu) {   // chunks in which this CTA has no rows (ragged last chunk)
    while (cu.c < chunks) {
      uint64_t lo, hi;
      range(cu.c, &lo, &hi);
      if (hi > lo) break;
      ++cu.c;
    }
  };
  Cur ld = {0, 0}, cp = {0, 0};
  uint32_t ld_i = 0, cp_i = 0;
  const char* src_base = reinterpret_cast<const char*>(p.a_local);
  char* dst_base = mc_ptr(p.symm, ws_local + static_cast<uint64_t>(rank) * p.seg_rows * row_bytes);
  auto issue_load = [&]() {   // thread 0
    skip_empty(ld);
    uint64_t so;
    uint32_t bytes;
    if (!piece_of(ld, &so, &bytes)) return;
    const int slot = ld_i % kPushSlots;
    mbar_arrive_expect_tx(&bars[slot], bytes);
    bulk_load(smem + slot * kPushPiece, src_base + so, bytes, &bars[slot]);
    ++ld_i;
    advance(ld, bytes);
  };
  if (tid == 0)
    for (int i = 0; i < kPushAhead; ++i) issue_load();
  // flags of chunks in which this CTA has no rows are raised as well, so that a consumer can wait for all n_comm
  auto raise = [&](int c) {
    if (tid < W) {
      fence_acq_rel_sys();
      uint32_t* flag = p.ag_flags + (static_cast<uint64_t>(buf) * W + rank) * p.max_chunks + c * p.n_comm + bi;
      st_release_sys(symm_at(p.symm, flag, (rank + tid) % W), epoch);
    }
  };
  int next_flag = 0;   // chunks below this one have been flagged
  while (true) {
    skip_empty(cp);
    uint64_t so;
    uint32_t bytes;
    if (!piece_of(cp, &so, &bytes)) break;
    const int slot = cp_i % kPushSlots;
    if (!mbar_wait(&bars[slot], (cp_i / kPushSlots) & 1, nullptr, p.mbar_timeout_ns)) {
      if (tid == 0) report(p.symm, kTimeoutMbarrier, kKernelAgGemm, 42, -1, slot, 0, static_cast<int>(cp_i));
      s_ok = 0;
    }
    __syncthreads();
    if (s_ok == 0) break;
    const uint8_t* sl = smem + slot * kPushPiece;
    char* dst = dst_base + so;
    const uint32_t nvec = bytes >> 4;
    for (uint32_t v = tid; v < nvec; v += kThreads)
      multimem_st_v4(dst + (static_cast<uint64_t>(v) << 4), *reinterpret_cast<const uint4*>(sl + (static_cast<uint64_t>(v) << 4)));
    const int c_done = cp.c;
    const bool last = advance(cp, bytes);
    ++cp_i;
    __syncthreads();           // the slot has been read by everyone; the CTA's stores of this piece are issued
    if (tid == 0) issue_load();
    if (last) {
      for (; next_flag <= c_done; ++next_flag) raise(next_flag);
    }
  }
  if (s_ok != 0)
    for (; next_flag < chunks; ++next_flag) raise(next_flag);
}

// Owner-side reduction of the reduce-scatter mode: out[rows of my segment] = sum over sources.
__device__ void rs_reduce(const KParams& p, uint32_t epoch, int BN) {
  const int buf = epoch & 1;
  const int W = p.symm.world;
  const int items = p.tiles_m_seg * p.tiles_n;
  const int vec_per_row = BN / 8;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int mt = it / p.tiles_n, nt = it - mt * p.tiles_n;
    bool ok = true;
    if (threadIdx.x < W) {
      const uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * W + threadIdx.x) * p.max_tiles + it;
      ok = wait_until(p.symm, flag, epoch, kCmpGe, kKernelGemmRs, 2, threadIdx.x, it);
    }
    ok = __syncthreads_and(ok);
    if (!ok) return;
    const int r0 = mt * kBM;
    const int rows = min(kBM, p.seg_rows - r0);
    const int n0 = nt * BN;
    const int total = rows * vec_per_row;
    for (int v = threadIdx.x; v < total; v += kThreads) {
      const int r = v / vec_per_row, cv = v - r * vec_per_row;
      const int col = n0 + cv * 8;
      if (col >= p.N) continue;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s = 0; s < W; ++s) {
        const __nv_bfloat16* src = p.rs_slots + (static_cast<uint64_t>(buf) * W + s) * p.rs_slot_elems +
                                   static_cast<uint64_t>(r0 + r) * p.N + col;
        const uint4 u = ld_relaxed_sys_v4(src);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                     f3 = unpack_bf16x2(u.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
        acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      st_v4(p.rs_out + static_cast<uint64_t>(r0 + r) * p.ld_out + col, o);
    }
  }
}

TDB_DEVICE void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ PeerMaps peer_maps,
            const __grid_constant__ CUtensorMap tmap_a_local, const KParams p) {
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to 1024
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int buf = epoch & 1;

  const bool is_comm = (p.mode == kGemmAllGather) && (static_cast<int>(blockIdx.x) < p.n_comm);
  if (is_comm) {
    if (p.use_mc) {
      ag_push_multimem(p, epoch);
    } else {
      ag_push_bulk(p, epoch, smem);
    }
  } else {
    // ------------------------------------------------------------------ setup
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
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      if (p.mode == kGemmAllGather) tma_prefetch_desc(&tmap_a_local);
      if (p.tma_store && p.mode != kGemmReduceScatter) tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) {
      tmem_alloc(tmem_base_smem, 2 * BN);
      tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_smem;

    const int n_gemm = gridDim.x - ((p.mode == kGemmAllGather) ? p.n_comm : 0);
    const int g_idx = blockIdx.x - ((p.mode == kGemmAllGather) ? p.n_comm : 0);
    const int num_tiles = p.num_seg * p.tiles_m_seg * p.tiles_n;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        uint32_t it = 0;
        uint32_t issued = 0;
        bool ok = true;
        for (int t = g_idx; t < num_tiles && ok; t += n_gemm) {
          const Tile tl = decode_tile(p, t, BN);
          const int expert = p.tile_expert ? __ldg(p.tile_expert + tl.mt) : 0;
          if (expert < 0) continue;
          // all-gather mode: the local shard is read where it is, remote shards from the workspace once they arrived
          const bool local_seg = (p.mode == kGemmAllGather) && tl.seg == p.symm.rank;
          if (p.mode == kGemmAllGather && !local_seg) {
            const uint32_t* flag = p.ag_flags + (static_cast<uint64_t>(buf) * p.symm.world + tl.seg) * p.max_chunks + tl.mt;
            ok = wait_until(p.symm, flag, epoch, kCmpGe, kKernelAgGemm, 1, tl.seg, tl.mt);
            if (!ok) break;
            fence_proxy_async();
          }
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.mbar_timeout_ns)) {
              ok = false;
              report(p.symm, kTimeoutMbarrier, kKernelGemm, 10, -1, s, (int)ph, t);
              break;
            }
            uint8_t* sa = smem + s * L::kStageBytes;
            uint8_t* sb = sa + L::kABytes;
            mbar_arrive_expect_tx(&full_bar[s], L::kStageBytes);
            if (local_seg) {
              tma_load_3d(sa, &tmap_a_local, &full_bar[s], kb * kBK, tl.mt * kBM, 0);
            } else {
              tma_load_3d(sa, &tmap_a, &full_bar[s], kb * kBK, tl.m0, (p.mode == kGemmAllGather) ? buf : 0);
            }
            tma_load_3d(sb, &tmap_b, &full_bar[s], kb * kBK, tl.n0, expert);
            ++issued;
          }
        }
        if (!ok) {
          *abort_flag = 1;
          // drain: every load already issued completes its full barrier on its own
          const uint32_t first = issued > (uint32_t)kStages ? issued - kStages : 0;
          for (uint32_t j = first; j < issued; ++j)
            mbar_wait(&full_bar[j % kStages], (j / kStages) & 1, nullptr, 200000000ull);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc(1u, kBM, BN);
        uint32_t it = 0;
        int local = 0;
        bool ok = true;
        for (int t = g_idx; t < num_tiles && ok; t += n_gemm) {
          if (p.tile_expert) {
            const Tile tl = decode_tile(p, t, BN);
            if (__ldg(p.tile_expert + tl.mt) < 0) continue;
          }
          const int b = local & 1;
          const uint32_t aph = (local >> 1) & 1;
          ++local;
          if (!mbar_wait(&tmem_empty[b], aph ^ 1, abort_flag, p.mbar_timeout_ns)) {
            ok = false;
            report(p.symm, kTimeoutMbarrier, kKernelGemm, 20, -1, b, (int)aph, t);
            break;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + b * BN;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_wait(&full_bar[s], ph, abort_flag, p.mbar_timeout_ns)) {
              ok = false;
              report(p.symm, kTimeoutMbarrier, kKernelGemm, 21, -1, s, (int)ph, t);
              break;
            }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              // advance 16 elements (32 bytes) along K inside the swizzle row: +2 in the >>4 address field
              umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty_bar[s]);
          }
          if (ok) umma_commit(&tmem_full[b]);
        }
        if (!ok) *abort_flag = 1;
      }
    } else {
      // ------------------------------------------------------------ epilogue (warps 2..5)
      const int q = warp & 3;  // TMEM lane quarter this warp may access
      const bool leader = (warp == 2 && lane == 0);
      uint8_t* stage_base = smem + L::kEpiOffset;
      const int row_in_tile = q * 32 + lane;
      uint32_t chunk_ctr = 0;   // staging buffers alternate over all chunks of all tiles
      int local = 0;
      bool ok = true;
      for (int t = g_idx; t < num_tiles && ok; t += n_gemm) {
        const Tile tl = decode_tile(p, t, BN);
        if (p.tile_expert && __ldg(p.tile_expert + tl.mt) < 0) continue;
        const int b = local & 1;
        const uint32_t aph = (local >> 1) & 1;
        ++local;
        if (!mbar_wait(&tmem_full[b], aph, abort_flag, p.mbar_timeout_ns)) {
          ok = false;
          if (lane == 0) report(p.symm, kTimeoutMbarrier, kKernelGemm, 30, -1, b, (int)aph, t);
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_acc = tmem_base + b * BN + (static_cast<uint32_t>(q * 32) << 16);
        if (p.tma_store) {
          const CUtensorMap* cmap = (p.mode == kGemmReduceScatter) ? &peer_maps.m[tl.seg] : &tmap_c;
          const int c2 = (p.mode == kGemmReduceScatter) ? (buf * p.symm.world + p.symm.rank) : tl.seg;
#pragma unroll 1
          for (int c = 0; c < BN / kEpiCols; ++c, ++chunk_ctr) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(t_acc + c * kEpiCols, r0);
            tmem_ld_32x32(t_acc + c * kEpiCols + 32, r1);
            tmem_ld_wait();
            if (c == BN / kEpiCols - 1) {
              // whole accumulator is in registers / staged: hand the TMEM buffer back to the MMA warp
              tc_fence_before_sync();
              mbar_arrive(&tmem_empty[b]);
            }
            uint8_t* stg = stage_base + (chunk_ctr & 1) * kEpiBytes;
            // the store that read this staging buffer two chunks ago must have drained it
            if (leader) bulk_wait_read<1>();
            epi_bar();
            uint8_t* srow = stg + row_in_tile * 128;
            const int sw = row_in_tile & 7;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
              *reinterpret_cast<uint4*>(srow + ((j ^ sw) << 4)) = o;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
              *reinterpret_cast<uint4*>(srow + (((j + 4) ^ sw) << 4)) = o;
            }
            fence_proxy_async_smem();
            epi_bar();
            if (leader && tl.n0 + c * kEpiCols < p.N) {
              tma_store_3d(cmap, stg, tl.n0 + c * kEpiCols, tl.mt * kBM, c2);
              bulk_commit();
            }
          }
          if (p.mode == kGemmReduceScatter && leader) {
            // the tile's stores must have landed in the owner's memory before its flag does
            bulk_wait<0>();
            fence_proxy_async();
            fence_acq_rel_sys();
            uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * p.symm.world + p.symm.rank) * p.max_tiles +
                             tl.mt * p.tiles_n + tl.nt;
            st_release_sys(symm_at(p.symm, flag, tl.seg), epoch);
          }
        } else {
          // direct stores (any N / leading dimension)
          const int row = tl.m0 + row_in_tile;
          const bool row_ok = row < tl.m_end;
          __nv_bfloat16* dst_row;
          if (p.mode == kGemmReduceScatter) {
            __nv_bfloat16* slot = p.rs_slots + (static_cast<uint64_t>(buf) * p.symm.world + p.symm.rank) * p.rs_slot_elems +
                                  static_cast<uint64_t>(row - tl.seg * p.seg_rows) * p.N;
            dst_row = symm_at(p.symm, slot, tl.seg);
          } else {
            dst_row = p.c + static_cast<uint64_t>(row) * p.ldc;
          }
          const bool vec_ok = (p.mode == kGemmReduceScatter) ? (p.N % 8 == 0) : (p.ldc % 8 == 0);
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * 32, r);
            tmem_ld_wait();
            const int col0 = tl.n0 + c * 32;
            if (row_ok && col0 < p.N) {
              if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                  o.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                  o.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                  o.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                  st_v4(dst_row + col0 + 8 * j, o);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) dst_row[col0 + j] = __float2bfloat16(__uint_as_float(r[j]));
              }
            }
          }
          tc_fence_before_sync();
          mbar_arrive(&tmem_empty[b]);
          if (p.mode == kGemmReduceScatter) {
            epi_bar();
            if (leader) {
              fence_acq_rel_sys();
              uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * p.symm.world + p.symm.rank) * p.max_tiles +
                               tl.mt * p.tiles_n + tl.nt;
              st_release_sys(symm_at(p.symm, flag, tl.seg), epoch);
            }
          }
        }
      }
      if (!ok) *abort_flag = 1;
      // shared memory must stay valid until the last TMA store has read it, and the stores must be complete
      if (leader) bulk_wait<0>();
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, 2 * BN);
    }
    if (p.mode == kGemmReduceScatter && *abort_flag == 0) rs_reduce(p, epoch, BN);
  }

  // last CTA out advances the call epoch
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


// ---------------------------------------------------------------------------
// CTA-pair form of the same kernel (cta_group::2).  Two CTAs of a cluster, on the two SMs of one TPC, share one
// 256 x 256 output tile: CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and of the B tile, CTA 0
// issues tcgen05.mma.cta_group::2 (M = 256) which reads both CTAs' shared memory and writes 128 accumulator rows
// into each CTA's TMEM, and each CTA runs the epilogue of its own 128 rows.  Per output element this halves the
// B-operand traffic into shared memory and the shared-memory read bandwidth the tensor core needs, which is what
// limits the single-CTA 128 x 256 form.  Barrier protocol:
//   full[s]       in CTA 0, count 1 (+ 64 KB of transactions): both CTAs' TMA loads credit it (cta_group::2 loads)
//   empty[s]      in each CTA, count 1: CTA 0 commits to both after the MMAs that read stage s
//   tmem_full[b]  in each CTA, count 1: CTA 0 commits to both after a tile's last MMA
//   tmem_empty[b] in CTA 0, count 256: the 2 x 128 epilogue threads arrive (remote arrive from CTA 1)
// The fused modes work on 128-row units exactly as in the single-CTA kernel (all-gather flags per 128-row chunk,
// reduce-scatter flags per 128 x 256 tile), so the comm CTAs, the workspaces and the owner-side reduction are shared.
// ---------------------------------------------------------------------------
struct PairLayout {
  static constexpr int kStages = 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = 128 * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;
  static constexpr int kBarOffset = kEpiOffset + 2 * kEpiBytes;
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 16;
};
constexpr int kPairBN = 256;

// Work items of the pair kernel.  Items [0, full_items) are 256 x 256 tiles in the order of decode_tile (M tiles of
// 256 rows; r.mt is the pair-row index).  When the tile count leaves an incomplete last wave of at most half the
// pairs, each tile of that wave is computed as two 256 x 128 halves by two pairs (items full_items + 2 j + h), so
// the tail costs half a tile time instead of a whole one.  r.bn is the item's width in columns, 0 for a half that
// lies beyond N.
struct PairSched {
  int tiles_m_pair, full_items, total_items;
};
__device__ __forceinline__ PairSched make_pair_sched(const KParams& p, int n_pairs) {
  PairSched s;
  s.tiles_m_pair = (p.tiles_m_seg + 1) / 2;
  const int num_tiles = p.num_seg * s.tiles_m_pair * p.tiles_n;
  const int rem = num_tiles % n_pairs;
  const bool split = p.split_tail != 0 && rem > 0 && 2 * rem <= n_pairs;
  s.full_items = split ? num_tiles - rem : num_tiles;
  s.total_items = s.full_items + (split ? 2 * rem : 0);
  return s;
}
struct PairTile {
  int seg, mt, nt, n0, bn;
};
__device__ __forceinline__ PairTile decode_pair_item(const KParams& p, const PairSched& sc, int w) {
  int t = w, half = -1;
  if (w >= sc.full_items) {
    t = sc.full_items + ((w - sc.full_items) >> 1);
    half = (w - sc.full_items) & 1;
  }
  PairTile r;
  const int per_seg = sc.tiles_m_pair * p.tiles_n;
  if (p.mode == kGemmAllGather && p.use_mc && t >= per_seg) {
    // NVLS all-gather: every shard arrives chunk by chunk at the same pace, so the remote part is visited chunk-major:
    // the M tiles are ordered (pair chunk, ring distance) and swept in groups of p.pair_group_m over all columns
    const int rem = t - per_seg;
    const int nrem = p.num_seg - 1;
    const int total_m = sc.tiles_m_pair * nrem;
    const int group_sz = p.pair_group_m * p.tiles_n;
    const int g = rem / group_sz;
    const int first_m = g * p.pair_group_m;
    const int gm = min(total_m - first_m, p.pair_group_m);
    const int in_g = rem - g * group_sz;
    const int m_lin = first_m + in_g % gm;
    r.nt = in_g / gm;
    r.mt = m_lin / nrem;
    r.seg = (p.seg_first + 1 + m_lin % nrem) % p.num_seg;
  } else {
    const int si = t / per_seg;
    const int rem = t - si * per_seg;
    r.seg = (p.seg_first + si) % p.num_seg;
    const int group_sz = p.pair_group_m * p.tiles_n;
    const int g = rem / group_sz;
    const int first_m = g * p.pair_group_m;
    const int gm = min(sc.tiles_m_pair - first_m, p.pair_group_m);
    const int in_g = rem - g * group_sz;
    r.mt = first_m + in_g % gm;
    r.nt = in_g / gm;
  }
  r.n0 = r.nt * kPairBN + (half > 0 ? 128 : 0);
  r.bn = half < 0 ? kPairBN : (r.n0 < p.N ? 128 : 0);
  return r;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ PeerMaps peer_maps,
                 const __grid_constant__ CUtensorMap tmap_a_local, const __grid_constant__ CUtensorMap tmap_out,
                 const __grid_constant__ CUtensorMap tmap_b_half, const KParams p) {
  using L = PairLayout;
  constexpr int kStages = L::kStages;
  constexpr int BN = kPairBN;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();
  const uint32_t epoch = (p.ctx != nullptr) ? ld_volatile(&p.ctx->epoch) : 1u;
  const int buf = epoch & 1;
  const long long cta_t0 = p.stats != nullptr ? clock64() : 0;

  // n_comm is even, so both CTAs of a pair take the same role
  const bool is_comm = (p.mode == kGemmAllGather) && (static_cast<int>(blockIdx.x) < p.n_comm);
  if (is_comm) {
    if (p.use_mc) {
      ag_push_mc_ring(p, epoch, smem);
    } else {
      ag_push_bulk(p, epoch, smem);
    }
  } else {
    if (threadIdx.x == 0) {
      for (int i = 0; i < kStages; ++i) {
        mbar_init(&full_bar[i], 1);
        mbar_init(&empty_bar[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&tmem_full[i], 1);
        mbar_init(&tmem_empty[i], 256);
      }
      *abort_flag = 0;
      fence_mbar_init();
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      if (p.split_tail) tma_prefetch_desc(&tmap_b_half);
      if (p.mode == kGemmAllGather) tma_prefetch_desc(&tmap_a_local);
      if (p.mode != kGemmReduceScatter) tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) {
      // collective over the pair: the same warp of both CTAs allocates all 512 columns in both TMEMs
      tmem_alloc_pair(tmem_base_smem, 2 * BN);
      tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_smem;

    const int n_pairs = (gridDim.x - p.n_comm) / 2;
    const int pair_idx = (blockIdx.x - p.n_comm) / 2;
    const PairSched sched = make_pair_sched(p, n_pairs);
    const int num_kb = (p.K + kBK - 1) / kBK;
    const int tiles_n128 = (p.N + 127) / 128;   // reduce-scatter flags are kept per 128 x 128 unit

    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer (both CTAs, own operand halves)
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        long long w_flag = 0, w_empty = 0;
        for (int w = pair_idx; w < sched.total_items && ok; w += n_pairs) {
          const PairTile tl = decode_pair_item(p, sched, w);
          if (tl.bn == 0) continue;
          const int mt = 2 * tl.mt + static_cast<int>(cr);     // this CTA's 128-row chunk of the segment
          const bool valid_m = mt < p.tiles_m_seg;
          const bool local_seg = (p.mode == kGemmAllGather) && tl.seg == p.symm.rank;
          if (p.mode == kGemmAllGather && !local_seg && valid_m) {
            StallTimer st(p);
            const uint32_t* flags = p.ag_flags + (static_cast<uint64_t>(buf) * p.symm.world + tl.seg) * p.max_chunks;
            if (p.use_mc) {
              // one flag per comm CTA of the source: all of them have delivered their rows of this chunk
              for (int i = 0; i < p.n_comm && ok; ++i)
                ok = wait_until(p.symm, flags + mt * p.n_comm + i, epoch, kCmpGe, kKernelAgGemm, 2, tl.seg, mt * p.n_comm + i);
            } else {
              ok = wait_until(p.symm, flags + mt, epoch, kCmpGe, kKernelAgGemm, 1, tl.seg, mt);
            }
            st.stop(w_flag);
            if (!ok) break;
            fence_proxy_async();
          }
          const bool half = tl.bn != BN;
          const uint32_t tx = 2u * (L::kABytes + (half ? L::kBBytes / 2 : L::kBBytes));
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_try_wait(&empty_bar[s], ph ^ 1)) {
              StallTimer st(p);
              const bool got = mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.mbar_timeout_ns);
              st.stop(w_empty);
              if (!got) {
                ok = false;
                report(p.symm, kTimeoutMbarrier, kKernelGemm, 110, -1, s, (int)ph, w);
                break;
              }
            }
            uint8_t* sa = smem + s * L::kStageBytes;
            uint8_t* sb = sa + L::kABytes;
            const uint32_t full0 = mapa_u32(smem_u32(&full_bar[s]), 0);
            if (cr == 0) mbar_arrive_expect_tx(&full_bar[s], tx);
            if (local_seg) {
              tma_load_3d_pair(sa, &tmap_a_local, full0, kb * kBK, mt * kBM, 0);
            } else {
              tma_load_3d_pair(sa, &tmap_a, full0, kb * kBK, tl.seg * p.seg_rows + mt * kBM,
                               (p.mode == kGemmAllGather) ? buf : 0);
            }
            if (half) {
              tma_load_3d_pair(sb, &tmap_b_half, full0, kb * kBK, tl.n0 + static_cast<int>(cr) * 64, 0);
            } else {
              tma_load_3d_pair(sb, &tmap_b, full0, kb * kBK, tl.n0 + static_cast<int>(cr) * 128, 0);
            }
          }
        }
        stat_flush(p, kStatProdFlagWait, w_flag);
        stat_flush(p, kStatProdEmptyWait, w_empty);
        if (!ok) {
          *abort_flag = 1;
          // loads already issued land within microseconds; give them time before the CTA may leave
          const uint64_t t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 2000000ull) nanosleep(1000);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (CTA 0 of the pair only)
      if (lane == 0 && cr == 0) {
        constexpr uint32_t idesc_full = make_idesc(1u, 2 * kBM, BN);
        constexpr uint32_t idesc_half = make_idesc(1u, 2 * kBM, 128);
        uint32_t it = 0;
        int local = 0;
        bool ok = true;
        long long w_full = 0, w_tmem = 0;
        for (int w = pair_idx; w < sched.total_items && ok; w += n_pairs) {
          const PairTile tl = decode_pair_item(p, sched, w);
          if (tl.bn == 0) continue;
          const uint32_t idesc = tl.bn == BN ? idesc_full : idesc_half;
          const int b = local & 1;
          const uint32_t aph = (local >> 1) & 1;
          ++local;
          if (!mbar_try_wait(&tmem_empty[b], aph ^ 1)) {
            StallTimer st(p);
            const bool got = mbar_wait(&tmem_empty[b], aph ^ 1, abort_flag, p.mbar_timeout_ns);
            st.stop(w_tmem);
            if (!got) {
              ok = false;
              report(p.symm, kTimeoutMbarrier, kKernelGemm, 120, -1, b, (int)aph, w);
              break;
            }
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + b * BN;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_try_wait(&full_bar[s], ph)) {
              StallTimer st(p);
              const bool got = mbar_wait(&full_bar[s], ph, abort_flag, p.mbar_timeout_ns);
              st.stop(w_full);
              if (!got) {
                ok = false;
                report(p.symm, kTimeoutMbarrier, kKernelGemm, 121, -1, s, (int)ph, w);
                break;
              }
            }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k)
              umma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit_pair_mask(&empty_bar[s], 3);
          }
          if (ok) umma_commit_pair_mask(&tmem_full[b], 3);
        }
        stat_flush(p, kStatMmaFullWait, w_full);
        stat_flush(p, kStatMmaTmemWait, w_tmem);
        if (!ok) *abort_flag = 1;
      }
    } else {
      // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
      const int q = warp & 3;
      const bool leader = (warp == 2 && lane == 0);
      uint8_t* stage_base = smem + L::kEpiOffset;
      const int row_in_tile = q * 32 + lane;
      uint32_t chunk_ctr = 0;
      int local = 0;
      bool ok = true;
      long long w_tmem = 0, w_flag = 0, w_store = 0;
      for (int w = pair_idx; w < sched.total_items && ok; w += n_pairs) {
        const PairTile tl = decode_pair_item(p, sched, w);
        if (tl.bn == 0) continue;
        const int n_chunks = tl.bn / kEpiCols;
        const int mt = 2 * tl.mt + static_cast<int>(cr);
        const bool valid_m = mt < p.tiles_m_seg;
        const int b = local & 1;
        const uint32_t aph = (local >> 1) & 1;
        ++local;
        {
          StallTimer st(p);
          const bool got = mbar_wait_sleepy(&tmem_full[b], aph, abort_flag, p.mbar_timeout_ns, p.epi_sleep_ns);
          if (leader) st.stop(w_tmem);
          if (!got) {
            ok = false;
            if (lane == 0) report(p.symm, kTimeoutMbarrier, kKernelGemm, 130, -1, b, (int)aph, w);
            break;
          }
        }
        tc_fence_after_sync();
        const uint32_t t_acc = tmem_base + b * BN + (static_cast<uint32_t>(q * 32) << 16);
        // reduce-scatter: tiles of this rank's own segment (computed last) are summed with the partials the other
        // ranks have already delivered, straight from the fp32 accumulators, and go to the output; no separate
        // reduction pass remains
        const bool own_seg = (p.mode == kGemmReduceScatter) && tl.seg == p.symm.rank;
        const CUtensorMap* cmap = own_seg ? &tmap_out : (p.mode == kGemmReduceScatter) ? &peer_maps.m[tl.seg] : &tmap_c;
        const int c2 = own_seg ? 0 : (p.mode == kGemmReduceScatter) ? (buf * p.symm.world + p.symm.rank) : tl.seg;
        // flags of the 128-column units this item covers
        const int unit0 = mt * tiles_n128 + tl.n0 / 128;
        const int n_units = min(tl.bn / 128, tiles_n128 - tl.n0 / 128);
        if (own_seg && valid_m) {
          const int et = threadIdx.x - 64;
          bool wok = true;
          if (et < p.symm.world && et != p.symm.rank) {
            StallTimer st(p);
            const uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * p.symm.world + et) * p.max_tiles + unit0;
            for (int u = 0; u < n_units && wok; ++u)
              wok = wait_until(p.symm, flag + u, epoch, kCmpGe, kKernelGemmRs, 3, et, unit0 + u);
            st.stop(w_flag);
          }
          if (!wok) *abort_flag = 1;
          epi_bar();
          if (*abort_flag != 0) {
            ok = false;
            break;
          }
        }
        const int seg_row = mt * kBM + row_in_tile;
        const bool row_ok = valid_m && seg_row < p.seg_rows;
#pragma unroll 1
        for (int c = 0; c < n_chunks; ++c, ++chunk_ctr) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_acc + c * kEpiCols, r0);
          tmem_ld_32x32(t_acc + c * kEpiCols + 32, r1);
          tmem_ld_wait();
          if (c == n_chunks - 1) {
            tc_fence_before_sync();
            mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[b]), 0));
          }
          if (own_seg && row_ok) {
            // 32 columns at a time: the 64-byte pieces of ALL other ranks' partials are requested together (one
            // round trip per half chunk instead of one per source), then added to the accumulators
            const int W = p.symm.world;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int col0 = tl.n0 + c * kEpiCols + half * 32;
              uint4 u[kMaxRanks - 1][4];
#pragma unroll
              for (int i = 0; i < kMaxRanks - 1; ++i) {
                if (i < W - 1) {
                  const int src_rank = (p.symm.rank + 1 + i) % W;
                  const __nv_bfloat16* src = p.rs_slots + (static_cast<uint64_t>(buf) * W + src_rank) * p.rs_slot_elems +
                                             static_cast<uint64_t>(seg_row) * p.N + col0;
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    u[i][j] = (col0 + 8 * j + 8 <= p.N) ? ld_relaxed_sys_v4(src + 8 * j) : make_uint4(0u, 0u, 0u, 0u);
                }
              }
#pragma unroll
              for (int i = 0; i < kMaxRanks - 1; ++i) {
                if (i < W - 1) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    uint32_t* r = half ? &r1[8 * j] : &r0[8 * j];
                    const float2 f0 = unpack_bf16x2(u[i][j].x), f1 = unpack_bf16x2(u[i][j].y),
                                 f2 = unpack_bf16x2(u[i][j].z), f3 = unpack_bf16x2(u[i][j].w);
                    r[0] = __float_as_uint(__uint_as_float(r[0]) + f0.x);
                    r[1] = __float_as_uint(__uint_as_float(r[1]) + f0.y);
                    r[2] = __float_as_uint(__uint_as_float(r[2]) + f1.x);
                    r[3] = __float_as_uint(__uint_as_float(r[3]) + f1.y);
                    r[4] = __float_as_uint(__uint_as_float(r[4]) + f2.x);
                    r[5] = __float_as_uint(__uint_as_float(r[5]) + f2.y);
                    r[6] = __float_as_uint(__uint_as_float(r[6]) + f3.x);
                    r[7] = __float_as_uint(__uint_as_float(r[7]) + f3.y);
                  }
                }
              }
            }
          }
          uint8_t* stg = stage_base + (chunk_ctr & 1) * kEpiBytes;
          if (leader) {
            StallTimer st(p);
            bulk_wait_read<1>();
            st.stop(w_store);
          }
          epi_bar();
          uint8_t* srow = stg + row_in_tile * 128;
          const int sw = row_in_tile & 7;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
            o.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            o.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            o.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            *reinterpret_cast<uint4*>(srow + ((j ^ sw) << 4)) = o;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
            o.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            o.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            o.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            *reinterpret_cast<uint4*>(srow + (((j + 4) ^ sw) << 4)) = o;
          }
          fence_proxy_async_smem();
          epi_bar();
          if (leader && valid_m && tl.n0 + c * kEpiCols < p.N) {
            tma_store_3d(cmap, stg, tl.n0 + c * kEpiCols, mt * kBM, c2);
            bulk_commit();
          }
        }
        if (p.mode == kGemmReduceScatter && !own_seg && leader && valid_m) {
          StallTimer st(p);
          bulk_wait<0>();
          st.stop(w_store);
          fence_proxy_async();
          fence_acq_rel_sys();
          uint32_t* flag = p.rs_flags + (static_cast<uint64_t>(buf) * p.symm.world + p.symm.rank) * p.max_tiles + unit0;
          uint32_t* dst = symm_at(p.symm, flag, tl.seg);
          if (n_units == 2 && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
            // both 128-column units of the tile with one release store
            st_release_sys_u64(reinterpret_cast<uint64_t*>(dst), (static_cast<uint64_t>(epoch) << 32) | epoch);
          } else {
            for (int u = 0; u < n_units; ++u) st_release_sys(dst + u, epoch);
          }
        }
      }
      if (leader) {
        stat_flush(p, kStatEpiTmemWait, w_tmem);
        stat_flush(p, kStatEpiStoreWait, w_store);
      }
      // one representative waiter: the partials of rank + 1 are produced last
      if (static_cast<int>(threadIdx.x) - 64 == (p.symm.rank + 1) % p.symm.world) stat_flush(p, kStatEpiFlagWait, w_flag);
      if (!ok) *abort_flag = 1;
      if (leader) bulk_wait<0>();
    }

    // ------------------------------------------------------------ teardown
    // neither CTA may leave (or free TMEM) while its partner can still read its shared memory or signal its barriers
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, 2 * BN);
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

// Fills the kernel parameters shared by both kernel forms; BN is the tile width.
cudaError_t fill_params(const GemmArgs& a, int BN, KParams& p) {
  p.mode = a.mode;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.c = reinterpret_cast<__nv_bfloat16*>(a.c);
  p.ldc = a.ldc;
  const bool fused = a.mode != kGemmPlain;
  p.num_seg = fused ? a.symm.world : 1;
  p.seg_rows = fused ? a.seg_rows : a.M;
  p.tiles_m_seg = (p.seg_rows + kBM - 1) / kBM;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.seg_first = a.mode == kGemmAllGather ? a.symm.rank
               : a.mode == kGemmReduceScatter ? (a.symm.rank + 1) % a.symm.world : 0;
  p.n_comm = a.mode == kGemmAllGather ? a.n_comm_ctas : 0;
  p.tma_store = a.use_tma_store;
  p.a_local = reinterpret_cast<const __nv_bfloat16*>(a.a_local);
  p.ag_ws = reinterpret_cast<__nv_bfloat16*>(a.ag_ws);
  p.ag_buf_elems = static_cast<uint64_t>(a.symm.world) * a.max_seg_rows * static_cast<uint64_t>(a.K);
  p.ag_flags = a.ag_flags;
  p.max_chunks = a.max_chunks;
  p.use_mc = a.use_multimem && a.symm.mc_base != 0;
  p.rs_slots = reinterpret_cast<__nv_bfloat16*>(a.rs_slots);
  p.rs_slot_elems = static_cast<uint64_t>(a.max_seg_rows) * a.N;
  p.rs_flags = a.rs_flags;
  p.max_tiles = a.max_tiles;
  p.rs_out = reinterpret_cast<__nv_bfloat16*>(a.rs_out);
  p.ld_out = a.ld_out;
  p.tile_expert = a.tile_expert;
  p.ctx = a.ctx;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&p.symm, &a.symm, sizeof(SymmInfo));
  // shared-memory barriers complete within microseconds when everything works; their limit follows the configured
  // wait limit (a flag wait of a producer can legitimately hold a consumer's barrier for that long)
  p.mbar_timeout_ns = a.symm.timeout_ns > 0 ? a.symm.timeout_ns : 4000000000ull;
  static const uint32_t epi_sleep = [] {
    const char* e = std::getenv("TDB200_EPI_SLEEP_NS");
    return e != nullptr ? static_cast<uint32_t>(std::atoi(e)) : 0u;
  }();
  p.epi_sleep_ns = epi_sleep;
  // Rasterisation of the pair kernel: a group of M tiles is swept over all columns, so its A rows (group x 256 x K
  // elements) stay in L2 while B streams through once per group.  A larger group halves the number of passes over B;
  // it is taken while the group's A rows fit comfortably in L2 (67 MB at K = 8192).
  {
    static const int forced = [] {
      const char* e = std::getenv("TDB200_PAIR_GROUP_M");
      return e != nullptr ? std::atoi(e) : 0;
    }();
    const uint64_t a_bytes_16 = 16ull * 256ull * static_cast<uint64_t>(a.K) * 2ull;
    // (plain mode only: in the fused modes the order also decides which chunk flags a wave waits for)
    p.pair_group_m = forced > 0 ? forced : ((a.mode == kGemmPlain && a_bytes_16 <= (80ull << 20)) ? 16 : kGroupM);
  }
  p.split_tail = a.split_tail;
  p.stats = reinterpret_cast<unsigned long long*>(a.stats);
  if (a.mode == kGemmAllGather && p.tiles_m_seg > a.max_chunks) return cudaErrorInvalidValue;
  if (a.mode == kGemmAllGather && a.cta_pair && p.use_mc) {
    // the NVLS ring push splits every 128-row chunk over the comm CTAs and keeps one flag per (chunk, comm CTA)
    if (p.n_comm < 2 || p.n_comm > 8 || kBM % p.n_comm != 0 || p.tiles_m_seg * p.n_comm > a.max_chunks) return cudaErrorInvalidValue;
  }
  // the pair kernel keeps reduce-scatter flags per 128 x 128 unit, the single-CTA kernel per tile
  const int rs_flag_units = a.cta_pair ? p.tiles_m_seg * ((a.N + 127) / 128) : p.tiles_m_seg * p.tiles_n;
  if (a.mode == kGemmReduceScatter && rs_flag_units > a.max_tiles) return cudaErrorInvalidValue;
  if (a.mode == kGemmAllGather && (a.n_comm_ctas < 1 || a.n_comm_ctas >= a.num_ctas)) return cudaErrorInvalidValue;
  if (a.K % 8 != 0) return cudaErrorInvalidValue;
  return cudaSuccess;
}

template <int BN>
cudaError_t launch_impl(const GemmArgs& a, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  static_assert(kPushSlots * kPushPiece + kPushSlots * 8 <= L::kTotal, "push ring must fit the GEMM's shared memory");
  const int smem = L::kTotal + 1024;
  {
    static SmemOptIn opt_in;
    cudaError_t e = opt_in.ensure(gemm_kernel<BN>, smem);
    if (e != cudaSuccess) return e;
  }
  KParams p;
  cudaError_t e = fill_params(a, BN, p);
  if (e != cudaSuccess) return e;
  CUtensorMap ta, tb, tc, tl;
  memcpy(&tl, a.tmap_a_local.bytes, sizeof(CUtensorMap));
  memcpy(&ta, a.tmap_a.bytes, sizeof(CUtensorMap));
  memcpy(&tb, a.tmap_b.bytes, sizeof(CUtensorMap));
  memcpy(&tc, a.tmap_c.bytes, sizeof(CUtensorMap));
  PeerMaps pm;
  memcpy(&pm, a.tmap_peer_c, sizeof(PeerMaps));
  gemm_kernel<BN><<<a.num_ctas, kThreads, smem, stream>>>(ta, tb, tc, pm, tl, p);
  return cudaGetLastError();
}

// CTA-pair form: needs the TMA-store epilogue, no grouped mode, an even grid and an even number of comm CTAs;
// the B tensor map must have a 128-row box.
cudaError_t launch_pair(const GemmArgs& a, cudaStream_t stream) {
  using L = PairLayout;
  static_assert(kPushSlots * kPushPiece + kPushSlots * 8 <= L::kTotal, "push ring must fit the GEMM's shared memory");
  static_assert(L::kTotal + 1024 <= 227 * 1024, "pair kernel exceeds the shared memory of an SM");
  const int smem = L::kTotal + 1024;
  {
    static SmemOptIn opt_in;
    cudaError_t e = opt_in.ensure(gemm_pair_kernel, smem);
    if (e != cudaSuccess) return e;
  }
  if (!a.use_tma_store || a.tile_expert != nullptr) return cudaErrorInvalidValue;
  KParams p;
  cudaError_t e = fill_params(a, kPairBN, p);
  if (e != cudaSuccess) return e;
  if ((p.n_comm & 1) != 0) return cudaErrorInvalidValue;
  int grid = a.num_ctas & ~1;
  if (grid - p.n_comm < 2) return cudaErrorInvalidValue;
  CUtensorMap ta, tb, tc, tl;
  memcpy(&tl, a.tmap_a_local.bytes, sizeof(CUtensorMap));
  memcpy(&ta, a.tmap_a.bytes, sizeof(CUtensorMap));
  memcpy(&tb, a.tmap_b.bytes, sizeof(CUtensorMap));
  memcpy(&tc, a.tmap_c.bytes, sizeof(CUtensorMap));
  PeerMaps pm;
  memcpy(&pm, a.tmap_peer_c, sizeof(PeerMaps));
  CUtensorMap to, tbh;
  memcpy(&to, a.tmap_out.bytes, sizeof(CUtensorMap));
  memcpy(&tbh, a.tmap_b_half.bytes, sizeof(CUtensorMap));
  gemm_pair_kernel<<<grid, kThreads, smem, stream>>>(ta, tb, tc, pm, tl, to, tbh, p);
  return cudaGetLastError();
}

}  // namespace

int gemm_smem_bytes(int block_n) {
  return (block_n == 256 ? SmemLayout<256>::kTotal : SmemLayout<128>::kTotal) + 1024;
}

cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.cta_pair) return launch_pair(a, stream);
  if (a.block_n == 256) return launch_impl<256>(a, stream);
  if (a.block_n == 128) return launch_impl<128>(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace tdb
