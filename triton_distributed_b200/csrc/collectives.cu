// Collectives over the symmetric heap: rank barrier, all-reduce (one-shot push,
// two-shot push, NVLS one-shot, NVLS two-shot), reduce-scatter, all-gather
// (push / NVLS / low-latency packets), and the device-API self-test kernels.
//
// Reference behaviour being matched (not its code):
//   all-reduce family   python/triton_dist/kernels/nvidia/allreduce.py:333-682, method enum
//                       python/triton_dist/kernels/allreduce.py:28-61
//   reduce-scatter      python/triton_dist/kernels/nvidia/reduce_scatter.py:285-866
//   all-gather          python/triton_dist/kernels/nvidia/allgather.py:81-263,
//                       low_latency_allgather.py:48-779 (LL packets :531-566)
//   barriers            python/triton_dist/kernels/nvidia/common_ops.py:141-243
//
// Design: one NVSwitch domain, so there is no ring / tree / NUMA variant.  Work is
// partitioned by CTA index identically on every rank, so CTA c of rank r only
// ever depends on CTA c of the peers: flags are per (phase, source rank, CTA),
// carry the call epoch, and no grid barrier is needed.  Buffers alternate with
// the epoch parity, which makes back-to-back calls safe without a trailing
// barrier (a rank cannot run two calls ahead of a peer because every call needs
// data from every peer).
#include "tdb/api.h"
#include "tdb/coll.h"
#include "tdb/symm_device.cuh"

namespace tdb {

namespace {

constexpr int kCollThreads = 512;

template <typename T>
struct Vec16;  // 16-byte vector helpers: to/from fp32 accumulators
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static TDB_DEVICE void add(float* acc, uint4 u) {
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
    acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
  }
  static TDB_DEVICE uint4 pack(const float* acc) {
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    return o;
  }
  static TDB_DEVICE uint4 mc_reduce(const void* p) { return multimem_ld_reduce_bf16x8(p); }
};
template <>
struct Vec16<__half> {
  static constexpr int kElems = 8;
  static TDB_DEVICE void add(float* acc, uint4 u) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  static TDB_DEVICE uint4 pack(const float* acc) {
    uint4 o;
    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    return o;
  }
  static TDB_DEVICE uint4 mc_reduce(const void* p) { return multimem_ld_reduce_f16x8(p); }
};
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  static TDB_DEVICE void add(float* acc, uint4 u) {
    acc[0] += __uint_as_float(u.x); acc[1] += __uint_as_float(u.y);
    acc[2] += __uint_as_float(u.z); acc[3] += __uint_as_float(u.w);
  }
  static TDB_DEVICE uint4 pack(const float* acc) {
    uint4 o;
    o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]);
    o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]);
    return o;
  }
  static TDB_DEVICE uint4 mc_reduce(const void* p) {
    float4 f = multimem_ld_reduce_f32x4(p);
    uint4 o;
    o.x = __float_as_uint(f.x); o.y = __float_as_uint(f.y); o.z = __float_as_uint(f.z); o.w = __float_as_uint(f.w);
    return o;
  }
};

struct CollParams {
  const char* in;       // local input (any device memory)
  char* out;            // local output (any device memory)
  uint64_t nvec;        // 16-byte vectors in the message (input padded by the caller's tail handling)
  uint64_t tail_bytes;  // bytes past the last full vector (handled by CTA 0 through the same path, scalar)
  char* ws;             // heap workspace, [2][ws_half_bytes]
  uint64_t ws_half_bytes;
  uint32_t* flags;      // heap, [2][2][W][max_ctas]
  int max_ctas;
  CtxDev* ctx;
  SymmInfo symm;
  int method;
  int stop_after_rs;    // reduce-scatter: write this rank's shard to out and stop
};

TDB_DEVICE uint32_t* flag_ptr(const CollParams& p, int buf, int phase, int src, int cta) {
  return p.flags + ((static_cast<uint64_t>(buf) * 2 + phase) * p.symm.world + src) * p.max_ctas + cta;
}

// Signal "CTA c of rank `rank` finished `phase`" on every rank, then wait for the same from all ranks.
TDB_DEVICE bool signal_and_wait_all(const CollParams& p, int buf, int phase, uint32_t epoch, int where) {
  __syncthreads();
  bool ok = true;
  const int W = p.symm.world;
  if (threadIdx.x < W) {
    fence_acq_rel_sys();
    const int peer = (p.symm.rank + threadIdx.x) % W;
    st_release_sys(symm_at(p.symm, flag_ptr(p, buf, phase, p.symm.rank, blockIdx.x), peer), epoch);
    ok = wait_until(p.symm, flag_ptr(p, buf, phase, threadIdx.x, blockIdx.x), epoch, kCmpGe, kKernelAllReduce, where,
                    threadIdx.x, blockIdx.x);
  }
  return __syncthreads_and(ok);
}

TDB_DEVICE void cta_range(uint64_t n, uint64_t* lo, uint64_t* hi) {
  const uint64_t per = (n + gridDim.x - 1) / gridDim.x;
  *lo = min(n, per * blockIdx.x);
  *hi = min(n, *lo + per);
}

// ---------------------------------------------------------------------------
// one-shot push: every rank writes its part into slot [rank] on every peer, then
// sums the W slots.  Workspace half = [W][nvec*16].
// ---------------------------------------------------------------------------
template <typename T>
__device__ bool ar_oneshot_push(const CollParams& p, uint32_t epoch) {
  const int buf = epoch & 1, W = p.symm.world, rank = p.symm.rank;
  char* ws = p.ws + buf * p.ws_half_bytes;
  const uint64_t slot_bytes = p.nvec << 4;
  uint64_t lo, hi;
  cta_range(p.nvec, &lo, &hi);
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint4 v = ld_nc_v4(p.in + (i << 4));
    for (int j = 0; j < W; ++j) {
      const int peer = (rank + j) % W;
      st_v4(symm_at(p.symm, ws + rank * slot_bytes + (i << 4), peer), v);
    }
  }
  if (!signal_and_wait_all(p, buf, 0, epoch, 1)) return false;
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < W; ++s) Vec16<T>::add(acc, ld_relaxed_sys_v4(ws + s * slot_bytes + (i << 4)));
    st_v4(p.out + (i << 4), Vec16<T>::pack(acc));
  }
  return true;
}

// ---------------------------------------------------------------------------
// two-shot push: reduce-scatter (push shard d to rank d) + all-gather of the
// reduced shards.  Workspace half = [W][shard] for phase 0, then [W][shard] for
// phase 1 (second quarter).
// ---------------------------------------------------------------------------
template <typename T>
__device__ bool ar_twoshot_push(const CollParams& p, uint32_t epoch) {
  const int buf = epoch & 1, W = p.symm.world, rank = p.symm.rank;
  const uint64_t shard = (p.nvec + W - 1) / W;  // vectors per shard
  char* ws0 = p.ws + buf * p.ws_half_bytes;      // [W][shard] partials for my shard
  char* ws1 = ws0 + (static_cast<uint64_t>(W) * shard << 4);  // [W][shard] reduced shards
  uint64_t lo, hi;
  cta_range(shard, &lo, &hi);
  for (int j = 0; j < W; ++j) {
    const int dst = (rank + 1 + j) % W;
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const uint64_t g = dst * shard + i;
      if (g < p.nvec) st_v4(symm_at(p.symm, ws0 + ((rank * shard + i) << 4), dst), ld_nc_v4(p.in + (g << 4)));
    }
  }
  if (!signal_and_wait_all(p, buf, 0, epoch, 2)) return false;
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint64_t g = rank * shard + i;
    if (g >= p.nvec) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < W; ++s) Vec16<T>::add(acc, ld_relaxed_sys_v4(ws0 + ((s * shard + i) << 4)));
    const uint4 o = Vec16<T>::pack(acc);
    if (p.stop_after_rs) {
      st_v4(p.out + (i << 4), o);
    } else {
      for (int j = 0; j < W; ++j) st_v4(symm_at(p.symm, ws1 + ((rank * shard + i) << 4), (rank + j) % W), o);
    }
  }
  if (p.stop_after_rs) return true;
  if (!signal_and_wait_all(p, buf, 1, epoch, 3)) return false;
  for (int s = 0; s < W; ++s) {
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const uint64_t g = s * shard + i;
      if (g < p.nvec) st_v4(p.out + (g << 4), ld_relaxed_sys_v4(ws1 + (g << 4)));
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// NVLS one-shot: copy in -> heap, flags, multimem.ld_reduce everything.
// ---------------------------------------------------------------------------
template <typename T>
__device__ bool ar_nvls_oneshot(const CollParams& p, uint32_t epoch) {
  const int buf = epoch & 1;
  char* ws = p.ws + buf * p.ws_half_bytes;
  uint64_t lo, hi;
  cta_range(p.nvec, &lo, &hi);
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) st_v4(ws + (i << 4), ld_nc_v4(p.in + (i << 4)));
  if (!signal_and_wait_all(p, buf, 0, epoch, 4)) return false;
  const char* mc = mc_ptr(p.symm, ws);
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) st_v4(p.out + (i << 4), Vec16<T>::mc_reduce(mc + (i << 4)));
  return true;
}

// ---------------------------------------------------------------------------
// NVLS two-shot: each rank reduces its shard through the switch and broadcasts
// the result with multimem.st into the second region of the workspace.
// ---------------------------------------------------------------------------
template <typename T>
__device__ bool ar_nvls_twoshot(const CollParams& p, uint32_t epoch) {
  const int buf = epoch & 1, W = p.symm.world, rank = p.symm.rank;
  const uint64_t shard = (p.nvec + W - 1) / W;
  char* ws0 = p.ws + buf * p.ws_half_bytes;
  char* ws1 = ws0 + (static_cast<uint64_t>(W) * shard << 4);
  uint64_t lo, hi;
  cta_range(shard, &lo, &hi);
  // copy-in of the parts of every shard this CTA index is responsible for
  for (int s = 0; s < W; ++s) {
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const uint64_t g = s * shard + i;
      if (g < p.nvec) st_v4(ws0 + (g << 4), ld_nc_v4(p.in + (g << 4)));
    }
  }
  if (!signal_and_wait_all(p, buf, 0, epoch, 5)) return false;
  const char* mc0 = mc_ptr(p.symm, ws0);
  char* mc1 = mc_ptr(p.symm, ws1);
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint64_t g = rank * shard + i;
    if (g >= p.nvec) continue;
    const uint4 o = Vec16<T>::mc_reduce(mc0 + (g << 4));
    if (p.stop_after_rs) {
      st_v4(p.out + (i << 4), o);
    } else {
      multimem_st_v4(mc1 + (g << 4), o);
    }
  }
  if (p.stop_after_rs) return true;
  if (!signal_and_wait_all(p, buf, 1, epoch, 6)) return false;
  for (int s = 0; s < W; ++s) {
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const uint64_t g = s * shard + i;
      if (g < p.nvec) st_v4(p.out + (g << 4), ld_relaxed_sys_v4(ws1 + (g << 4)));
    }
  }
  return true;
}

__device__ void bump_epoch(CtxDev* ctx, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(&ctx->done, 1u);
    if (prev == gridDim.x - 1) {
      ctx->done = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&ctx->epoch) = epoch + 1;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kCollThreads) allreduce_kernel(const CollParams p) {
  const uint32_t epoch = ld_volatile(&p.ctx->epoch);
  switch (p.method) {
    case kArOneShotPush: ar_oneshot_push<T>(p, epoch); break;
    case kArTwoShotPush: ar_twoshot_push<T>(p, epoch); break;
    case kArNvlsOneShot: ar_nvls_oneshot<T>(p, epoch); break;
    case kArNvlsTwoShot: ar_nvls_twoshot<T>(p, epoch); break;
    default: break;
  }
  bump_epoch(p.ctx, epoch);
}

// ---------------------------------------------------------------------------
// Rank barrier as a stream operation: one CTA.
// ---------------------------------------------------------------------------
__global__ void barrier_kernel(uint32_t* flags, CtxDev* ctx, const SymmInfo symm) {
  const uint32_t epoch = ld_volatile(&ctx->epoch);
  rank_barrier_block(symm, flags, epoch, kKernelBarrier, 1);
  if (threadIdx.x == 0) {
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(&ctx->epoch) = epoch + 1;
  }
}

// ---------------------------------------------------------------------------
// All-gather, in place on a symmetric buffer [W][shard_bytes]: every rank's slot
// [rank] is valid on entry; on exit all slots are.  kAgPush: plain peer stores;
// kAgNvls: multimem.st; kAgPull: read the peers' slots.
// ---------------------------------------------------------------------------
struct AgParams {
  char* buf;             // heap
  uint64_t shard_vec;    // 16-byte vectors per shard
  uint32_t* flags;       // heap [2][2][W][max_ctas]
  int max_ctas;
  CtxDev* ctx;
  SymmInfo symm;
  int method;
};

__global__ void __launch_bounds__(kCollThreads) allgather_kernel(const AgParams a) {
  const uint32_t epoch = ld_volatile(&a.ctx->epoch);
  const int buf = epoch & 1, W = a.symm.world, rank = a.symm.rank;
  CollParams p;  // only the fields used by signal_and_wait_all
  p.flags = a.flags;
  p.max_ctas = a.max_ctas;
  p.symm = a.symm;
  uint64_t lo, hi;
  cta_range(a.shard_vec, &lo, &hi);
  char* mine = a.buf + ((rank * a.shard_vec) << 4);
  bool ok = true;
  if (a.method == kAgPull) {
    // peers' slots must be complete before they are read: entry flags first
    ok = signal_and_wait_all(p, buf, 0, epoch, 10);
    if (ok) {
      for (int j = 1; j < W; ++j) {
        const int src = (rank + j) % W;
        const char* remote = symm_at(a.symm, a.buf + ((src * a.shard_vec) << 4), src);
        char* dst = a.buf + ((src * a.shard_vec) << 4);
        for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) st_v4(dst + (i << 4), ld_relaxed_sys_v4(remote + (i << 4)));
      }
      // nobody may overwrite its slot (next call) before all peers have read it
      ok = signal_and_wait_all(p, buf, 1, epoch, 11);
    }
  } else {
    // entry flags: every rank has finished reading the previous contents
    ok = signal_and_wait_all(p, buf, 0, epoch, 12);
    if (ok) {
      if (a.method == kAgNvls && a.symm.mc_base != 0) {
        char* mc = mc_ptr(a.symm, mine);
        for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) multimem_st_v4(mc + (i << 4), ld_v4(mine + (i << 4)));
      } else {
        for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
          const uint4 v = ld_v4(mine + (i << 4));
          for (int j = 1; j < W; ++j) st_v4(symm_at(a.symm, mine + (i << 4), (rank + j) % W), v);
        }
      }
      ok = signal_and_wait_all(p, buf, 1, epoch, 13);
    }
  }
  bump_epoch(a.ctx, epoch);
}

// ---------------------------------------------------------------------------
// Low-latency all-gather with in-band flags: the sender interleaves every 8 data
// bytes with an 8-byte (flag, flag) pair... here: 16-byte packets {d0, d1, flag, flag}
// would waste half the bandwidth too; we use {d0, flag, d1, flag} so that each
// 8-byte half is atomic on its own.  The receiver polls the packet until both
// flags equal the call epoch.  No separate signal, no ordering requirement.
// Staging = heap [2][W][2 * shard_bytes]; out = local [W][shard_bytes].
// ---------------------------------------------------------------------------
struct AgLLParams {
  const char* in;        // local shard, shard_words 32-bit words... 8-byte units
  char* out;             // local [W][shard]
  uint64_t shard_u64;    // 8-byte units per shard
  char* staging;         // heap [2][W][shard_u64 * 16]
  uint64_t staging_half_bytes;
  CtxDev* ctx;
  SymmInfo symm;
};

__global__ void __launch_bounds__(kCollThreads) allgather_ll_kernel(const AgLLParams a) {
  const uint32_t epoch = ld_volatile(&a.ctx->epoch);
  const int buf = epoch & 1, W = a.symm.world, rank = a.symm.rank;
  char* st = a.staging + buf * a.staging_half_bytes;
  const uint64_t slot_bytes = a.shard_u64 * 16;
  uint64_t lo, hi;
  cta_range(a.shard_u64, &lo, &hi);
  // send
  for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint2 d = *reinterpret_cast<const uint2*>(a.in + (i << 3));
    uint4 pkt;
    pkt.x = d.x; pkt.y = epoch; pkt.z = d.y; pkt.w = epoch;
    for (int j = 0; j < W; ++j) st_relaxed_sys_v4(symm_at(a.symm, st + rank * slot_bytes + (i << 4), (rank + j) % W), pkt);
  }
  // receive
  bool ok = true;
  const uint64_t t0 = globaltimer_ns();
  for (int s = 0; s < W && ok; ++s) {
    for (uint64_t i = lo + threadIdx.x; i < hi && ok; i += blockDim.x) {
      const char* src = st + s * slot_bytes + (i << 4);
      uint4 pkt = ld_relaxed_sys_v4(src);
      uint32_t spins = 0;
      while (pkt.y != epoch || pkt.w != epoch) {
        if ((++spins & 255u) == 0u && (abort_requested(a.symm) || globaltimer_ns() - t0 > a.symm.timeout_ns)) {
          report(a.symm, kTimeoutFlag, kKernelAllGather, 20, s, static_cast<int>(i), (int)epoch, (int)pkt.y);
          ok = false;
          break;
        }
        pkt = ld_relaxed_sys_v4(src);
      }
      if (ok) *reinterpret_cast<uint2*>(a.out + ((s * a.shard_u64 + i) << 3)) = make_uint2(pkt.x, pkt.z);
    }
  }
  bump_epoch(a.ctx, epoch);
}

// ---------------------------------------------------------------------------
// Device-API self test (one CTA per rank): exercises symm_at, putmem/getmem at
// thread / warp / block scope, putmem_signal, notify set/add, wait_until,
// rank barrier.  data/scratch/sig live in the heap.
//   step 1  rank r puts (r+1)*1000+i into data[r*n + i] on the next rank (block scope),
//           with a signal add of 1 on sig[0]
//   step 2  waits for sig[0] >= epoch, then gets the previous rank's `data` slot of ITS
//           predecessor with getmem_warp into scratch
//   step 3  barrier; thread-scope put of one word into every peer's sig[8 + rank]
// ---------------------------------------------------------------------------
__global__ void primitives_test_kernel(int32_t* data, int32_t* scratch, uint32_t* sig, uint32_t* bar_flags, int n,
                                       uint32_t epoch, const SymmInfo symm) {
  extern __shared__ int32_t sm_stage[];
  const int W = symm.world, rank = symm.rank;
  const int next = (rank + 1) % W, prev = (rank + W - 1) % W;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sm_stage[i] = (rank + 1) * 1000 + i;
  __syncthreads();
  // stage in global scratch (second half) because put sources must be in global memory
  int32_t* src = scratch + n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) src[i] = sm_stage[i];
  __syncthreads();
  putmem_signal_block(symm, data + rank * n, src, static_cast<uint64_t>(n) * 4, sig, 1, kSignalAdd, next);
  bool ok = true;
  if (threadIdx.x == 0) ok = wait_until(symm, sig, epoch, kCmpGe, kKernelPrimitive, 1, prev, 0);
  ok = __syncthreads_and(ok);
  if (!ok) return;
  if (!rank_barrier_block(symm, bar_flags, 2 * epoch - 1, kKernelPrimitive, 2)) return;
  // after the barrier every rank holds its predecessor's row: fetch the predecessor's copy of ITS predecessor
  if (threadIdx.x < 32) {
    const int pp = (prev + W - 1) % W;
    getmem_warp(symm, scratch, data + pp * n, static_cast<uint64_t>(n) * 4, prev);
  }
  __syncthreads();
  if (threadIdx.x < W) {
    uint32_t v = epoch * 100 + rank;
    // thread-scope put of one word to peer `threadIdx.x`
    *symm_at(symm, sig + 8 + rank, threadIdx.x) = v;
    __threadfence_system();
  }
  rank_barrier_block(symm, bar_flags, 2 * epoch, kKernelPrimitive, 3);
}

// Stream-ordered bounded wait on one flag: the stream continues when cmp(flag, expected) holds, or after the time
// limit with a status record (also the probe that shows a wait nothing satisfies returns a status).
__global__ void timeout_probe_kernel(const uint32_t* flag, uint32_t expected, int cmp, const SymmInfo symm) {
  if (threadIdx.x == 0) wait_until(symm, flag, expected, static_cast<CmpOp>(cmp), kKernelPrimitive, 99, -1, 0);
}

// One warp-scope put with the checked translation forced on: a destination outside the heap or a peer rank outside
// [0, world) records kBadArgument and issues no store (the check is arithmetic on the arguments, nothing is accessed).
__global__ void bounds_probe_kernel(void* dst_local, const void* src, uint64_t bytes, int peer, SymmInfo symm) {
  symm.debug = 1u;
  if (threadIdx.x < 32) putmem_warp(symm, dst_local, src, bytes, peer);
}

// ---------------------------------------------------------------------------
// Plain copy kernel between any two device-visible buffers (local or peer-mapped): the transport of the
// pipeline-parallel CommOp and the calibration kernel for NVLink bandwidth.
//   mode 0: every thread moves 16-byte vectors (4 loads in flight per thread)
//   mode 1: one thread per CTA drives a ring of bulk-TMA copies (global -> shared -> global)
// ---------------------------------------------------------------------------
constexpr int kCopyPiece = 32 * 1024;
constexpr int kCopySlots = 6;
constexpr int kCopyAhead = 4;

__global__ void __launch_bounds__(kCollThreads) p2p_copy_kernel(char* dst, const char* src, uint64_t bytes, int mode) {
  extern __shared__ __align__(128) uint8_t cp_smem[];
  uint64_t lo, hi;
  if (mode == 0) {
    cta_range(bytes >> 4, &lo, &hi);
    uint64_t i = lo + threadIdx.x;
    const uint64_t T = blockDim.x;
    for (; i + 3 * T < hi; i += 4 * T) {
      const uint4 a = ld_v4(src + (i << 4)), b = ld_v4(src + ((i + T) << 4)), c = ld_v4(src + ((i + 2 * T) << 4)),
                  d = ld_v4(src + ((i + 3 * T) << 4));
      st_v4(dst + (i << 4), a);
      st_v4(dst + ((i + T) << 4), b);
      st_v4(dst + ((i + 2 * T) << 4), c);
      st_v4(dst + ((i + 3 * T) << 4), d);
    }
    for (; i < hi; i += T) st_v4(dst + (i << 4), ld_v4(src + (i << 4)));
    return;
  }
  if (threadIdx.x != 0) return;
  uint64_t* bars = reinterpret_cast<uint64_t*>(cp_smem + kCopySlots * kCopyPiece);
  for (int i = 0; i < kCopySlots; ++i) mbar_init(&bars[i], 1);
  fence_mbar_init();
  const uint64_t npieces_total = (bytes + kCopyPiece - 1) / kCopyPiece;
  cta_range(npieces_total, &lo, &hi);
  const uint64_t n = hi - lo;
  for (uint64_t step = 0; step < n + kCopyAhead; ++step) {
    if (step < n) {
      const int slot = step % kCopySlots;
      bulk_wait_read<kCopySlots - kCopyAhead - 1>();
      const uint64_t off = (lo + step) * kCopyPiece;
      const uint32_t sz = static_cast<uint32_t>(bytes - off < (uint64_t)kCopyPiece ? bytes - off : (uint64_t)kCopyPiece);
      mbar_arrive_expect_tx(&bars[slot], sz);
      bulk_load(cp_smem + slot * kCopyPiece, src + off, sz, &bars[slot]);
    }
    if (step >= kCopyAhead) {
      const uint64_t j = step - kCopyAhead;
      const int slot = j % kCopySlots;
      if (!mbar_wait(&bars[slot], (j / kCopySlots) & 1, nullptr, 2000000000ull)) break;
      const uint64_t off = (lo + j) * kCopyPiece;
      const uint32_t sz = static_cast<uint32_t>(bytes - off < (uint64_t)kCopyPiece ? bytes - off : (uint64_t)kCopyPiece);
      bulk_store(dst + off, cp_smem + slot * kCopyPiece, sz);
      bulk_commit();
    }
  }
  bulk_wait<0>();
}

SymmInfo to_dev(const SymmInfoHost& h) {
  SymmInfo s;
  static_assert(sizeof(SymmInfo) == sizeof(SymmInfoHost), "SymmInfo mirrors must match");
  memcpy(&s, &h, sizeof(s));
  return s;
}

}  // namespace

cudaError_t launch_allreduce(const AllReduceArgs& a, cudaStream_t stream) {
  CollParams p;
  p.in = reinterpret_cast<const char*>(a.in);
  p.out = reinterpret_cast<char*>(a.out);
  p.nvec = a.bytes >> 4;
  p.tail_bytes = a.bytes & 15;
  p.ws = reinterpret_cast<char*>(a.ws);
  p.ws_half_bytes = a.ws_half_bytes;
  p.flags = a.flags;
  p.max_ctas = a.max_ctas;
  p.ctx = a.ctx;
  p.symm = to_dev(a.symm);
  p.method = a.method;
  p.stop_after_rs = a.reduce_scatter;
  if (p.tail_bytes != 0) return cudaErrorInvalidValue;  // callers pad to 16 bytes
  if ((a.method == kArNvlsOneShot || a.method == kArNvlsTwoShot) && a.symm.mc_base == 0) return cudaErrorInvalidValue;
  const int W = a.symm.world;
  const uint64_t shard = (p.nvec + W - 1) / W;
  uint64_t need = 0;
  switch (a.method) {
    case kArOneShotPush: need = static_cast<uint64_t>(W) * p.nvec * 16; break;
    case kArTwoShotPush:
    case kArNvlsTwoShot: need = 2ull * W * shard * 16; break;
    case kArNvlsOneShot: need = p.nvec * 16; break;
    default: return cudaErrorInvalidValue;
  }
  if (need > a.ws_half_bytes) return cudaErrorInvalidValue;
  int ctas = a.num_ctas;
  if (ctas < 1) ctas = 1;
  if (ctas > a.max_ctas) ctas = a.max_ctas;
  switch (a.dtype) {
    case kBF16: allreduce_kernel<__nv_bfloat16><<<ctas, kCollThreads, 0, stream>>>(p); break;
    case kF16: allreduce_kernel<__half><<<ctas, kCollThreads, 0, stream>>>(p); break;
    case kF32: allreduce_kernel<float><<<ctas, kCollThreads, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_barrier(uint32_t* flags, CtxDev* ctx, const SymmInfoHost& symm, cudaStream_t stream) {
  barrier_kernel<<<1, 32, 0, stream>>>(flags, ctx, to_dev(symm));
  return cudaGetLastError();
}

cudaError_t launch_allgather(const AllGatherArgs& a, cudaStream_t stream) {
  if (a.shard_bytes & 15) return cudaErrorInvalidValue;
  AgParams p;
  p.buf = reinterpret_cast<char*>(a.buf);
  p.shard_vec = a.shard_bytes >> 4;
  p.flags = a.flags;
  p.max_ctas = a.max_ctas;
  p.ctx = a.ctx;
  p.symm = to_dev(a.symm);
  p.method = a.method;
  int ctas = a.num_ctas < 1 ? 1 : (a.num_ctas > a.max_ctas ? a.max_ctas : a.num_ctas);
  allgather_kernel<<<ctas, kCollThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_allgather_ll(const AllGatherLLArgs& a, cudaStream_t stream) {
  if (a.shard_bytes & 7) return cudaErrorInvalidValue;
  AgLLParams p;
  p.in = reinterpret_cast<const char*>(a.in);
  p.out = reinterpret_cast<char*>(a.out);
  p.shard_u64 = a.shard_bytes >> 3;
  p.staging = reinterpret_cast<char*>(a.staging);
  p.staging_half_bytes = a.staging_half_bytes;
  p.ctx = a.ctx;
  p.symm = to_dev(a.symm);
  if (static_cast<uint64_t>(a.symm.world) * p.shard_u64 * 16 > a.staging_half_bytes) return cudaErrorInvalidValue;
  int ctas = a.num_ctas < 1 ? 1 : a.num_ctas;
  allgather_ll_kernel<<<ctas, kCollThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_p2p_copy(void* dst, const void* src, uint64_t bytes, int num_ctas, int mode, cudaStream_t stream) {
  if ((bytes & 15) != 0 || ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) != 0)
    return cudaErrorInvalidValue;
  if (bytes == 0) return cudaSuccess;
  const int smem = mode == 1 ? kCopySlots * kCopyPiece + 64 : 0;
  if (mode == 1) {
    static bool set = false;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(p2p_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return e;
      set = true;
    }
  }
  if (num_ctas < 1) num_ctas = 1;
  p2p_copy_kernel<<<num_ctas, kCollThreads, smem, stream>>>(reinterpret_cast<char*>(dst), reinterpret_cast<const char*>(src),
                                                            bytes, mode);
  return cudaGetLastError();
}

cudaError_t launch_primitives_test(int32_t* data, int32_t* scratch, uint32_t* sig, uint32_t* bar_flags, int n,
                                   uint32_t epoch, const SymmInfoHost& symm, cudaStream_t stream) {
  primitives_test_kernel<<<1, 256, n * 4, stream>>>(data, scratch, sig, bar_flags, n, epoch, to_dev(symm));
  return cudaGetLastError();
}

cudaError_t launch_bounds_probe(void* dst_local, const void* src, uint64_t bytes, int peer, const SymmInfoHost& symm,
                                cudaStream_t stream) {
  bounds_probe_kernel<<<1, 32, 0, stream>>>(dst_local, src, bytes, peer, to_dev(symm));
  return cudaGetLastError();
}

cudaError_t launch_timeout_probe(const uint32_t* flag, uint32_t expected, int cmp, const SymmInfoHost& symm,
                                 cudaStream_t stream) {
  if (cmp < 0 || cmp > 2) return cudaErrorInvalidValue;
  timeout_probe_kernel<<<1, 32, 0, stream>>>(flag, expected, cmp, to_dev(symm));
  return cudaGetLastError();
}

}  // namespace tdb
