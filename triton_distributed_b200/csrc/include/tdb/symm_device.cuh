// Device API of the symmetric heap: pointer translation, signals, bounded
// waits, put/get at thread / warp / CTA scope, grid and rank barriers.
//
// This is the CUDA C++ restatement of the reference's device language:
//   wait / notify / symm_at / rank / num_ranks
//     (python/triton_dist/language/distributed_ops.py:57-111, lowering in
//      lib/Conversion/TritonDistributedToLLVM/NVIDIA/DistributedOpToLLVM.cpp:146-423)
//   the NVSHMEM device calls it exposes as libshmem_device.*
//     (python/triton_dist/language/extra/libshmem_device.py:28-289): my_pe, n_pes,
//     remote_ptr, remote_mc_ptr, putmem/getmem{,_nbi}{,_warp,_block},
//     putmem_signal, signal_op, signal_wait_until, fence, quiet, barrier_all.
//   grid / intra-node barriers (python/triton_dist/kernels/nvidia/common_ops.py:57-209)
//
// Differences by design: every wait has a time limit and returns a status, and
// flags carry per-call epochs so nothing is reset between calls.
#pragma once
#include "ptx.cuh"
#include "status.h"

namespace tdb {

constexpr int kMaxRanks = 8;  // one NVSwitch domain

// Passed by value to every kernel that touches the heap.
struct SymmInfo {
  uint64_t peer_base[kMaxRanks];  // this process' mapping of every rank's heap
  uint64_t mc_base;               // multicast (NVLS) mapping of the heap, 0 if none
  uint64_t heap_bytes;
  StatusPage* status;             // pinned host memory, device-visible
  int32_t rank;
  int32_t world;
  uint64_t timeout_ns;            // limit of every wait
  uint32_t debug;                 // != 0: put / get / notify check their heap ranges and peer ranks
  uint32_t pad_;
};

TDB_DEVICE int my_pe(const SymmInfo& s) { return s.rank; }
TDB_DEVICE int n_pes(const SymmInfo& s) { return s.world; }

// Translate a pointer into this rank's heap into the same offset of `peer`'s heap.
template <typename T>
TDB_DEVICE T* symm_at(const SymmInfo& s, T* local, int peer) {
  const uint64_t off = reinterpret_cast<uint64_t>(local) - s.peer_base[s.rank];
  return reinterpret_cast<T*>(s.peer_base[peer] + off);
}
// Same offset in the multicast mapping (a store reaches every rank, a
// multimem.ld_reduce sums over every rank).
template <typename T>
TDB_DEVICE T* mc_ptr(const SymmInfo& s, T* local) {
  const uint64_t off = reinterpret_cast<uint64_t>(local) - s.peer_base[s.rank];
  return reinterpret_cast<T*>(s.mc_base + off);
}
TDB_DEVICE bool in_heap(const SymmInfo& s, const void* p, uint64_t bytes) {
  const uint64_t a = reinterpret_cast<uint64_t>(p), b = s.peer_base[s.rank];
  return a >= b && a + bytes <= b + s.heap_bytes;
}

// ---------------------------------------------------------------------------
// Status reporting
// ---------------------------------------------------------------------------
TDB_DEVICE void report(const SymmInfo& s, int code, int kernel, int where, int peer, int index, int expected,
                       int observed) {
  // The page lives in pinned host memory, so no atomics: the first reporter to
  // see code == kOk fills the record (a benign race between simultaneous
  // reporters can only mix fields of two equally valid reports).
  volatile StatusRecord* rec = s.status != nullptr ? &s.status->rec : nullptr;
  if (rec == nullptr || rec->code != kOk) return;
  rec->kernel = kernel;
  rec->where = where;
  rec->block = blockIdx.x;
  rec->peer = peer;
  rec->index = index;
  rec->expected = expected;
  rec->observed = observed;
  __threadfence_system();
  rec->code = code;
  __threadfence_system();
}
TDB_DEVICE bool abort_requested(const SymmInfo& s) {
  return s.status != nullptr && *reinterpret_cast<volatile int32_t*>(&s.status->abort_word) != 0;
}

// Checked translation used by the put / get / signal primitives.  With s.debug set, a peer rank outside [0, world) or
// a range that leaves this rank's heap records kBadArgument (where = `site`, index = low bits of the offending offset)
// and yields nullptr, and the primitive then skips the access: a wrong pointer becomes an error on the host instead
// of a fault on a peer GPU.  Without s.debug it is symm_at.
static __device__ __noinline__ void symm_check_failed(const SymmInfo& s, const void* local, uint64_t bytes, int peer, int site) {
  const uint64_t off = reinterpret_cast<uint64_t>(local) - s.peer_base[s.rank];
  report(s, kBadArgument, kKernelPrimitive, site, peer, static_cast<int>(off & 0x7fffffffu),
         static_cast<int>(s.heap_bytes >> 20), static_cast<int>(bytes & 0x7fffffffu));
}
template <typename T>
TDB_DEVICE T* symm_at_checked(const SymmInfo& s, T* local, uint64_t bytes, int peer, int site) {
  if (s.debug != 0u && (peer < 0 || peer >= s.world || !in_heap(s, local, bytes))) {
    symm_check_failed(s, local, bytes, peer, site);
    return nullptr;
  }
  return symm_at(s, local, peer);
}

// ---------------------------------------------------------------------------
// Signals
// ---------------------------------------------------------------------------
enum SignalOp : int { kSignalSet = 0, kSignalAdd = 1 };

// notify: fence, then set / add a 32-bit flag on `peer` (the flag pointer is a
// pointer into this rank's heap).  Call from ONE thread after the CTA's data
// stores have been ordered by __syncthreads().
TDB_DEVICE void notify(const SymmInfo& s, uint32_t* flag_local, int peer, uint32_t value, SignalOp op) {
  uint32_t* dst = symm_at_checked(s, flag_local, sizeof(uint32_t), peer, 100);
  if (dst == nullptr) return;
  if (op == kSignalSet) {
    st_release_sys(dst, value);
  } else {
    red_release_sys_add(dst, value);
  }
}
TDB_DEVICE void notify_all(const SymmInfo& s, uint32_t* flag_local, uint32_t value, SignalOp op) {
  for (int i = 0; i < s.world; ++i) notify(s, flag_local, (s.rank + i) % s.world, value, op);
}

enum CmpOp : int { kCmpEq = 0, kCmpGe = 1, kCmpNe = 2 };

TDB_DEVICE bool cmp_ok(uint32_t v, uint32_t expected, CmpOp cmp) {
  return cmp == kCmpEq ? v == expected : cmp == kCmpGe ? static_cast<int32_t>(v - expected) >= 0 : v != expected;
}

// wait_until: spin with ld.acquire.sys on a flag in this rank's memory until
// cmp(flag, expected) holds.  Gives up after s.timeout_ns or when the abort
// word is set; then records a status and returns false.
TDB_DEVICE bool wait_until(const SymmInfo& s, const uint32_t* flag, uint32_t expected, CmpOp cmp, int kernel,
                           int where, int peer, int index) {
  uint32_t v = ld_acquire_sys(flag);
  if (cmp_ok(v, expected, cmp)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    v = ld_acquire_sys(flag);
    if (cmp_ok(v, expected, cmp)) return true;
    ++it;
    if ((it & 255u) == 0u && globaltimer_ns() - t0 > s.timeout_ns) {
      report(s, kTimeoutFlag, kernel, where, peer, index, (int)expected, (int)v);
      return false;
    }
    // the abort word lives in pinned host memory: a read crosses PCIe, so look at it rarely
    if ((it & 4095u) == 0u && abort_requested(s)) {
      report(s, kAborted, kernel, where, peer, index, (int)expected, (int)v);
      return false;
    }
  }
}

// The reference's `wait(ptr, n, scope, semantic, value)`: the first n lanes of a
// warp each wait for one of n consecutive flags.  Returns true for the whole
// warp only if every lane's wait succeeded.  All 32 lanes must call.
TDB_DEVICE bool warp_wait_flags(const SymmInfo& s, const uint32_t* flags, int n, uint32_t expected, CmpOp cmp,
                                int kernel, int where) {
  bool ok = true;
  for (int i = lane_id(); i < n; i += 32) ok = ok && wait_until(s, flags + i, expected, cmp, kernel, where, i, i);
  return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------
// put / get (bytes, 16-byte aligned fast path, byte tail otherwise)
// ---------------------------------------------------------------------------
template <int NTHREADS_IS_DYNAMIC = 1>
TDB_DEVICE void copy_bytes_strided(char* dst, const char* src, uint64_t bytes, int tid, int nthreads) {
  const bool aligned = ((reinterpret_cast<uint64_t>(dst) | reinterpret_cast<uint64_t>(src)) & 15u) == 0;
  if (aligned) {
    const uint64_t nvec = bytes >> 4;
    uint64_t i = tid;
    // 4-way unrolled for memory-level parallelism
    for (; i + 3ull * nthreads < nvec; i += 4ull * nthreads) {
      uint4 a = ld_v4(src + (i << 4));
      uint4 b = ld_v4(src + ((i + nthreads) << 4));
      uint4 c = ld_v4(src + ((i + 2ull * nthreads) << 4));
      uint4 d = ld_v4(src + ((i + 3ull * nthreads) << 4));
      st_v4(dst + (i << 4), a);
      st_v4(dst + ((i + nthreads) << 4), b);
      st_v4(dst + ((i + 2ull * nthreads) << 4), c);
      st_v4(dst + ((i + 3ull * nthreads) << 4), d);
    }
    for (; i < nvec; i += nthreads) st_v4(dst + (i << 4), ld_v4(src + (i << 4)));
    for (uint64_t b = (nvec << 4) + tid; b < bytes; b += nthreads) dst[b] = src[b];
  } else {
    for (uint64_t b = tid; b < bytes; b += nthreads) dst[b] = src[b];
  }
}

// putmem: copy `bytes` from local memory `src` to the heap object `dst_local` on `peer`.
TDB_DEVICE void putmem_block(const SymmInfo& s, void* dst_local, const void* src, uint64_t bytes, int peer) {
  char* dst = symm_at_checked(s, reinterpret_cast<char*>(dst_local), bytes, peer, 101);
  if (dst != nullptr) copy_bytes_strided(dst, reinterpret_cast<const char*>(src), bytes, threadIdx.x, blockDim.x);
}
TDB_DEVICE void putmem_warp(const SymmInfo& s, void* dst_local, const void* src, uint64_t bytes, int peer) {
  char* dst = symm_at_checked(s, reinterpret_cast<char*>(dst_local), bytes, peer, 101);
  if (dst != nullptr) copy_bytes_strided(dst, reinterpret_cast<const char*>(src), bytes, lane_id(), 32);
}
TDB_DEVICE void putmem_thread(const SymmInfo& s, void* dst_local, const void* src, uint64_t bytes, int peer) {
  char* dst = symm_at_checked(s, reinterpret_cast<char*>(dst_local), bytes, peer, 101);
  if (dst != nullptr) copy_bytes_strided(dst, reinterpret_cast<const char*>(src), bytes, 0, 1);
}
// getmem: copy from the heap object `src_local` on `peer` into local memory `dst`.
TDB_DEVICE void getmem_block(const SymmInfo& s, void* dst, const void* src_local, uint64_t bytes, int peer) {
  const char* src = symm_at_checked(s, const_cast<char*>(reinterpret_cast<const char*>(src_local)), bytes, peer, 102);
  if (src != nullptr) copy_bytes_strided(reinterpret_cast<char*>(dst), src, bytes, threadIdx.x, blockDim.x);
}
TDB_DEVICE void getmem_warp(const SymmInfo& s, void* dst, const void* src_local, uint64_t bytes, int peer) {
  const char* src = symm_at_checked(s, const_cast<char*>(reinterpret_cast<const char*>(src_local)), bytes, peer, 102);
  if (src != nullptr) copy_bytes_strided(reinterpret_cast<char*>(dst), src, bytes, lane_id(), 32);
}
// putmem_signal: data, then a signal that the receiver can wait for.
TDB_DEVICE void putmem_signal_block(const SymmInfo& s, void* dst_local, const void* src, uint64_t bytes,
                                    uint32_t* sig_local, uint32_t sig_value, SignalOp op, int peer) {
  putmem_block(s, dst_local, src, bytes, peer);
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    notify(s, sig_local, peer, sig_value, op);
  }
}
// fence: order this thread's earlier remote stores before its later ones.
TDB_DEVICE void fence(const SymmInfo&) { fence_acq_rel_sys(); }
// quiet: plain stores are fire-and-forget; a system-scope fence is the strongest
// completion guarantee the memory model offers a thread for its own stores.
TDB_DEVICE void quiet(const SymmInfo&) { __threadfence_system(); }

// ---------------------------------------------------------------------------
// Barriers
// ---------------------------------------------------------------------------
// Grid barrier on one 32-bit word (all CTAs of the launch must be resident:
// use a cooperative launch or a grid no larger than the SM count x occupancy).
// Sense-reversing through bit 31 as in common_ops.py:57-138; needs no reset.
TDB_DEVICE bool grid_barrier(const SymmInfo& s, uint32_t* word, int kernel, int where) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    const uint32_t nb = gridDim.x * gridDim.y * gridDim.z;
    const bool master = (blockIdx.x + blockIdx.y + blockIdx.z) == 0;
    const uint32_t inc = master ? (0x80000000u - (nb - 1)) : 1u;
    __threadfence();
    const uint32_t old = atom_add_acqrel_gpu(word, inc);
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while ((((old ^ ld_acquire_gpu(word)) & 0x80000000u) == 0)) {
      if ((++it & 1023u) == 0u) {
        if (abort_requested(s) || globaltimer_ns() - t0 > s.timeout_ns) {
          report(s, kTimeoutBarrier, kernel, where, -1, blockIdx.x, 0, (int)ld_volatile(word));
          ok = false;
          break;
        }
      }
    }
    __threadfence();
  }
  return __syncthreads_and(ok);
}

// Rank barrier with epoch flags (the "non-atomic" barrier of common_ops.py:171-209,
// with the call count kept on the device so CUDA graphs can replay it):
// `flags` = W words in this rank's heap, `epoch` = value of this call (>0,
// increasing).  Thread t < W stores epoch into peer t's flags[rank] and waits
// for its own flags[t] to reach it.  Call from all threads of ONE CTA.
TDB_DEVICE bool rank_barrier_block(const SymmInfo& s, uint32_t* flags, uint32_t epoch, int kernel, int where) {
  __syncthreads();
  bool ok = true;
  const int t = threadIdx.x;
  if (t < s.world) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(s, flags, t) + s.rank, epoch);
    ok = wait_until(s, flags + t, epoch, kCmpGe, kernel, where, t, t);
  }
  return __syncthreads_and(ok);
}

}  // namespace tdb
