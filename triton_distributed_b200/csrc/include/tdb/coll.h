// Host API of the collective kernels (collectives.cu).
#pragma once
#include "api.h"

namespace tdb {

enum AllReduceMethod : int {
  kArOneShotPush = 0,   // every rank pushes everything to everyone, local sum
  kArTwoShotPush = 1,   // reduce-scatter + all-gather with peer stores
  kArNvlsOneShot = 2,   // multimem.ld_reduce of the whole message on every rank
  kArNvlsTwoShot = 3,   // multimem.ld_reduce of a shard + multimem.st broadcast
};

struct AllReduceArgs {
  const void* in;
  void* out;
  uint64_t bytes;          // multiple of 16
  DType dtype;
  int method;
  int reduce_scatter;      // 1: stop after the reduce-scatter half (two-shot methods), out = this rank's shard
  void* ws;                // heap workspace [2][ws_half_bytes]
  uint64_t ws_half_bytes;
  uint32_t* flags;         // heap [2][2][world][max_ctas]
  int max_ctas;
  int num_ctas;
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_allreduce(const AllReduceArgs& a, cudaStream_t stream);

cudaError_t launch_barrier(uint32_t* flags, CtxDev* ctx, const SymmInfoHost& symm, cudaStream_t stream);

enum AllGatherMethod : int { kAgPush = 0, kAgNvls = 1, kAgPull = 2 };

struct AllGatherArgs {
  void* buf;               // heap [world][shard_bytes], slot [rank] valid on entry
  uint64_t shard_bytes;    // multiple of 16
  int method;
  uint32_t* flags;         // heap [2][2][world][max_ctas]
  int max_ctas;
  int num_ctas;
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_allgather(const AllGatherArgs& a, cudaStream_t stream);

struct AllGatherLLArgs {
  const void* in;          // local shard
  void* out;               // local [world][shard_bytes]
  uint64_t shard_bytes;    // multiple of 8
  void* staging;           // heap [2][staging_half_bytes], half >= world * 2 * shard_bytes
  uint64_t staging_half_bytes;
  int num_ctas;
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_allgather_ll(const AllGatherLLArgs& a, cudaStream_t stream);

// Copy `bytes` (multiple of 16) between device-visible buffers; mode 0 = vector ld/st, 1 = bulk-TMA ring.
cudaError_t launch_p2p_copy(void* dst, const void* src, uint64_t bytes, int num_ctas, int mode, cudaStream_t stream);

cudaError_t launch_primitives_test(int32_t* data, int32_t* scratch, uint32_t* sig, uint32_t* bar_flags, int n,
                                   uint32_t epoch, const SymmInfoHost& symm, cudaStream_t stream);
// Checked warp-scope put (debug translation forced on): bad ranges / ranks are reported, never accessed.
cudaError_t launch_bounds_probe(void* dst_local, const void* src, uint64_t bytes, int peer, const SymmInfoHost& symm,
                                cudaStream_t stream);
cudaError_t launch_timeout_probe(const uint32_t* flag, uint32_t expected, int cmp, const SymmInfoHost& symm,
                                 cudaStream_t stream);

}  // namespace tdb
