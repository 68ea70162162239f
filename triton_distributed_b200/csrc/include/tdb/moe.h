// Host API of the mixture-of-experts support kernels (moe.cu).
#pragma once
#include <vector>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace tdb {

// softmax over E router logits (fp32 [T, E]) and top-k: ids int32 [T, k], weights fp32 [T, k] (optionally renormalised).
cudaError_t launch_topk_router(const float* logits, int32_t* ids, float* weights, int T, int E, int k, int normalize,
                               cudaStream_t s);

// Sort the n = T*k (token, slot) pairs by expert with every expert's rows padded to a multiple of `align`.
//   counts[E], offsets[E+1], cursor[E]   scratch / results (int32)
//   sorted_ids[sorted_cap]               flat pair index per sorted row, -1 = padding
//   pos_of[n]                            sorted row of every pair (-1 if its expert id is outside [0, E))
//   tile_expert[max_tiles]               expert of every `align`-row tile, -1 beyond the last tile
//   meta[2]                              {padded row count, tile count}
cudaError_t launch_moe_align_sort(const int32_t* ids, int64_t n, int E, int align, int32_t* counts, int32_t* offsets,
                                  int32_t* cursor, int32_t* sorted_ids, int64_t sorted_cap, int32_t* pos_of,
                                  int32_t* tile_expert, int max_tiles, int32_t* meta, cudaStream_t s);
// Same, for the all-gather -> grouped GEMM overlap: inside an expert the rows are ordered by the ring distance
// ("stage") of their token's source rank, (src - rank) mod world, so that an expert's first tiles need only the
// shards that arrive first.  bucket_counts [E * world] and cursor [E * world] are scratch.
cudaError_t launch_moe_align_sort_staged(const int32_t* ids, int64_t n, int E, int align, int k, int tokens_per_rank, int rank,
                                         int world, int32_t* bucket_counts, int32_t* counts, int32_t* offsets,
                                         int32_t* cursor, int32_t* sorted_ids, int64_t sorted_cap, int32_t* pos_of,
                                         int32_t* tile_expert, int max_tiles, int32_t* meta, cudaStream_t s);
// Device-side tile schedule: stage[t] of every `block`-row tile (largest ring distance of its rows, -1 = padding only)
// and the visiting order (by stage, padding-only tiles last, index order inside a stage); bucket_start [world + 2]
// (optional) = first position of every stage in `order`.  Same result as the host reference moe_tile_arrival_order.
cudaError_t launch_moe_tile_schedule(const int32_t* sorted_ids, int64_t n_sorted, int k, int tokens_per_rank, int rank, int world,
                                     int block, int32_t* stage, int32_t* order, int32_t* bucket_start, cudaStream_t s);
// out[r] = src[sorted_ids[r] / k] (bf16 rows of H elements), zeros for padding.
cudaError_t launch_moe_gather(const void* src, const int32_t* sorted_ids, const int32_t* meta, void* out, int64_t rows_cap,
                              int H, int k, int64_t src_ld, cudaStream_t s);
// out[t] = sum_j w[t,j] * y[pos_of[t*k+j]]  (w may be null = 1).
cudaError_t launch_moe_topk_reduce(const void* y, const int32_t* pos_of, const float* w, void* out, int64_t T, int H, int k,
                                   int64_t out_ld, cudaStream_t s);
// out[pair] = y[pos_of[pair]]: sorted layout back to (token, slot) order.
cudaError_t launch_moe_unsort(const void* y, const int32_t* pos_of, void* out, int64_t rows, int N, cudaStream_t s);

// ---------------------------------------------------------------------------
// Fused tensor-parallel MoE launches (moe_fused_sm100.cu): a persistent grouped tcgen05 GEMM over expert-sorted rows
// whose A rows are gathered inside the kernel, plus (all-gather mode) comm CTAs that push the local tokens to every
// rank, or (reduce modes) reducer CTAs that top-k-sum finished N chunks and exchange them over NVLink.
// ---------------------------------------------------------------------------
enum MoeFusedMode : int { kMoePlain = 0, kMoeAllGather = 1, kMoeReduceRS = 2, kMoeReduceAR = 3 };

struct MoeFusedArgs {
  int mode;
  int K, N, k_top;
  const void* x;               // bf16 source rows [rows, ldx]; all-gather mode: the local token shard [t_local, ldx = K]
  int64_t ldx;
  int a_row_div;               // source row of sorted row r = sorted_ids[r] / a_row_div
  const int32_t* sorted_ids;   // [max_tiles * 128]
  const int32_t* tile_expert;  // [max_tiles]
  const int32_t* order;        // optional tile visiting order [max_tiles]
  const int32_t* meta;         // {padded rows, tiles}
  int max_tiles;
  TensorMap tmap_b;            // weights [E][N][K], box [256 x 64], 128-byte swizzle
  void* y;                     // bf16 output rows [*, ldy]
  int64_t ldy;
  int scatter_out;             // 1: (token, slot) order, 0: sorted layout
  const float* row_weight;     // optional [pairs]
  int num_ctas;
  // all-gather
  int t_local, max_t_local, n_comm;
  void* ag_ws;                 // heap bf16 [2][world * max_t_local][K]
  uint32_t* ag_flags;          // heap [2][world][max_chunks]
  int max_chunks;
  // reduce
  int n_chunks, n_red, T;
  const int32_t* pos_of;       // [T * k_top]
  uint32_t* chunk_done;        // device [2][n_chunks], zero before the first call
  void* red_slots;             // heap bf16 [2][world][slot rows][N]
  uint64_t red_slot_elems;     // slot rows * N
  uint32_t* red_flags;         // heap [2][world][n_chunks * n_red]
  void* out;                   // bf16 [T / world or T, ld_out]
  int64_t ld_out;
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_moe_fused(const MoeFusedArgs& a, cudaStream_t stream);

// Host reference (moe_sched.cc): stage at which every `block`-row tile of the expert-sorted layout becomes computable
// during a ring all-gather (largest ring distance of its rows' source ranks; -1 = padding only) and the tile visiting
// order by stage.
void moe_tile_arrival_order(const int32_t* sorted_ids, int64_t n_sorted, int topk, int tokens_per_rank, int rank, int world,
                            int block, std::vector<int32_t>* order, std::vector<int32_t>* stage);

}  // namespace tdb
