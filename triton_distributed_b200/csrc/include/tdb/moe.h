// Host API of the mixture-of-experts support kernels (moe.cu).
#pragma once
#include <vector>
#include <cuda_runtime.h>
#include <stdint.h>

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
// out[r] = src[sorted_ids[r] / k] (bf16 rows of H elements), zeros for padding.
cudaError_t launch_moe_gather(const void* src, const int32_t* sorted_ids, const int32_t* meta, void* out, int64_t rows_cap,
                              int H, int k, int64_t src_ld, cudaStream_t s);
// out[t] = sum_j w[t,j] * y[pos_of[t*k+j]]  (w may be null = 1).
cudaError_t launch_moe_topk_reduce(const void* y, const int32_t* pos_of, const float* w, void* out, int64_t T, int H, int k,
                                   int64_t out_ld, cudaStream_t s);
// out[pair] = y[pos_of[pair]]: sorted layout back to (token, slot) order.
cudaError_t launch_moe_unsort(const void* y, const int32_t* pos_of, void* out, int64_t rows, int N, cudaStream_t s);

// Host reference (moe_sched.cc): stage at which every `block`-row tile of the expert-sorted layout becomes computable
// during a ring all-gather (largest ring distance of its rows' source ranks; -1 = padding only) and the tile visiting
// order by stage.
void moe_tile_arrival_order(const int32_t* sorted_ids, int64_t n_sorted, int topk, int tokens_per_rank, int rank, int world,
                            int block, std::vector<int32_t>* order, std::vector<int32_t>* stage);

}  // namespace tdb
