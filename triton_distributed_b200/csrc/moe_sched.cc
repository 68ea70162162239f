// Tile visiting order for the all-gather -> grouped-GEMM overlap of tensor-parallel MoE (host reference).
//
// After the all-gather the token rows arrive rank by rank (ring distance 0 = local, 1 = the next rank's shard, ...).
// A 128-row tile of the expert-sorted layout can be computed once the shard with the largest ring distance among its
// rows has arrived, its "stage".  Visiting tiles by stage lets the grouped GEMM start on what is already there; this
// file is the plain C++ statement of that order, used as the oracle for any device-side scheduler and by callers that
// chunk the launch per stage.  The reference computes the same order with a 1024-thread CUDA kernel and keeps a C++
// CPU version for its tests (python/triton_dist/kernels/nvidia/threadblock_swizzle_ag_moe.cu:248-413, .cc).
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "tdb/moe.h"

namespace tdb {

void moe_tile_arrival_order(const int32_t* sorted_ids, int64_t n_sorted, int topk, int tokens_per_rank, int rank, int world,
                            int block, std::vector<int32_t>* order, std::vector<int32_t>* stage) {
  const int64_t tiles = (n_sorted + block - 1) / block;
  stage->assign(tiles, -1);                      // -1: the tile holds only padding and can be skipped
  for (int64_t t = 0; t < tiles; ++t) {
    int s = -1;
    for (int64_t r = t * block; r < std::min<int64_t>(n_sorted, (t + 1) * block); ++r) {
      const int32_t id = sorted_ids[r];
      if (id < 0) continue;
      const int src = (id / topk) / tokens_per_rank;
      const int dist = ((src - rank) % world + world) % world;
      s = std::max(s, dist);
    }
    (*stage)[t] = s;
  }
  order->resize(tiles);
  std::iota(order->begin(), order->end(), 0);
  // padding-only tiles go last; ties keep the expert order so that consecutive tiles still share weights
  std::stable_sort(order->begin(), order->end(), [&](int32_t a, int32_t b) {
    const int sa = (*stage)[a] < 0 ? world : (*stage)[a], sb = (*stage)[b] < 0 ? world : (*stage)[b];
    return sa < sb;
  });
}

}  // namespace tdb
