// Mixture-of-experts support kernels: top-k router, token sort / tile alignment, row gather, top-k weighted reduce.
//
// The grouped GEMM itself is the tcgen05 kernel of gemm_sm100.cu run over rows sorted by expert: every 128-row tile
// belongs to one expert (padding rows are zero) and the per-tile expert id selects the weight slice through the third
// coordinate of the B tensor map.
//
// Reference behaviour being matched (not its code):
//   router                  layers/nvidia/tp_moe.py:247-250 (softmax + top-k in torch)
//   align / sort            csrc/lib/moe_utils.cu:60-312, kernels/nvidia/moe_utils.py:144-250,
//                           allgather_group_gemm.py:85-250 (sorted gather index, per-tile expert, block alignment)
//   weighted top-k reduce   kernels/nvidia/moe_utils.py:285 (reduce_topk_kernel)
// Unlike the reference's native prototype there is no per-call cudaMalloc and no single-CTA limit.
#include "tdb/moe.h"
#include "tdb/ptx.cuh"

namespace tdb {

namespace {

// One warp per token: softmax over E logits (fp32), then k rounds of arg-max.  E <= 32 * kMaxPerLane.
constexpr int kMaxPerLane = 16;

__global__ void topk_router_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids, float* __restrict__ weights,
                                   int T, int E, int k, int normalize) {
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x * warps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[static_cast<int64_t>(t) * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    v[i] = (lane + 32 * i < E) ? __expf(v[i] - mx) : -1.f;   // probabilities are >= 0, -1 marks "not a candidate"
    sum += fmaxf(v[i], 0.f);
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      if (v[i] > best) {
        best = v[i];
        bi = lane + 32 * i;
      }
    }
    // warp arg-max, ties to the lowest expert index (matches torch.topk on distinct values; stable on ties)
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (lane + 32 * i == bi) v[i] = -1.f;
    picked_sum += best * inv;
    if (lane == j) {
      my_w = best * inv;
      my_id = bi;
    }
  }
  if (lane < k) {
    ids[static_cast<int64_t>(t) * k + lane] = my_id;
    weights[static_cast<int64_t>(t) * k + lane] = normalize ? my_w / picked_sum : my_w;
  }
}

// ---- align / sort -----------------------------------------------------------------------------------------------
// counts[e] = number of (token, slot) pairs routed to expert e (ids equal to E, "dropped", are ignored)
__global__ void moe_count_kernel(const int32_t* __restrict__ ids, int64_t n, int E, int32_t* counts) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(counts + e, 1);
  }
}

// One CTA: padded exclusive offsets (each expert's rows start at a multiple of `align`), per-tile expert ids, total.
// offsets[E + 1]; cursor[e] = offsets[e] (scatter cursors); tile_expert[max_tiles] (-1 beyond the last tile);
// meta[0] = padded total rows, meta[1] = number of tiles.
__global__ void moe_offsets_kernel(const int32_t* __restrict__ counts, int E, int align, int32_t* offsets,
                                   int32_t* cursor, int32_t* tile_expert, int max_tiles, int32_t* meta) {
  extern __shared__ int32_t sh[];   // E + 1
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      sh[e] = acc;
      acc += (counts[e] + align - 1) / align * align;
    }
    sh[E] = acc;
    meta[0] = acc;
    meta[1] = acc / align;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = sh[e];
    if (e < E) cursor[e] = sh[e];
  }
  const int total_tiles = sh[E] / align;
  for (int tl = threadIdx.x; tl < max_tiles; tl += blockDim.x) {
    int ex = -1;
    if (tl < total_tiles) {
      // binary search: last e with offsets[e] <= tl * align
      int lo = 0, hi = E - 1;
      const int row = tl * align;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (sh[mid] <= row) lo = mid; else hi = mid - 1;
      }
      ex = lo;
    }
    tile_expert[tl] = ex;
  }
}

// sorted_ids[pos] = flat (token * k + slot) index, -1 for padding; pos_of[flat] = pos (or -1 when dropped)
__global__ void moe_scatter_kernel(const int32_t* __restrict__ ids, int64_t n, int E, int32_t* cursor,
                                   int32_t* sorted_ids, int32_t* pos_of) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      const int pos = atomicAdd(cursor + e, 1);
      sorted_ids[pos] = static_cast<int32_t>(i);
      pos_of[i] = pos;
    } else {
      pos_of[i] = -1;
    }
  }
}

// out[r, :] = src[sorted_ids[r] / k, :]  (zeros for padding rows); one CTA per row, 16-byte vectors
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ sorted_ids,
                                  const int32_t* __restrict__ meta, __nv_bfloat16* __restrict__ out, int H, int k,
                                  int64_t src_ld) {
  const int64_t r = blockIdx.x;
  if (r >= meta[0]) return;   // beyond the padded total: never read by the GEMM (its tiles are skipped)
  const int id = sorted_ids[r];
  uint4* dst = reinterpret_cast<uint4*>(out + r * H);
  if (id < 0) {
    for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<int64_t>(id / k) * src_ld);
    for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = s[i];
  }
}

// out[t, :] = sum_j w[t, j] * y[pos_of[t * k + j], :]   (dropped slots contribute nothing)
__global__ void moe_topk_reduce_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ pos_of,
                                       const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int H, int k,
                                       int64_t out_ld) {
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int pos = pos_of[t * k + j];
      if (pos < 0) continue;
      const float wj = w ? w[t * k + j] : 1.f;
      const uint4 u = reinterpret_cast<const uint4*>(y + static_cast<int64_t>(pos) * H)[i];
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      acc[0] += wj * f0.x; acc[1] += wj * f0.y; acc[2] += wj * f1.x; acc[3] += wj * f1.y;
      acc[4] += wj * f2.x; acc[5] += wj * f2.y; acc[6] += wj * f3.x; acc[7] += wj * f3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + t * out_ld)[i] = o;
  }
}

// out[flat, :] = y[pos_of[flat], :]  (sorted layout -> original (token, slot) layout; zeros when dropped)
__global__ void moe_unsort_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ pos_of,
                                  __nv_bfloat16* __restrict__ out, int N) {
  const int64_t r = blockIdx.x;
  const int pos = pos_of[r];
  uint4* dst = reinterpret_cast<uint4*>(out + r * N);
  if (pos < 0) {
    for (int i = threadIdx.x; i < (N >> 3); i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* s = reinterpret_cast<const uint4*>(y + static_cast<int64_t>(pos) * N);
    for (int i = threadIdx.x; i < (N >> 3); i += blockDim.x) dst[i] = s[i];
  }
}


// ---- staged sort and device-side tile schedule for the all-gather -> grouped GEMM overlap ---------------------------
// Ring distance ("stage") of a (token, slot) pair's source rank: tokens are laid out rank-major in the gathered buffer.
__device__ __forceinline__ int pair_stage(int flat, int k, int tokens_per_rank, int rank, int world) {
  const int src = (flat / k) / tokens_per_rank;
  return ((src - rank) % world + world) % world;
}

// counts[e * world + stage]
__global__ void moe_count_staged_kernel(const int32_t* __restrict__ ids, int64_t n, int E, int k, int tokens_per_rank,
                                        int rank, int world, int32_t* counts) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(counts + e * world + pair_stage(static_cast<int>(i), k, tokens_per_rank, rank, world), 1);
  }
}

// One CTA.  Experts are padded to `align` rows as in moe_offsets_kernel; inside an expert the rows of stage 0 come
// first, then stage 1, ...: cursor[e * world + st] = first row of that bucket.  expert_counts[e] = rows of expert e.
__global__ void moe_offsets_staged_kernel(const int32_t* __restrict__ counts, int E, int world, int align, int32_t* offsets,
                                          int32_t* cursor, int32_t* expert_counts, int32_t* tile_expert, int max_tiles,
                                          int32_t* meta) {
  extern __shared__ int32_t sh[];   // E + 1
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int st = 0; st < world; ++st) c += counts[e * world + st];
    expert_counts[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      sh[e] = acc;
      acc += (expert_counts[e] + align - 1) / align * align;
    }
    sh[E] = acc;
    meta[0] = acc;
    meta[1] = acc / align;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = sh[e];
    if (e < E) {
      int acc = sh[e];
      for (int st = 0; st < world; ++st) {
        cursor[e * world + st] = acc;
        acc += counts[e * world + st];
      }
    }
  }
  const int total_tiles = sh[E] / align;
  for (int tl = threadIdx.x; tl < max_tiles; tl += blockDim.x) {
    int ex = -1;
    if (tl < total_tiles) {
      int lo = 0, hi = E - 1;
      const int row = tl * align;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (sh[mid] <= row) lo = mid; else hi = mid - 1;
      }
      ex = lo;
    }
    tile_expert[tl] = ex;
  }
}

__global__ void moe_scatter_staged_kernel(const int32_t* __restrict__ ids, int64_t n, int E, int k, int tokens_per_rank,
                                          int rank, int world, int32_t* cursor, int32_t* sorted_ids, int32_t* pos_of) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      const int pos = atomicAdd(cursor + e * world + pair_stage(static_cast<int>(i), k, tokens_per_rank, rank, world), 1);
      sorted_ids[pos] = static_cast<int32_t>(i);
      pos_of[i] = pos;
    } else {
      pos_of[i] = -1;
    }
  }
}

// Device-side tile schedule (one CTA of 1024 threads): stage[t] = largest ring distance of tile t's rows (-1: padding
// only), order = tiles by stage, padding-only tiles last, expert order kept inside a stage - the order of the host
// reference moe_tile_arrival_order.  A warp computes the stage of a tile; then warp b collects the tiles of bucket b
// (stage b, bucket `world` = padding only) in index order with ballots, and the buckets are laid end to end.
__global__ void __launch_bounds__(1024) moe_tile_schedule_kernel(const int32_t* __restrict__ sorted_ids, int64_t n_sorted,
                                                                 int k, int tokens_per_rank, int rank, int world, int block,
                                                                 int32_t* stage, int32_t* order, int32_t* bucket_start) {
  const int tiles = static_cast<int>((n_sorted + block - 1) / block);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  __shared__ int32_t s_count[16];
  __shared__ int32_t s_start[16];
  for (int t = warp; t < tiles; t += nwarps) {
    int s = -1;
    for (int64_t r = static_cast<int64_t>(t) * block + lane; r < min(n_sorted, static_cast<int64_t>(t + 1) * block); r += 32) {
      const int id = sorted_ids[r];
      if (id >= 0) s = max(s, pair_stage(id, k, tokens_per_rank, rank, world));
    }
    for (int o = 16; o > 0; o >>= 1) s = max(s, __shfl_xor_sync(0xffffffffu, s, o));
    if (lane == 0) stage[t] = s;
  }
  __syncthreads();
  // pass 1: bucket sizes
  if (warp <= world) {
    int cnt = 0;
    for (int t0 = 0; t0 < tiles; t0 += 32) {
      const int t = t0 + lane;
      const int b = t < tiles ? (stage[t] < 0 ? world : stage[t]) : -1;
      cnt += __popc(__ballot_sync(0xffffffffu, b == warp));
    }
    if (lane == 0) s_count[warp] = cnt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int b = 0; b <= world; ++b) {
      s_start[b] = acc;
      if (bucket_start != nullptr) bucket_start[b] = acc;
      acc += s_count[b];
    }
    if (bucket_start != nullptr) bucket_start[world + 1] = acc;
  }
  __syncthreads();
  // pass 2: stable placement
  if (warp <= world) {
    int base = s_start[warp];
    for (int t0 = 0; t0 < tiles; t0 += 32) {
      const int t = t0 + lane;
      const int b = t < tiles ? (stage[t] < 0 ? world : stage[t]) : -1;
      const unsigned m = __ballot_sync(0xffffffffu, b == warp);
      if (b == warp) order[base + __popc(m & ((1u << lane) - 1u))] = t;
      base += __popc(m);
    }
  }
}

int grid_1d(int64_t n, int threads, int cap) {
  int64_t g = (n + threads - 1) / threads;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

cudaError_t launch_topk_router(const float* logits, int32_t* ids, float* weights, int T, int E, int k, int normalize,
                               cudaStream_t s) {
  if (E > 32 * kMaxPerLane || k > 32 || k > E) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  const int warps = 4;
  topk_router_kernel<<<(T + warps - 1) / warps, warps * 32, 0, s>>>(logits, ids, weights, T, E, k, normalize);
  return cudaGetLastError();
}

cudaError_t launch_moe_align_sort(const int32_t* ids, int64_t n, int E, int align, int32_t* counts, int32_t* offsets,
                                  int32_t* cursor, int32_t* sorted_ids, int64_t sorted_cap, int32_t* pos_of,
                                  int32_t* tile_expert, int max_tiles, int32_t* meta, cudaStream_t s) {
  if (E < 1 || E > 4096 || align < 1) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, s);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(sorted_ids, 0xff, sizeof(int32_t) * sorted_cap, s);   // -1 = padding
  if (e != cudaSuccess) return e;
  if (n > 0) moe_count_kernel<<<grid_1d(n, 256, 592), 256, 0, s>>>(ids, n, E, counts);
  moe_offsets_kernel<<<1, 256, (E + 1) * sizeof(int32_t), s>>>(counts, E, align, offsets, cursor, tile_expert, max_tiles, meta);
  if (n > 0) moe_scatter_kernel<<<grid_1d(n, 256, 592), 256, 0, s>>>(ids, n, E, cursor, sorted_ids, pos_of);
  return cudaGetLastError();
}

cudaError_t launch_moe_align_sort_staged(const int32_t* ids, int64_t n, int E, int align, int k, int tokens_per_rank, int rank,
                                         int world, int32_t* bucket_counts, int32_t* counts, int32_t* offsets,
                                         int32_t* cursor, int32_t* sorted_ids, int64_t sorted_cap, int32_t* pos_of,
                                         int32_t* tile_expert, int max_tiles, int32_t* meta, cudaStream_t s) {
  if (E < 1 || E > 4096 || align < 1 || world < 1 || world > 8 || k < 1 || tokens_per_rank < 1) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(bucket_counts, 0, sizeof(int32_t) * E * world, s);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(sorted_ids, 0xff, sizeof(int32_t) * sorted_cap, s);   // -1 = padding
  if (e != cudaSuccess) return e;
  if (n > 0) moe_count_staged_kernel<<<grid_1d(n, 256, 592), 256, 0, s>>>(ids, n, E, k, tokens_per_rank, rank, world, bucket_counts);
  moe_offsets_staged_kernel<<<1, 256, (E + 1) * sizeof(int32_t), s>>>(bucket_counts, E, world, align, offsets, cursor, counts,
                                                                     tile_expert, max_tiles, meta);
  if (n > 0) moe_scatter_staged_kernel<<<grid_1d(n, 256, 592), 256, 0, s>>>(ids, n, E, k, tokens_per_rank, rank, world, cursor,
                                                                           sorted_ids, pos_of);
  return cudaGetLastError();
}

cudaError_t launch_moe_tile_schedule(const int32_t* sorted_ids, int64_t n_sorted, int k, int tokens_per_rank, int rank, int world,
                                     int block, int32_t* stage, int32_t* order, int32_t* bucket_start, cudaStream_t s) {
  if (world < 1 || world > 8 || block < 1 || k < 1 || tokens_per_rank < 1) return cudaErrorInvalidValue;
  if (n_sorted == 0) return cudaSuccess;
  moe_tile_schedule_kernel<<<1, 1024, 0, s>>>(sorted_ids, n_sorted, k, tokens_per_rank, rank, world, block, stage, order,
                                             bucket_start);
  return cudaGetLastError();
}

cudaError_t launch_moe_gather(const void* src, const int32_t* sorted_ids, const int32_t* meta, void* out, int64_t rows_cap,
                              int H, int k, int64_t src_ld, cudaStream_t s) {
  if (H % 8 != 0 || src_ld % 8 != 0) return cudaErrorInvalidValue;
  if (rows_cap == 0) return cudaSuccess;
  moe_gather_kernel<<<static_cast<unsigned>(rows_cap), 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(src), sorted_ids,
                                                                   meta, reinterpret_cast<__nv_bfloat16*>(out), H, k, src_ld);
  return cudaGetLastError();
}

cudaError_t launch_moe_topk_reduce(const void* y, const int32_t* pos_of, const float* w, void* out, int64_t T, int H, int k,
                                   int64_t out_ld, cudaStream_t s) {
  if (H % 8 != 0 || out_ld % 8 != 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  moe_topk_reduce_kernel<<<static_cast<unsigned>(T), 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(y), pos_of, w,
                                                                 reinterpret_cast<__nv_bfloat16*>(out), H, k, out_ld);
  return cudaGetLastError();
}

cudaError_t launch_moe_unsort(const void* y, const int32_t* pos_of, void* out, int64_t rows, int N, cudaStream_t s) {
  if (N % 8 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  moe_unsort_kernel<<<static_cast<unsigned>(rows), 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(y), pos_of,
                                                               reinterpret_cast<__nv_bfloat16*>(out), N);
  return cudaGetLastError();
}

}  // namespace tdb
