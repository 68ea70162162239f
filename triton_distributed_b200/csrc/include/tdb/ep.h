// Host API of the expert-parallel all-to-all kernels (ep_a2a.cu).
#pragma once
#include "api.h"

namespace tdb {

struct EpDispatchArgs {
  const void* x;              // bf16 [T, H] local tokens
  const int32_t* topk_ids;    // [T, k] global expert ids; outside [0, E) = dropped
  int T, H, k, E;
  int quant;                  // 1: rows travel as fp8 e4m3 + one fp32 scale per 128 elements
  int max_tokens;             // per-rank token capacity of the context
  void* recv_x;               // heap [2][rows_per_parity][row bytes]
  float* recv_scale;          // heap [2][rows_per_parity][H/128]
  int32_t* recv_meta;         // heap [2][rows_per_parity]
  int32_t* recv_count;        // heap [2][E/W][W]
  uint32_t* flags;            // heap [W]
  uint64_t rows_per_parity;
  const int32_t* base;        // [W][E/W][W] packed layout offsets, or null for the fixed-stride layout
  int32_t* cursor;            // local [E], zero on entry (the kernel leaves it zero)
  int32_t* sent_row;          // local [T*k]
  int num_ctas;
  int parts = 1;              // warps that share a row (1, 2, 4, 8): more for few rows (latency), 1 for many (throughput)
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_ep_dispatch(const EpDispatchArgs& a, cudaStream_t s);
cudaError_t launch_ep_count(const int32_t* ids, int64_t n, int E, int32_t* counts, cudaStream_t s);
cudaError_t launch_ep_layout(const int32_t* counts_all, int32_t* base, int epr, int W, int E, cudaStream_t s);
cudaError_t launch_ep_recv_ids(const int32_t* recv_count, const int32_t* base_self, int32_t* row_expert, int epr, int W,
                               int max_tokens, int64_t rows, const CtxDev* dispatch_ctx, cudaStream_t s);
cudaError_t launch_ep_gather_rows(const void* recv_x, const float* recv_scale, const int32_t* sorted_ids, const int32_t* meta,
                                  void* out, int64_t rows_cap, int H, int quant, int64_t rows_per_parity,
                                  const CtxDev* dispatch_ctx, cudaStream_t s);

// Receive side of a dispatch in one launch: grouped-GEMM layout (rows sorted by local expert, 128-row padding) built
// from the per-(expert, source) counts, fp8 rows de-quantised on the way.  sorted_ids hold receive-row indices.
struct EpFinishArgs {
  const void* recv_x;
  const float* recv_scale;
  const int32_t* recv_count;  // heap [2][epr][W]
  const int32_t* base_self;   // packed layout [epr * W], or null for the fixed-stride layout
  int epr, W, max_tokens, H, quant;
  int64_t rows_per_parity;
  const CtxDev* dispatch_ctx;
  void* x_sorted;             // bf16 [cap, H]
  int32_t* sorted_ids;        // [cap]
  int32_t* tile_expert;       // [cap / 128]
  int32_t* offsets;           // [epr + 1]
  int32_t* counts;            // [epr]
  int32_t* meta;              // [2]
  int32_t* real_rows;         // [cap + 1] packed list of the sorted rows that carry a token; [cap] = their number
  int64_t cap;                // multiple of 128
  int num_ctas;
  int parts = 1;              // warps per token row
};
cudaError_t launch_ep_finish(const EpFinishArgs& a, cudaStream_t s);

struct EpCombineArgs {
  const void* y;              // bf16 [sorted rows, H]
  const int32_t* pos_of;      // [recv rows]; may be null when sorted_ids is given
  const int32_t* sorted_ids = nullptr;   // [sorted rows] receive row per sorted row (-1 padding) + sort_meta {rows, tiles}:
  const int32_t* sort_meta = nullptr;    //   the send loop walks the sorted rows instead of the receive capacity
  const int32_t* real_rows = nullptr;    // optional, with sorted_ids: EpFinishArgs::real_rows of the matching dispatch
  int64_t real_cap = 0;                  //   and its cap: `parts` warps per token row, nothing is scanned
  int parts = 1;
  const int32_t* recv_meta;   // heap [2][recv rows]
  const CtxDev* dispatch_ctx;
  const int32_t* base_self;   // [E/W * W] packed layout, or null
  int max_tokens;
  int64_t recv_rows;
  void* ret;                  // heap [2][max_tokens*k][H] bf16
  uint64_t ret_half;
  uint32_t* flags;            // heap [W]
  const int32_t* topk_ids;
  const float* topk_w;        // may be null
  void* out;                  // bf16 [T, H]
  int T, H, k, E;
  int num_ctas;
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_ep_combine(const EpCombineArgs& a, cudaStream_t s);

cudaError_t launch_a2a_single(const void* in, void* out, const int32_t* splits_all, int64_t row_bytes, uint32_t* flags,
                              CtxDev* ctx, const SymmInfoHost& symm, int parts, cudaStream_t s);
// Ulysses head-to-sequence exchange: rows [d * s_local, ...) of `in` ([W * s_local][row_bytes], pitch in_pitch) go to
// rank d's out [s_local][W * row_bytes] (heap, one buffer; peers are written only after they have entered the call),
// column block [rank * row_bytes, ...).  flags: heap [2][W].  Returns when all sources' blocks have arrived.
cudaError_t launch_a2a_cols(const void* in, int64_t in_pitch, void* out, uint64_t out_bytes, int64_t row_bytes, int s_local,
                            uint32_t* flags, CtxDev* ctx, const SymmInfoHost& symm, int parts, cudaStream_t s);
cudaError_t launch_fp8_quant(const void* x, void* q, float* scales, int64_t T, int H, cudaStream_t s);
cudaError_t launch_fp8_dequant(const void* q, const float* scales, void* out, int64_t T, int H, cudaStream_t s);

}  // namespace tdb
