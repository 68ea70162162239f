// Host API of the attention kernels (attn.cu).  bf16 q / k / v, paged KV cache.
#pragma once
#include "api.h"

namespace tdb {

// Paged cache: k_cache / v_cache [num_pages, page_size, num_kv_heads, head_dim]; block_table [batch, max_pages].
// A dense cache [batch, max_len, Hkv, D] is the special case page_size = max_len, block_table[b] = {b}.
struct AttnKV {
  const void* k_cache;
  const void* v_cache;
  const int32_t* block_table;
  int max_pages;
  int page_size;
  int num_kv_heads;
};

struct FlashFwdArgs {
  const void* q;             // [total_q, Hq, D]
  void* out;                 // [total_q, Hq, D]
  float* lse;                // [Hq, total_q] or null
  const int32_t* cu_seqlens_q;  // [batch + 1]
  const int32_t* q_pos0;     // [batch] absolute position of each sequence's first query row; null = kv_len - q_len
  const int32_t* kv_lens;    // [batch]
  AttnKV kv;
  int batch, max_q_len, num_q_heads, head_dim;
  int64_t total_q;
  int causal;
  float scale, softcap;
};
cudaError_t launch_flash_fwd(const FlashFwdArgs& a, cudaStream_t stream);

// Prefill on tcgen05 (attn_sm100.cu): head dim 128.  The launcher first packs the visible KV into dense tensors
// (k_dense [batch * Hkv][Lp][128], vt_dense [batch * Hkv][128][Lp], both caller-provided scratch, Lp a multiple of 64 and
// >= the longest kv_len), then runs the attention kernel.  error_flag (device int, may be null) is set if a bounded wait
// inside the kernel gave up.
struct FlashFwdSm100Args {
  const void* q;
  void* out;
  float* lse;
  const int32_t* cu_seqlens_q;
  const int32_t* q_pos0;
  const int32_t* kv_lens;
  AttnKV kv;
  int batch, max_q_len, num_q_heads, num_kv_heads, head_dim;
  int64_t total_q;
  int causal;
  float scale;
  int Lp;
  void* k_dense;
  void* vt_dense;
  int* error_flag;
};
cudaError_t launch_flash_fwd_sm100(const FlashFwdSm100Args& a, cudaStream_t stream);

struct DecodeArgs {
  const void* q;             // [batch, Hq, D]
  float* workspace;          // decode_workspace_floats(...) floats: partial out, then partial LSE
  const int32_t* kv_lens;    // [batch]
  AttnKV kv;
  int batch, num_q_heads, head_dim, splits;
  float scale, softcap;
  // Optional fused combine: with both set, the CTA that finishes last for a (sequence, KV head) merges the split
  // partials of its query heads into fuse_out (bf16 [batch, Hq, D]) and no combine launch is needed.
  uint32_t* fuse_counters = nullptr;   // [batch * Hkv * head_chunks], zero between calls (the kernel leaves them zero)
  void* fuse_out = nullptr;
};
int decode_workspace_floats(int batch, int num_q_heads, int head_dim, int splits);
cudaError_t launch_decode_splitkv(const DecodeArgs& a, cudaStream_t stream);
// out_bf16 [B,Hq,D] and/or out_lse [B,Hq] and/or out_f32 [B,Hq,D+1] (out || LSE); any may be null.
cudaError_t launch_decode_combine(const DecodeArgs& a, void* out_bf16, float* out_lse, float* out_f32,
                                  cudaStream_t stream);
// Distributed tail: staging = heap, 2 * staging_half_packets packets of 8 bytes.
cudaError_t launch_dist_combine(const DecodeArgs& a, void* out_bf16, void* staging, int64_t staging_half_packets,
                                CtxDev* ctx, const SymmInfoHost& symm, cudaStream_t stream);

// The whole distributed flash-decode step in one launch (a.fuse_counters and a.fuse_out must be set): usable while
// batch x KV heads x head chunks <= SM count, cudaErrorInvalidValue otherwise.
cudaError_t launch_dist_decode_fused(const DecodeArgs& a, void* staging, int64_t staging_half_packets, CtxDev* ctx,
                                     const SymmInfoHost& symm, cudaStream_t stream);

}  // namespace tdb
