// Host API of the gated delta rule forward (gdn.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace tdb {

struct GdnArgs {
  const void* q;              // bf16 [T_total, H, K], K = 128
  const void* k;              // bf16 [T_total, H, K]
  const void* v;              // bf16 [T_total, H, V], V a multiple of 32
  const float* g;             // fp32 [T_total, H], log of the per-token decay
  const void* beta;           // bf16 [T_total, H]
  void* o;                    // bf16 [T_total, H, V]
  const float* initial_state; // fp32 [N, H, K, V] or null
  float* final_state;         // fp32 [N, H, K, V] or null
  const int32_t* cu_seqlens;  // int32 [N + 1], device memory
  int num_seqs, H, K, V;
  float scale;
};
cudaError_t launch_gdn_fwd(const GdnArgs& a, cudaStream_t stream);

// Chunk-parallel form (gdn_chunk.cu): 64-token chunks, three launches (per-chunk WY factors, sequential state pass,
// per-chunk output), tensor-core products.  The chunk tables come from the host (cu_seqlens is known there).
struct GdnChunkArgs {
  const void* q;              // bf16 [T_total, H, 128]
  const void* k;
  const void* v;              // bf16 [T_total, H, V], V in {64, 128, 192, 256}
  const float* g;             // fp32 [T_total, H]
  const void* beta;           // bf16 [T_total, H]
  const int32_t* cu_seqlens;  // [N + 1] device
  const int32_t* chunk_seq;   // [NC] sequence of every chunk
  const int32_t* chunk_t0;    // [NC] first token of every chunk
  const int32_t* seq_chunk0;  // [N + 1] first chunk of every sequence
  float* g_cumsum;            // out fp32 [T_total, H]
  float* a_out;               // out fp32 [T_total, H, 64] or null
  void* w;                    // scratch bf16 [NC, H, 64, 128]
  void* u;                    // scratch bf16 [NC, H, 64, V]
  void* v_new;                // scratch bf16 [NC, H, 64, V]
  void* h_chunks;             // scratch bf16 [NC, H, 128, V]
  const float* initial_state; // fp32 [N, H, 128, V] or null
  float* final_state;         // fp32 [N, H, 128, V] or null
  void* o;                    // out bf16 [T_total, H, V]
  int num_seqs, num_chunks, H, K, V;
  float scale;
};
cudaError_t launch_gdn_chunk_fwd(const GdnChunkArgs& a, cudaStream_t stream);

}  // namespace tdb
