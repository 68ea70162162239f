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

}  // namespace tdb
