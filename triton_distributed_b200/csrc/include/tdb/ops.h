// Host API of the memory-bound single-GPU kernels (ops.cu).  bf16 activations.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tdb {

// out[T,H] = rmsnorm(x (+ residual)) * w; residual (may be null) is updated in place to x + residual.
cudaError_t launch_rmsnorm(const void* x, void* residual, const void* w, void* out, int64_t T, int H, int64_t ldx,
                           float eps, cudaStream_t s);
// out[T,I] = silu(in[:, :I]) * in[:, I:2I]
cudaError_t launch_silu_mul(const void* in, void* out, int64_t T, int I, int64_t ld_in, cudaStream_t s);
cudaError_t launch_add(const void* a, const void* b, void* out, int64_t n, cudaStream_t s);
// Packed qkv rows -> normed+rotated q, and k / v written into a slot-addressed cache of `cache_rows` rows; tokens whose
// slot is negative or >= cache_rows are not stored.
cudaError_t launch_qk_norm_rope_kv(const void* qkv, const void* qw, const void* kw, const int64_t* positions,
                                   const int64_t* slots, void* q_out, void* k_cache, void* v_cache, int T, int Hq,
                                   int Hkv, int D, int64_t ld_qkv, float eps, float rope_theta,
                                   int64_t cache_slot_stride, int64_t cache_rows, cudaStream_t s);
cudaError_t launch_embedding(const int64_t* ids, const void* table, void* out, int64_t T, int H, int64_t vocab,
                             cudaStream_t s);
cudaError_t launch_argmax(const float* logits, int64_t* out, int64_t B, int64_t V, cudaStream_t s);
cudaError_t launch_abs_sum(const void* x, int64_t n, float* out, cudaStream_t s);

}  // namespace tdb
