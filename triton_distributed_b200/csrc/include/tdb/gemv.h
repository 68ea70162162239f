// Host API of the decode GEMV (gemv.cu): out[M, N] = f(x)[M, K] * W[N, K]^T for M <= 16 tokens, with the element-wise
// neighbours of a transformer layer and the tensor-parallel all-reduce folded into the same launch.
#pragma once
#include "api.h"

namespace tdb {

struct GemvArgs {
  int M, N, K;
  const void* x;        // bf16 [M, ldx]; with silu_mul: [M, 2K] as gate | up
  int64_t ldx;
  const void* w;        // bf16 [N, ldw], K contiguous
  int64_t ldw;
  void* out;            // bf16 [M, ld_out]
  int64_t ld_out;
  const void* norm_w;   // bf16 [K] or null: f(x) = rmsnorm(x) * norm_w
  float eps;
  int silu_mul;         // f(x) = silu(x[:, :K]) * x[:, K:]
  const void* residual; // bf16 [M, ld_res] or null, added to the result; may be `out` itself
  int64_t ld_res;
  int num_ctas;
  // all-reduce over the ranks of the heap (sum of the per-rank results before the residual is added)
  int all_reduce;
  int use_multimem;
  void* partial;        // heap: NVLS [2][m_cap][N] bf16; push [2][world][m_cap][N] bf16
  uint32_t* flags;      // heap [world][max_ctas] epochs
  int max_ctas;
  int m_cap;
  CtxDev* ctx;
  SymmInfoHost symm;
};

// Largest K for which M tokens of activations fit the kernel's shared memory.
int gemv_max_k(int M);
cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t stream);

}  // namespace tdb
