// Decode attention for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference library; it exists for one class of callers of THIS
// library: code that runs under somebody else's memory manager.  A plug-in of an inference server, a custom
// op inside a framework whose allocator owns the whole device, or a plain C program that was handed a fixed
// set of buffers and a stream cannot call cudaMalloc (it would bypass the owner's accounting, and it
// synchronises the device in the middle of a serving loop), and it has no torch caching allocator to ask.
// The regular entry point (`decode_attn` in the Python module) needs a workspace tensor for the split-KV
// partial results; here that workspace is a fixed array inside the library image instead.
//
// Contract
//   * Same maths as the regular split-KV decode: q [batch, Hq, D] bf16, paged KV cache
//     [pages, page_size, Hkv, D] bf16, block_table [batch, max_pages] int32, kv_lens [batch] int32,
//     out [batch, Hq, D] bf16.  The caller passes every input and output; only the scratch is internal.
//   * Limit: batch * Hq * splits * (D + 1) must not exceed tdb_decode_attn_noalloc_capacity() floats
//     (1 Mi floats = 4 MiB).  Larger requests are rejected with TDB_NOALLOC_TOO_LARGE and nothing is launched.
//     Every GPU whose context loads the library holds these 4 MiB until the process exits.
//   * The call never calls cudaMalloc / cudaFree or any allocating library routine.
//   * The first call on a device looks up the device address of the scratch array (once per device, with that
//     device current).  Make that first call before starting any stream capture.
//   * All calls share the one array and it keeps the previous call's contents.  Nothing in it has to start at
//     zero: every partial the combine step reads is written by the first step of the same call.  Two calls
//     that overlap on the GPU (different streams, no ordering between them) race on the array; serialise them.
//   * Host threads: the per-device set-up state (array address, shared-memory opt-in of the kernels) is published
//     atomically, so several host threads may call concurrently, each with its own device current; what they must
//     not do is overlap two calls on the SAME device's GPU timeline (previous point).
//   * Returns 0 on success, a negative TDB_NOALLOC_* code otherwise; tdb_noalloc_last_error() gives the text of
//     the last failure on the calling thread.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TDB_NOALLOC_OK = 0,
  TDB_NOALLOC_BAD_ARGUMENT = -1,
  TDB_NOALLOC_TOO_LARGE = -2,
  TDB_NOALLOC_CUDA_ERROR = -3,
};

// Number of floats of scratch available to one call.
int64_t tdb_decode_attn_noalloc_capacity(void);

// `stream` is a cudaStream_t passed as void* (0 = the legacy default stream).
int tdb_decode_attn_noalloc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                            const int32_t* kv_lens, void* out, int batch, int num_q_heads, int num_kv_heads,
                            int head_dim, int page_size, int max_pages, int splits, float scale, float softcap,
                            void* stream);

const char* tdb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
