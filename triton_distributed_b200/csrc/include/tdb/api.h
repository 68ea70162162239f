// Host-side C++ API of the native library: launchers take raw device pointers
// and a CUDA stream, never allocate, and return a cudaError_t (0 = success).
// The torch binding (bind.cc) and the C entry points are thin wrappers.
#pragma once
#include <cstdlib>
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.h"

namespace tdb {

constexpr int kMaxRanksHost = 8;

// Host mirror of the device-side SymmInfo (symm_device.cuh).
struct SymmInfoHost {
  uint64_t peer_base[kMaxRanksHost];
  uint64_t mc_base;
  uint64_t heap_bytes;
  StatusPage* status;
  int32_t rank;
  int32_t world;
  uint64_t timeout_ns;
  uint32_t debug;      // TDB200_DEBUG: device primitives check heap ranges and peer ranks
  uint32_t pad_;
};

// 128-byte opaque CUtensorMap image.
struct alignas(64) TensorMap {
  unsigned char bytes[128];
};

enum DType : int { kBF16 = 0, kF16 = 1, kF32 = 2, kE4M3 = 3, kU8 = 4, kI32 = 5 };

// 2-D row-major tensor [rows, cols] with `row_stride_bytes`; box = [box_rows, box_cols];
// swizzle_bytes in {0, 32, 64, 128}.  Returns 0 on success, CUresult otherwise.
int encode_tensor_map_2d(TensorMap* out, const void* base, DType dtype, uint64_t rows, uint64_t cols,
                         uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle_bytes);
// 3-D [d2, rows, cols] (used for grouped / batched weights).
int encode_tensor_map_3d(TensorMap* out, const void* base, DType dtype, uint64_t d2, uint64_t rows, uint64_t cols,
                         uint64_t row_stride_bytes, uint64_t d2_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                         int swizzle_bytes);

// Per-context device state of the fused kernels: call epoch (bumped by the last
// CTA of every launch, so CUDA-graph replays advance it) and a CTA exit counter.
struct CtxDev {
  uint32_t epoch;
  uint32_t done;
  uint32_t grid_bar;   // word for in-kernel grid barriers
  uint32_t pad[5];
};

// ---------------------------------------------------------------------------
// GEMM family (gemm_sm100.cu): C[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate.
// ---------------------------------------------------------------------------
enum GemmMode : int { kGemmPlain = 0, kGemmAllGather = 1, kGemmReduceScatter = 2 };

struct GemmArgs {
  int mode;
  int M, N, K;
  // plain: output
  void* c;          // bf16 [M, ldc]
  int64_t ldc;
  // tensor maps: A tiles [128 x 64], B tiles [BN x 64], 128-byte swizzle
  TensorMap tmap_a;
  TensorMap tmap_b;
  // output through shared memory + TMA store: C as [segments][rows per segment][N], box [128 x 64], 128-byte swizzle;
  // reduce-scatter: one map per owner rank over its slots [2*world][rows per segment][N]
  TensorMap tmap_c;
  TensorMap tmap_a_local;   // all-gather: the local shard [seg_rows, K], read in place
  TensorMap tmap_peer_c[kMaxRanksHost];
  TensorMap tmap_out;       // reduce-scatter with the pair kernel: the output [1][seg_rows][N], box [128 x 64]
  TensorMap tmap_b_half;    // pair kernel with split_tail: B with a 64-row box (half-width tail tiles)
  int split_tail;           // pair kernel: compute an incomplete last wave as 256 x 128 half tiles
  void* stats;              // optional device buffer [num_ctas][8] of uint64 stall counters (cycles), null = off
  int use_tma_store;
  int block_n;      // 128 or 256
  int cta_pair;     // 1: CTA-pair kernel (256 x 256 tiles over two SMs); tmap_b then has a 128-row box
  int num_ctas;     // grid size (<= SM count)
  // fused modes
  int seg_rows;     // rows per rank segment (M = world * seg_rows)
  int max_seg_rows; // capacity the context was created with (per segment)
  int n_comm_ctas;  // all-gather: CTAs that only push
  const void* a_local;   // all-gather: local shard [seg_rows, K]
  void* ag_ws;           // all-gather: heap workspace [2][world*max_seg_rows][K]
  uint32_t* ag_flags;    // heap, [2][world][max_chunks]
  int max_chunks;
  void* rs_slots;        // reduce-scatter: heap [2][world][max_seg_rows][N]
  uint32_t* rs_flags;    // heap [2][world][max_tiles]
  int max_tiles;
  void* rs_out;          // [seg_rows, N] bf16
  int64_t ld_out;
  const int32_t* tile_expert;  // grouped GEMM (plain mode): expert of each 128-row tile (B is [experts][N][K]), <0 skips
  CtxDev* ctx;           // device memory
  SymmInfoHost symm;
  int use_multimem;      // all-gather push through the multicast mapping
};
cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream);
int gemm_smem_bytes(int block_n);

// ---------------------------------------------------------------------------
// Block-scaled fp8 GEMM (gemm_fp8_sm100.cu): e4m3 operands, fp32 scales 1 x 128 for A rows and 128 x 128 for B,
// bf16 output; plain / all-gather / reduce-scatter modes with the protocols of the bf16 pair kernel.
// ---------------------------------------------------------------------------
struct GemmFp8Args {
  int mode;                 // GemmMode
  int M, N, K;              // K a multiple of 128
  void* c;                  // bf16 [M, ldc] (plain / all-gather)
  int64_t ldc;
  const float* a_scales;    // [M, K/128] (plain / reduce-scatter)
  const float* b_scales;    // [ceil(N/128), K/128]
  TensorMap tmap_a;         // e4m3 as bytes: [d2][rows][K], box [128 x 128], 128-byte swizzle
  TensorMap tmap_b;         // [1][N][K], box [128 x 128]
  TensorMap tmap_a_local;   // all-gather: local shard [1][seg_rows][K]
  TensorMap tmap_peer_c[kMaxRanksHost];   // reduce-scatter: per owner rank, its slots [2*world][rows][N] bf16, box [128 x 64]
  int num_ctas;
  int seg_rows, max_seg_rows, n_comm_ctas;
  const void* a_local;          // all-gather: local e4m3 shard [seg_rows, K]
  const float* a_scales_local;  // [seg_rows, K/128]
  void* ag_ws;                  // heap [2][world*max_seg_rows][K] bytes
  float* ag_ws_scales;          // heap [2][world*max_seg_rows][K/128]
  uint32_t* ag_flags;           // heap [2][world][max_chunks]
  int max_chunks;
  void* rs_slots;               // heap [2][world][max_seg_rows][N] bf16
  uint32_t* rs_flags;           // heap [2][world][max_tiles] (one per 128 x 128 unit)
  int max_tiles;
  void* rs_out;                 // bf16 [seg_rows, ld_out]
  int64_t ld_out;
  CtxDev* ctx;
  SymmInfoHost symm;
  void* stats;
};
cudaError_t launch_gemm_fp8(const GemmFp8Args& a, cudaStream_t stream);

// ---------------------------------------------------------------------------
// Small-M GEMM with split-K and optional fused all-reduce (gemm_ar_sm100.cu):
// out[M,N] = (sum over ranks) X[M,K] * W[N,K]^T, M <= 256.
// ---------------------------------------------------------------------------
struct SkinnyGemmArgs {
  int M, N, K;
  TensorMap tmap_w;        // W [N, K], box [128 x 64], 128-byte swizzle
  TensorMap tmap_x;        // X [M, K], box [M_pad x 64], 128-byte swizzle
  void* out;               // bf16 [M, ld_out]
  int64_t ld_out;
  int splits;              // 0: automatic (cluster form where it fits); >= 1: stream-K form, about this many pieces per
                           // column tile
  int cluster_nt;          // cluster form: CTA tile width in units of 128 columns (1..4), 0 = chosen by the launcher
  int cluster_s;           // cluster form: CTAs per tile (1..8), 0 = chosen by the launcher
  int bulk_exchange;       // cluster form: 1 = parts travel as bulk copies into the reducing CTA's shared memory,
                           // 0 = the reducing CTA loads them from its peers' shared memory
  int num_ctas;
  float* acc;              // fp32 [m_cap, N], all zero between calls
  uint32_t* counters;      // [ceil(N/128)], zero between calls
  int all_reduce;
  int use_multimem;
  void* partial;           // heap: NVLS [2][m_cap][N] bf16, push [2][world][m_cap][N] bf16
  uint32_t* flags;         // heap [world][max_tiles]
  int max_tiles;
  int m_cap;
  CtxDev* ctx;
  SymmInfoHost symm;
};
cudaError_t launch_skinny_gemm(const SkinnyGemmArgs& a, cudaStream_t stream);
int skinny_gemm_mpad(int M);
int skinny_gemm_pick_splits(int N, int K, int num_sms, int M);

}  // namespace tdb
