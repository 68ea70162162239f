// Status words shared by host and device code.
//
// Every device-side wait in this library is bounded. When a wait gives up, the
// kernel records one StatusRecord in the context's status page (pinned host
// memory mapped into the device), stops waiting, skips the dependent work and
// returns normally, so the CUDA context stays usable and the host wrapper can
// raise an error.  The reference library spins forever in the same places
// (lib/Conversion/TritonDistributedToLLVM/NVIDIA/DistributedOpToLLVM.cpp:146-219).
#pragma once
#include <stdint.h>

namespace tdb {

enum StatusCode : int32_t {
  kOk = 0,
  kTimeoutFlag = 1,      // a flag / signal in global memory never reached the expected value
  kTimeoutMbarrier = 2,  // a shared-memory mbarrier phase never completed
  kTimeoutBarrier = 3,   // a rank or grid barrier never completed
  kBadArgument = 4,      // a bounds / alignment check in a debug build failed
  kAborted = 5,          // the host (or a peer) raised the abort word
};

// Identifiers of the kernels that can report.
enum KernelId : int32_t {
  kKernelNone = 0,
  kKernelGemm = 1,
  kKernelAgGemm = 2,
  kKernelGemmRs = 3,
  kKernelGemmAr = 4,
  kKernelAllReduce = 5,
  kKernelAllGather = 6,
  kKernelReduceScatter = 7,
  kKernelBarrier = 8,
  kKernelA2A = 9,
  kKernelEpDispatch = 10,
  kKernelEpCombine = 11,
  kKernelFlashDecode = 12,
  kKernelMega = 13,
  kKernelGroupGemm = 14,
  kKernelMoeReduce = 15,
  kKernelP2P = 16,
  kKernelPrimitive = 17,
  kKernelGemv = 18,
};

// One record; the first writer wins (code is set with atomicCAS from kOk).
struct StatusRecord {
  int32_t code;      // StatusCode
  int32_t kernel;    // KernelId
  int32_t where;     // kernel-specific site id
  int32_t block;     // blockIdx.x of the reporter
  int32_t peer;      // peer rank / source rank the wait was about, -1 if n/a
  int32_t index;     // tile / chunk / flag index
  int32_t expected;  // value waited for
  int32_t observed;  // last value seen
};

// Layout of the status page: record, then an abort word the host may set.
struct StatusPage {
  StatusRecord rec;
  int32_t abort_word;     // != 0: all spin loops give up with kAborted
  int32_t heartbeat;      // bumped by kernels that want a liveness signal
  int32_t reserved[6];
};

}  // namespace tdb
