// Kernel launch helpers shared by the .cu files.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

namespace tdb {

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of a kernel ON ONE DEVICE.  One object per
// kernel remembers, one bit per device ordinal, where it has been set; safe to call from several host threads.
struct SmemOptIn {
  std::atomic<unsigned long long> done{0};
  template <typename K>
  cudaError_t ensure(K kernel, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return e;
  }
};

// Launch with the programmatic-dependent-launch attribute: the kernel may be scheduled while its predecessor in the
// stream drains, and must execute griddepcontrol.wait (pdl_wait) before touching anything the predecessor writes.
// TDB200_PDL=0 turns the attribute off (the kernels' waits are then no-ops).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool pdl = [] {
    const char* e = std::getenv("TDB200_PDL");
    return e == nullptr || std::atoi(e) != 0;
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Cooperative launch: the kernel starts only when ALL of its CTAs can be resident at once, and the launch fails (instead
// of deadlocking later) when the grid exceeds what the device can hold.  For kernels whose CTAs wait for one another
// inside a rank (scoreboards, grid-wide counters).  TDB200_COOP=0 falls back to a plain launch.
template <typename... KArgs, typename... Args>
cudaError_t launch_coop(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool coop = [] {
    const char* e = std::getenv("TDB200_COOP");
    return e == nullptr || std::atoi(e) != 0;
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = coop ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tdb
