// Symmetric heap built directly on the CUDA virtual-memory API:
//   * one physical allocation per rank (cuMemCreate, POSIX-FD shareable),
//   * every rank maps every peer's allocation into one contiguous VA window
//     (rank r's heap lives at window + r * heap_bytes),
//   * optionally one NVLS multicast object bound to all ranks' allocations and
//     mapped once more (stores reach every rank, multimem.ld_reduce sums them),
//   * a pinned, device-visible status page for bounded-wait reporting.
// File descriptors travel between the local processes over abstract Unix
// datagram sockets (SCM_RIGHTS).  Collective steps are split into phases; the
// caller (Python, over torch.distributed) puts a barrier between phases.
//
// Takes the place of the NVSHMEM symmetric heap the reference allocates with
// nvshmem_create_tensor (python/triton_dist/utils.py:114-142) and of
// nvshmem_ptr / mc_ptr pointer translation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "api.h"

namespace tdb {

class SymmHeap {
 public:
  SymmHeap(int rank, int world, int device, uint64_t heap_bytes, const std::string& session, bool want_multicast);
  ~SymmHeap();

  // phase 1: physical allocation, VA window, listening socket.  Local only.
  void create();
  // phase 2 (after a barrier): send this rank's FD to every peer, receive theirs, map them.
  void exchange_and_map();
  // phase 3 (after a barrier): rank 0 creates the multicast object and sends it; all add their device.
  void multicast_setup();
  // phase 4 (after a barrier): bind local memory, map the multicast window.
  void multicast_bind();
  // legacy CUDA-IPC mode (no multicast): handles are exchanged by the caller.
  void create_ipc();
  std::string ipc_handle() const;
  void map_ipc(const std::vector<std::string>& handles);

  // teardown (local; call after a barrier while all ranks are alive)
  void destroy();

  // symmetric allocator: every rank must issue the same sequence of calls
  uint64_t alloc(uint64_t bytes, uint64_t align);
  void free(uint64_t offset);

  uint64_t local_base() const { return peer_base_[rank_]; }
  uint64_t peer_base(int r) const { return peer_base_[r]; }
  uint64_t mc_base() const { return mc_base_; }
  uint64_t heap_bytes() const { return bytes_; }
  bool has_multicast() const { return mc_base_ != 0; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  StatusPage* status_host() const { return status_host_; }
  SymmInfoHost info(uint64_t timeout_ns) const;
  uint64_t bytes_in_use() const { return in_use_; }
  const std::string& mode() const { return mode_; }

 private:
  int rank_, world_, device_;
  uint64_t bytes_;
  std::string session_;
  bool want_mc_;
  std::string mode_;  // "vmm", "ipc" or ""
  CUmemGenericAllocationHandle local_handle_ = 0;
  CUmemGenericAllocationHandle mc_handle_ = 0;
  bool mc_bound_ = false;
  std::vector<CUmemGenericAllocationHandle> peer_handles_;
  CUdeviceptr window_ = 0;
  CUdeviceptr mc_window_ = 0;
  uint64_t peer_base_[kMaxRanksHost] = {0};
  uint64_t mc_base_ = 0;
  int sock_ = -1;
  int local_fd_ = -1;
  void* ipc_ptr_ = nullptr;
  std::vector<void*> ipc_peer_ptrs_;
  StatusPage* status_host_ = nullptr;
  StatusPage* status_dev_ = nullptr;
  // allocator state: offset -> size of live blocks, and a sorted free list
  std::map<uint64_t, uint64_t> live_;
  std::map<uint64_t, uint64_t> free_;
  uint64_t in_use_ = 0;

  void alloc_status_page();
  void send_fd(int peer, int fd, int kind);
  int recv_fd(int* src, int* kind);
};

// Stream memory operations (the reference's wait_eq / set_signal helpers,
// python/triton_dist/kernels/nvidia/common_ops.py:347-397).
int stream_write_value32(uint64_t addr, uint32_t value, cudaStream_t stream);
int stream_wait_value32_geq(uint64_t addr, uint32_t value, cudaStream_t stream);
int stream_wait_value32_eq(uint64_t addr, uint32_t value, cudaStream_t stream);

}  // namespace tdb
