// Symmetric heap over cuMem + NVLS multicast; see tdb/symm_heap.h.
#include "tdb/symm_heap.h"

#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "tdb/driver.h"

namespace tdb {

namespace {

[[noreturn]] void fail(const std::string& what, long code) {
  throw std::runtime_error("symm_heap: " + what + " failed with code " + std::to_string(code));
}

#define DRV(name, ...)                                                    \
  do {                                                                    \
    auto fn_ = TDB_DRIVER_FN(name);                                       \
    if (fn_ == nullptr) fail(#name " (driver entry point missing)", -1);  \
    CUresult r_ = fn_(__VA_ARGS__);                                       \
    if (r_ != CUDA_SUCCESS) fail(#name, static_cast<long>(r_));           \
  } while (0)

#define RT(expr)                                                   \
  do {                                                             \
    cudaError_t e_ = (expr);                                       \
    if (e_ != cudaSuccess) fail(#expr, static_cast<long>(e_));     \
  } while (0)

uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

sockaddr_un abstract_addr(const std::string& session, int rank, socklen_t* len) {
  sockaddr_un a;
  std::memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  const std::string name = "tdb200." + session + "." + std::to_string(rank);
  // abstract namespace: leading NUL, no file on disk
  std::memcpy(a.sun_path + 1, name.data(), std::min(name.size(), sizeof(a.sun_path) - 2));
  *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  return a;
}

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

void set_access(CUdeviceptr p, uint64_t bytes, int device) {
  CUmemAccessDesc d;
  std::memset(&d, 0, sizeof(d));
  d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  d.location.id = device;
  d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV(cuMemSetAccess, p, bytes, &d, 1);
}

}  // namespace

SymmHeap::SymmHeap(int rank, int world, int device, uint64_t heap_bytes, const std::string& session,
                   bool want_multicast)
    : rank_(rank), world_(world), device_(device), bytes_(heap_bytes), session_(session), want_mc_(want_multicast) {
  if (world < 1 || world > kMaxRanksHost) throw std::runtime_error("symm_heap: world size must be 1..8");
  if (rank < 0 || rank >= world) throw std::runtime_error("symm_heap: bad rank");
}

SymmHeap::~SymmHeap() {
  try {
    destroy();
  } catch (...) {
  }
}

void SymmHeap::alloc_status_page() {
  void* h = nullptr;
  RT(cudaHostAlloc(&h, sizeof(StatusPage), cudaHostAllocMapped | cudaHostAllocPortable));
  std::memset(h, 0, sizeof(StatusPage));
  void* d = nullptr;
  RT(cudaHostGetDevicePointer(&d, h, 0));
  status_host_ = reinterpret_cast<StatusPage*>(h);
  status_dev_ = reinterpret_cast<StatusPage*>(d);
}

void SymmHeap::create() {
  RT(cudaSetDevice(device_));
  RT(cudaFree(nullptr));  // make sure the primary context exists
  CUmemAllocationProp prop = alloc_prop(device_);
  size_t gran = 0;
  DRV(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (want_mc_ && world_ > 1) {
    int supported = 0;
    CUdevice dev;
    DRV(cuDeviceGet, &dev, device_);
    DRV(cuDeviceGetAttribute, &supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
    if (!supported) want_mc_ = false;
  } else {
    want_mc_ = false;
  }
  if (want_mc_) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = world_;
    mp.size = bytes_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    DRV(cuMulticastGetGranularity, &mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (mg > gran) gran = mg;
  }
  bytes_ = round_up(bytes_, gran);
  DRV(cuMemCreate, &local_handle_, bytes_, &prop, 0);
  DRV(cuMemAddressReserve, &window_, bytes_ * world_, gran, 0, 0);
  for (int r = 0; r < world_; ++r) peer_base_[r] = window_ + static_cast<uint64_t>(r) * bytes_;
  DRV(cuMemMap, peer_base_[rank_], bytes_, 0, local_handle_, 0);
  set_access(peer_base_[rank_], bytes_, device_);
  RT(cudaMemset(reinterpret_cast<void*>(peer_base_[rank_]), 0, bytes_));
  RT(cudaDeviceSynchronize());
  peer_handles_.assign(world_, 0);
  peer_handles_[rank_] = local_handle_;
  alloc_status_page();
  free_.clear();
  free_[0] = bytes_;
  mode_ = "vmm";
  if (world_ > 1) {
    int fd = -1;
    DRV(cuMemExportToShareableHandle, &fd, local_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    local_fd_ = fd;
    sock_ = ::socket(AF_UNIX, SOCK_DGRAM, 0);
    if (sock_ < 0) fail("socket", errno);
    socklen_t len;
    sockaddr_un a = abstract_addr(session_, rank_, &len);
    if (::bind(sock_, reinterpret_cast<sockaddr*>(&a), len) != 0) fail("bind", errno);
    timeval tv;
    tv.tv_sec = 60;
    tv.tv_usec = 0;
    ::setsockopt(sock_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  }
}

void SymmHeap::send_fd(int peer, int fd, int kind) {
  socklen_t len;
  sockaddr_un a = abstract_addr(session_, peer, &len);
  int payload[2] = {rank_, kind};
  iovec iov;
  iov.iov_base = payload;
  iov.iov_len = sizeof(payload);
  char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  std::memset(&msg, 0, sizeof(msg));
  msg.msg_name = &a;
  msg.msg_namelen = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  if (::sendmsg(sock_, &msg, 0) < 0) fail("sendmsg", errno);
}

int SymmHeap::recv_fd(int* src, int* kind) {
  int payload[2] = {-1, -1};
  iovec iov;
  iov.iov_base = payload;
  iov.iov_len = sizeof(payload);
  char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  std::memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (::recvmsg(sock_, &msg, 0) < 0) fail("recvmsg", errno);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (c == nullptr || c->cmsg_type != SCM_RIGHTS) fail("recvmsg (no descriptor attached)", 0);
  int fd = -1;
  std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
  *src = payload[0];
  *kind = payload[1];
  return fd;
}

void SymmHeap::exchange_and_map() {
  if (world_ == 1) return;
  for (int i = 1; i < world_; ++i) send_fd((rank_ + i) % world_, local_fd_, 0);
  for (int i = 1; i < world_; ++i) {
    int src = -1, kind = -1;
    const int fd = recv_fd(&src, &kind);
    if (src < 0 || src >= world_ || kind != 0) fail("descriptor exchange (unexpected message)", src);
    DRV(cuMemImportFromShareableHandle, &peer_handles_[src], reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    DRV(cuMemMap, peer_base_[src], bytes_, 0, peer_handles_[src], 0);
    set_access(peer_base_[src], bytes_, device_);
  }
  ::close(local_fd_);
  local_fd_ = -1;
}

void SymmHeap::multicast_setup() {
  if (!want_mc_) return;
  if (rank_ == 0) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = world_;
    mp.size = bytes_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    DRV(cuMulticastCreate, &mc_handle_, &mp);
    int fd = -1;
    DRV(cuMemExportToShareableHandle, &fd, mc_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    for (int p = 1; p < world_; ++p) send_fd(p, fd, 1);
    ::close(fd);
  } else {
    int src = -1, kind = -1;
    const int fd = recv_fd(&src, &kind);
    if (src != 0 || kind != 1) fail("multicast handle exchange (unexpected message)", src);
    DRV(cuMemImportFromShareableHandle, &mc_handle_, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
  }
  CUdevice dev;
  DRV(cuDeviceGet, &dev, device_);
  DRV(cuMulticastAddDevice, mc_handle_, dev);
}

void SymmHeap::multicast_bind() {
  if (!want_mc_) return;
  DRV(cuMulticastBindMem, mc_handle_, 0, local_handle_, 0, bytes_, 0);
  mc_bound_ = true;
  CUmemAllocationProp prop = alloc_prop(device_);
  size_t gran = 0;
  DRV(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  DRV(cuMemAddressReserve, &mc_window_, bytes_, gran, 0, 0);
  DRV(cuMemMap, mc_window_, bytes_, 0, mc_handle_, 0);
  set_access(mc_window_, bytes_, device_);
  mc_base_ = mc_window_;
}

void SymmHeap::create_ipc() {
  RT(cudaSetDevice(device_));
  bytes_ = round_up(bytes_, 2ull << 20);
  RT(cudaMalloc(&ipc_ptr_, bytes_));
  RT(cudaMemset(ipc_ptr_, 0, bytes_));
  RT(cudaDeviceSynchronize());
  peer_base_[rank_] = reinterpret_cast<uint64_t>(ipc_ptr_);
  alloc_status_page();
  free_.clear();
  free_[0] = bytes_;
  want_mc_ = false;
  mode_ = "ipc";
}

std::string SymmHeap::ipc_handle() const {
  cudaIpcMemHandle_t h;
  RT(cudaIpcGetMemHandle(&h, ipc_ptr_));
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void SymmHeap::map_ipc(const std::vector<std::string>& handles) {
  if (static_cast<int>(handles.size()) != world_) fail("map_ipc (handle count)", handles.size());
  ipc_peer_ptrs_.assign(world_, nullptr);
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    cudaIpcMemHandle_t h;
    if (handles[r].size() != sizeof(h)) fail("map_ipc (handle size)", handles[r].size());
    std::memcpy(&h, handles[r].data(), sizeof(h));
    void* p = nullptr;
    RT(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    ipc_peer_ptrs_[r] = p;
    peer_base_[r] = reinterpret_cast<uint64_t>(p);
  }
}

void SymmHeap::destroy() {
  if (mode_.empty()) return;
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  if (mode_ == "ipc") {
    for (void* p : ipc_peer_ptrs_)
      if (p != nullptr) cudaIpcCloseMemHandle(p);
    ipc_peer_ptrs_.clear();
    if (ipc_ptr_ != nullptr) cudaFree(ipc_ptr_);
    ipc_ptr_ = nullptr;
  } else {
    auto unmap = TDB_DRIVER_FN(cuMemUnmap);
    auto release = TDB_DRIVER_FN(cuMemRelease);
    auto addr_free = TDB_DRIVER_FN(cuMemAddressFree);
    auto unbind = TDB_DRIVER_FN(cuMulticastUnbind);
    if (unmap != nullptr && release != nullptr && addr_free != nullptr) {
      if (mc_window_ != 0) {
        unmap(mc_window_, bytes_);
        addr_free(mc_window_, bytes_);
        mc_window_ = 0;
        mc_base_ = 0;
      }
      if (mc_bound_ && unbind != nullptr) {
        CUdevice dev;
        auto devget = TDB_DRIVER_FN(cuDeviceGet);
        if (devget != nullptr && devget(&dev, device_) == CUDA_SUCCESS) unbind(mc_handle_, dev, 0, bytes_);
        mc_bound_ = false;
      }
      if (mc_handle_ != 0) {
        release(mc_handle_);
        mc_handle_ = 0;
      }
      for (int r = 0; r < world_; ++r) {
        if (peer_handles_.size() > static_cast<size_t>(r) && peer_handles_[r] != 0) {
          unmap(peer_base_[r], bytes_);
          release(peer_handles_[r]);
          peer_handles_[r] = 0;
        }
      }
      if (window_ != 0) {
        addr_free(window_, bytes_ * world_);
        window_ = 0;
      }
    }
  }
  if (sock_ >= 0) ::close(sock_);
  sock_ = -1;
  if (local_fd_ >= 0) ::close(local_fd_);
  local_fd_ = -1;
  if (status_host_ != nullptr) cudaFreeHost(status_host_);
  status_host_ = nullptr;
  status_dev_ = nullptr;
  mode_.clear();
}

uint64_t SymmHeap::alloc(uint64_t bytes, uint64_t align) {
  if (align < 256) align = 256;
  bytes = round_up(bytes == 0 ? 1 : bytes, 256);
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    const uint64_t start = round_up(it->first, align);
    const uint64_t end = it->first + it->second;
    if (start + bytes <= end) {
      const uint64_t blk_off = it->first, blk_end = end;
      free_.erase(it);
      if (start > blk_off) free_[blk_off] = start - blk_off;
      if (start + bytes < blk_end) free_[start + bytes] = blk_end - (start + bytes);
      live_[start] = bytes;
      in_use_ += bytes;
      return start;
    }
  }
  throw std::runtime_error("symm_heap: out of symmetric memory (requested " + std::to_string(bytes) + " bytes, " +
                           std::to_string(bytes_ - in_use_) + " free of " + std::to_string(bytes_) +
                           "); raise TDB200_SYMM_HEAP_BYTES");
}

void SymmHeap::free(uint64_t offset) {
  auto it = live_.find(offset);
  if (it == live_.end()) throw std::runtime_error("symm_heap: free of an offset that is not allocated");
  uint64_t off = it->first, sz = it->second;
  live_.erase(it);
  in_use_ -= sz;
  // coalesce with the following and the preceding free block
  auto nxt = free_.lower_bound(off);
  if (nxt != free_.end() && nxt->first == off + sz) {
    sz += nxt->second;
    nxt = free_.erase(nxt);
  }
  if (nxt != free_.begin()) {
    auto prv = std::prev(nxt);
    if (prv->first + prv->second == off) {
      off = prv->first;
      sz += prv->second;
      free_.erase(prv);
    }
  }
  free_[off] = sz;
}

SymmInfoHost SymmHeap::info(uint64_t timeout_ns) const {
  SymmInfoHost s;
  std::memset(&s, 0, sizeof(s));
  for (int r = 0; r < world_; ++r) s.peer_base[r] = peer_base_[r];
  s.mc_base = mc_base_;
  s.heap_bytes = bytes_;
  s.status = status_dev_;
  s.rank = rank_;
  s.world = world_;
  s.timeout_ns = timeout_ns;
  static const bool debug = [] {
    const char* e = std::getenv("TDB200_DEBUG");
    return e != nullptr && std::atoi(e) != 0;
  }();
  s.debug = debug ? 1u : 0u;
  return s;
}

int stream_write_value32(uint64_t addr, uint32_t value, cudaStream_t stream) {
  auto fn = TDB_DRIVER_FN(cuStreamWriteValue32);
  if (fn == nullptr) return -1;
  return static_cast<int>(fn(reinterpret_cast<CUstream>(stream), addr, value, CU_STREAM_WRITE_VALUE_DEFAULT));
}
int stream_wait_value32_geq(uint64_t addr, uint32_t value, cudaStream_t stream) {
  auto fn = TDB_DRIVER_FN(cuStreamWaitValue32);
  if (fn == nullptr) return -1;
  return static_cast<int>(fn(reinterpret_cast<CUstream>(stream), addr, value, CU_STREAM_WAIT_VALUE_GEQ));
}
int stream_wait_value32_eq(uint64_t addr, uint32_t value, cudaStream_t stream) {
  auto fn = TDB_DRIVER_FN(cuStreamWaitValue32);
  if (fn == nullptr) return -1;
  return static_cast<int>(fn(reinterpret_cast<CUstream>(stream), addr, value, CU_STREAM_WAIT_VALUE_EQ));
}

}  // namespace tdb
