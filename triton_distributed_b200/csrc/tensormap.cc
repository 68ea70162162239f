// Host-side encoding of TMA tensor maps.  The driver entry point is looked up at
// run time through the CUDA runtime so the library does not link libcuda (and
// loads on machines without a driver, where only the non-GPU code is used).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "tdb/api.h"
#include "tdb/driver.h"

namespace tdb {

void* driver_entry(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return fn;
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
  return fn;
}

CUtensorMapDataType to_cu(DType t, int* elem) {
  switch (t) {
    case kBF16: *elem = 2; return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case kF16: *elem = 2; return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case kF32: *elem = 4; return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case kI32: *elem = 4; return CU_TENSOR_MAP_DATA_TYPE_INT32;
    case kE4M3:
    case kU8:
    default: *elem = 1; return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

CUtensorMapSwizzle to_swizzle(int bytes) {
  switch (bytes) {
    case 32: return CU_TENSOR_MAP_SWIZZLE_32B;
    case 64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case 128: return CU_TENSOR_MAP_SWIZZLE_128B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}

}  // namespace

int encode_tensor_map_3d(TensorMap* out, const void* base, DType dtype, uint64_t d2, uint64_t rows, uint64_t cols,
                         uint64_t row_stride_bytes, uint64_t d2_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                         int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  int elem = 0;
  const CUtensorMapDataType dt = to_cu(dtype, &elem);
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_bytes & 15u) != 0 || (d2_stride_bytes & 15u) != 0)
    return -2;
  if (swizzle_bytes != 0 && static_cast<uint64_t>(box_cols) * elem > static_cast<uint64_t>(swizzle_bytes)) return -3;
  if (box_rows > 256 || box_cols > 256) return -4;
  cuuint64_t dims[3] = {cols, rows, d2};
  cuuint64_t strides[2] = {row_stride_bytes, d2_stride_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  const CUresult r = fn(&m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        to_swizzle(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  static_assert(sizeof(CUtensorMap) == sizeof(TensorMap), "tensor map image size");
  std::memcpy(out->bytes, &m, sizeof(m));
  return 0;
}

int encode_tensor_map_2d(TensorMap* out, const void* base, DType dtype, uint64_t rows, uint64_t cols,
                         uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  int elem = 0;
  const CUtensorMapDataType dt = to_cu(dtype, &elem);
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_bytes & 15u) != 0) return -2;
  if (swizzle_bytes != 0 && static_cast<uint64_t>(box_cols) * elem > static_cast<uint64_t>(swizzle_bytes)) return -3;
  if (box_rows > 256 || box_cols > 256) return -4;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = fn(&m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        to_swizzle(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  std::memcpy(out->bytes, &m, sizeof(m));
  return 0;
}

}  // namespace tdb
