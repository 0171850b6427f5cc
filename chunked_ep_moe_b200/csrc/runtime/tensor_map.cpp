#include "tensor_map.h"

#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

namespace cem {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || sym == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeFn>(sym);
  });
  return fn;
}

}  // namespace

CUtensorMap make_bf16_map_2d(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("tensor map base must be 16-byte aligned");
  if ((cols * 2) % 16 != 0) throw std::runtime_error("tensor map row pitch must be a multiple of 16 bytes");
  if (box_rows == 0 || box_rows > 256) throw std::runtime_error("tensor map box rows must be in [1, 256]");
  CUtensorMap map;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult res = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    throw std::runtime_error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(res)));
  return map;
}

CUtensorMap make_bf16_map_chunked(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t chunks) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("tensor map base must be 16-byte aligned");
  if (cols % 64 != 0) throw std::runtime_error("chunked tensor map needs a multiple of 64 columns");
  if (box_rows == 0 || box_rows > 256 || chunks == 0 || chunks > 256)
    throw std::runtime_error("tensor map box rows and chunks must be in [1, 256]");
  CUtensorMap map;
  const cuuint64_t dims[3] = {64, rows, cols / 64};
  const cuuint64_t strides[2] = {cols * 2, 128};
  const cuuint32_t box[3] = {64, box_rows, chunks};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult res = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    throw std::runtime_error("cuTensorMapEncodeTiled (chunked) failed with CUresult " +
                             std::to_string(static_cast<int>(res)));
  return map;
}

}  // namespace cem
