// Host helpers of the tensor-core engine: TMA tensor-map construction through the driver entry point
// (fetched at run time, so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include "sa_common.cuh"

namespace sa {
namespace tc {

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// 4-D map over (d, token, head, batch) of a 16-bit tensor; box = (64 elements, box_rows tokens, 1, 1),
// 128-byte swizzle, zero fill outside the tensor.  Strides are in elements.
inline int make_map_16bit(CUtensorMap* map, const void* base, int head_dim, int seq, int heads, int batch,
                          int64_t st, int64_t sh, int64_t sb, int box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return SA_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return SA_ERR_ALIGNMENT;
  if (((st * 2) & 15) || ((sh * 2) & 15) || ((sb * 2) & 15)) return SA_ERR_ALIGNMENT;
  // A dimension of extent 1 may carry any stride; give it a valid one.
  if (heads == 1) sh = st * seq;
  if (batch == 1) sb = sh * heads;
  cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(10000 + (int)r);
    return SA_ERR_CUDA;
  }
  return SA_OK;
}

// 4-D map over (d, token, row, 1) of a contiguous fp32 tensor (rows x seq x 64); box = (32 floats, 128
// tokens, 1, 1) with the 128-byte swizzle: the target of the TMA reduce-add of dQ tiles.
inline int make_map_f32_rows(CUtensorMap* map, const void* base, int seq, int rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return SA_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return SA_ERR_ALIGNMENT;
  cuuint64_t dims[4] = {64, (cuuint64_t)seq, (cuuint64_t)rows, 1};
  cuuint64_t strides[3] = {64 * 4, (cuuint64_t)seq * 64 * 4, (cuuint64_t)rows * seq * 64 * 4};
  cuuint32_t box[4] = {32, 128, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(10000 + (int)r);
    return SA_ERR_CUDA;
  }
  return SA_OK;
}

int status_word(unsigned int** device_ptr);            // per-device status word of the bounded waits
int read_status(unsigned int* host_value, bool clear); // synchronous read (and reset) of that word
int selftest(void* scratch, float* result, cudaStream_t s);

}  // namespace tc
}  // namespace sa
