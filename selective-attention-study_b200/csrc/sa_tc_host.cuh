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
  // A dimension of extent 1 may carry any stride; give it a valid one before the alignment rule is applied.
  if (heads == 1) sh = st * seq;
  if (batch == 1) sb = sh * heads;
  if (((st * 2) & 15) || ((sh * 2) & 15) || ((sb * 2) & 15)) return SA_ERR_ALIGNMENT;
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

// What a kernel with bounded waits is given (see sa_tc_ptx.cuh for how the device side uses it).
struct WaitCtx {
  unsigned int* word;
  unsigned int* host_flag;
  unsigned int epoch;          // never 0
  unsigned int limit_kcycles;  // a wait gives up after this many clock64 ticks / 1024
};

// Context for the next launch sequence on the current device: a fresh epoch and the default limit.  The
// mapped host flag (one page of pinned host memory per device) is created on first use unless
// `may_create_host_flag` is false (entry points that must not call an allocating routine), in which case the
// context carries whatever exists (possibly none).
int wait_ctx(WaitCtx* out, bool may_create_host_flag = true);
// While one of these is alive on a host thread, wait_ctx never creates the host flag on that thread.
struct NoHostAllocScope {
  NoHostAllocScope();
  ~NoHostAllocScope();
};
// Non-zero when a bounded wait has run out on the current device and the word has not been cleared; reads
// only host memory, so entry points call it first and refuse to launch (SA_ERR_DEVICE_TIMEOUT).
unsigned int timeout_pending();
// Synchronous read (and reset) of the sticky word.  Uses cudaMemcpy on the legacy default stream: it is ordered
// after work on blocking streams only; callers on non-blocking streams synchronise first.
int read_status(unsigned int* host_value, bool clear);
// Runs one CTA that waits, with the given limit, on an mbarrier nobody arrives on: the wait runs out, reports
// site 900 and the kernel returns.
int selftest_wait_timeout(unsigned int limit_kcycles, cudaStream_t s);
int selftest(void* scratch, float* result, cudaStream_t s);

}  // namespace tc
}  // namespace sa
