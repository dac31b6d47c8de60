// Shared declarations of the Selective Attention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/selective_attention_b200.h"

namespace sa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kSimtCarryRows = 32;   // query rows per carry checkpoint, CUDA-core engine
constexpr int kTcCarryRows = 128;    // tensor-core engine: one checkpoint per 128-query tile

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

// Everything a kernel needs to find a (batch, head) row of q, k or v.
struct Strided {
  const void* ptr;
  int64_t sb, sh, st;   // batch, head, token strides in elements
};

// Element offset of row (b, h, t) of a (batch, heads, seq, head_dim) tensor with a contiguous innermost axis.
struct RowLayout {
  int64_t sb, sh, st;
  __host__ __device__ int64_t at(int b, int h, int64_t t) const { return b * sb + h * sh + t * st; }
};
inline RowLayout contiguous_rows(int heads, int seq, int dim) {
  return RowLayout{(int64_t)heads * seq * dim, (int64_t)seq * dim, (int64_t)dim};
}

struct Problem {
  int batch, heads, seq, head_dim;
  int exempt, damp, train_len;
  int dtype;
  float scale;          // 1 / sqrt(head_dim)
  Strided q, k, v;
  // The selector: the (batch, seq, head_dim) rows whose logits make the selection.  By default head 0 of q / k
  // (pointer and batch / token strides of q / k, head stride unused); with an external selector the caller's
  // own tensors, and then no head of q / k is the selector: nothing is folded into head 0 by the backward.
  Strided q0, k0;
  bool external_selector;
  // Layout-fused calls (tensor-core engine): an extra copy of the output in the operand dtype written straight into the
  // caller's (batch, seq, heads * head_dim) activation, and dv written straight into the caller's gradient buffer.
  // Prefill continuation (tensor-core engine): q holds only the queries from position q_offset on, k / v hold all `seq`
  // keys (the cache); carry_init[b * carry_init_stride + j] is the selection key j received from the queries before.
  int q_offset;
  const float* carry_init;
  int64_t carry_init_stride;
  void* out_lowp;        // null: not requested
  RowLayout out_lowp_rows;
  RowLayout dv_rows;     // where dv rows go (default: contiguous (batch, heads, seq, head_dim))
  // Tensor-core engine, optional: the table of live (query tile, key tile) pairs (sa_tc_skip.cu).  The forward
  // fills it after its selection pass and leaves out the dead tiles; the backward of the same call reads it.
  void* tile_table;      // null: every causal tile is computed
};

// ---- engine entry points (host) -------------------------------------------------------------------
int simt_forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s);
int simt_carry(const Problem& p, float* carry, float* total, cudaStream_t s);
int simt_backward(const Problem& p, const float* lse2, const float* carry, const float* dbar,
                  const float* d_out, float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv,
                  cudaStream_t s);

namespace tc {
size_t tile_table_bytes(const Problem& p);                                     // 0: not offered for this problem
int build_tile_table(const Problem& p, const float* carry, cudaStream_t s);
}  // namespace tc

int tc_available();
int tc_supported(const Problem& p);
int tc_forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s);
int tc_backward_supported(const Problem& p);
int tc_backward(const Problem& p, const float* lse2, const float* carry, const float* dbar,
                const void* d_out_lowp, float* dq_acc, float* dk_acc, float* dq0, float* dk0,
                void* dv, cudaStream_t s);

// ---- helper launches shared by both engines --------------------------------------------------------
// dbar[row] = sum_d d_out[row, d] * out[row, d]; optionally also writes d_out rounded to `lowp_dtype`.
// `d_out_rows` (may be null: contiguous) says where the rows of d_out start; `heads`, `seq` split a row index.
int launch_dbar(const float* out, const void* d_out, int d_out_dtype, int64_t rows, int head_dim,
                float* dbar, void* d_out_lowp, int lowp_dtype, const RowLayout* d_out_rows, int heads, int seq,
                cudaStream_t s);
// dst[b, h] = cast(acc[b, h] + (h == 0 ? acc0[b] : 0)), rows of head_dim elements; `dst_rows` (may be null:
// contiguous) says where the rows of dst start.
int launch_fold_cast(const float* acc, const float* acc0, void* dst, int dtype, int batch, int heads,
                     int64_t seq_times_dim, const RowLayout* dst_rows, int head_dim, cudaStream_t s);

size_t decode_workspace_floats(int batch, int heads, int groups, int length, int head_dim);
int decode_step(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim, int exempt,
                const void* q1, const void* k1, const void* v1, void* kc, void* vc, float* selected, float* y,
                float* ws, float* knorm, cudaStream_t s);   // knorm: per-key norms, or null (every key is read)

void set_last_cuda_error(int code);
void count_launch();   // every kernel launch of the library calls this once (sa_launch_count)

// ---- per-kernel timing hook (sa_profile_*) ------------------------------------------------------------
// Kernel ids of include/selective_attention_b200.h (SA_KERNEL_*).  When a kernel id is enabled, the
// launch site brackets that kernel with a CUDA event pair on the launching stream.
struct ProfileScope {
  ProfileScope(int kernel_id, cudaStream_t s);
  ~ProfileScope();
  int slot;
  cudaStream_t stream;
};

#define SA_CUDA_CHECK(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) {                                  \
      ::sa::set_last_cuda_error(static_cast<int>(_e));        \
      return SA_ERR_CUDA;                                     \
    }                                                         \
  } while (0)

}  // namespace sa
