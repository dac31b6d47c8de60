// Tensor-core (tcgen05) engine: what it accepts, and dispatch to the forward / backward kernels.
#include "sa_common.cuh"
#include "sa_tc_host.cuh"

namespace sa {
namespace tc {
int forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s);
int backward(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_bf16,
             float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s);
int backward_wide(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_bf16,
                  float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s);
}  // namespace tc

int tc_available() { return 1; }

int tc_supported(const Problem& p) {
  if (p.dtype != SA_BF16) return SA_ERR_UNSUPPORTED;
  if (p.head_dim != 64 && p.head_dim != 128) return SA_ERR_UNSUPPORTED;
  if (p.damp != SA_DAMP_NONE) return SA_ERR_UNSUPPORTED;
  return SA_OK;
}

int tc_forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  return tc::forward(p, out, lse2, carry, total, s);
}

int tc_backward_supported(const Problem& p) {
  return tc_supported(p);
}

int tc_backward(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_lowp,
                float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  if (p.head_dim == 128) return tc::backward_wide(p, lse2, carry, dbar, d_out_lowp, dq_acc, dk_acc, dq0, dk0, dv, s);
  return tc::backward(p, lse2, carry, dbar, d_out_lowp, dq_acc, dk_acc, dq0, dk0, dv, s);
}
}  // namespace sa
