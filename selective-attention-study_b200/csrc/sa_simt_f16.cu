// CUDA-core engine, instantiation for __half inputs (one translation unit per dtype keeps builds parallel).
#include "sa_simt_impl.cuh"

namespace sa {
int simt_forward_f16(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  return simt::forward_by_dim<__half>(p, out, lse2, carry, total, s);
}
int simt_carry_f16(const Problem& p, float* carry, float* total, cudaStream_t s) {
  return simt::carry_by_dim<__half>(p, carry, total, s);
}
int simt_backward_f16(const Problem& p, const float* lse2, const float* carry, const float* dbar,
                         const float* d_out, float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv,
                         cudaStream_t s) {
  return simt::backward_by_dim<__half, float>(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
}
}  // namespace sa
