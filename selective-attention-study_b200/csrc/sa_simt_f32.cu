// CUDA-core engine, instantiation for float inputs (one translation unit per dtype keeps builds parallel).
#include "sa_simt_impl.cuh"

namespace sa {
int simt_forward_f32(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  return simt::forward_by_dim<float>(p, out, lse2, carry, total, s);
}
int simt_carry_f32(const Problem& p, float* carry, float* total, cudaStream_t s) {
  return simt::carry_by_dim<float>(p, carry, total, s);
}
int simt_backward_f32(const Problem& p, const float* lse2, const float* carry, const float* dbar,
                         const float* d_out, float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv,
                         cudaStream_t s) {
  return simt::backward_by_dim<float, float>(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
}
}  // namespace sa
