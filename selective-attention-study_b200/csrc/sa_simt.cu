// CUDA-core engine: dispatch on the input dtype (kernels in sa_simt_impl.cuh).
#include "sa_common.cuh"

namespace sa {
#define SA_SIMT_DECL(name)                                                                                       \
  int simt_forward_##name(const Problem&, float*, float*, float*, float*, cudaStream_t);                         \
  int simt_carry_##name(const Problem&, float*, float*, cudaStream_t);                                           \
  int simt_backward_##name(const Problem&, const float*, const float*, const float*, const float*, float*, float*, \
                           float*, float*, void*, cudaStream_t);
SA_SIMT_DECL(f32)
SA_SIMT_DECL(bf16)
SA_SIMT_DECL(f16)
#undef SA_SIMT_DECL

int simt_forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  switch (p.dtype) {
    case SA_F32: return simt_forward_f32(p, out, lse2, carry, total, s);
    case SA_BF16: return simt_forward_bf16(p, out, lse2, carry, total, s);
    case SA_F16: return simt_forward_f16(p, out, lse2, carry, total, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}

int simt_carry(const Problem& p, float* carry, float* total, cudaStream_t s) {
  switch (p.dtype) {
    case SA_F32: return simt_carry_f32(p, carry, total, s);
    case SA_BF16: return simt_carry_bf16(p, carry, total, s);
    case SA_F16: return simt_carry_f16(p, carry, total, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}

int simt_backward(const Problem& p, const float* lse2, const float* carry, const float* dbar, const float* d_out,
                  float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  switch (p.dtype) {
    case SA_F32: return simt_backward_f32(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
    case SA_BF16: return simt_backward_bf16(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
    case SA_F16: return simt_backward_f16(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}
}  // namespace sa
