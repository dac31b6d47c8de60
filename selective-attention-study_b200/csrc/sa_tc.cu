// Tensor-core (tcgen05) engine: what it accepts, and dispatch to the forward / backward kernels.
#include "sa_common.cuh"
#include "sa_tc_host.cuh"

namespace sa {
namespace tc {
int forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s);
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

int tc_backward(const Problem&, const float*, const float*, const float*, const void*, float*, float*, float*, void*,
                void*, cudaStream_t) {
  return SA_ERR_UNSUPPORTED;
}
}  // namespace sa
