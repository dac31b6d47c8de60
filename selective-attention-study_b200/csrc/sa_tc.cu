// Tensor-core (tcgen05) engine — placeholder until the kernels land.
#include "sa_common.cuh"
namespace sa {
int tc_available() { return 0; }
int tc_supported(const Problem&) { return SA_ERR_UNSUPPORTED; }
int tc_forward(const Problem&, float*, float*, float*, float*, cudaStream_t) { return SA_ERR_UNSUPPORTED; }
int tc_backward(const Problem&, const float*, const float*, const float*, const void*, float*, float*, float*, void*,
                void*, cudaStream_t) { return SA_ERR_UNSUPPORTED; }
}  // namespace sa
