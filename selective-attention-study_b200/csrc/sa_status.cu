// Host side of the bounded waits: the per-device status words, the mapped host flag through which a timeout
// is seen without synchronising, the epoch handed to every launch sequence, and the probe that makes a wait
// run out on purpose (a wait on an mbarrier nobody arrives on, with a short limit: it returns, it does not hang).
#include <mutex>

#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {
namespace {

__device__ unsigned int g_status[2] = {0u, 0u};   // [0] sticky first error, [1] epoch that gave up

constexpr int kMaxDevices = 64;
struct DeviceState {
  unsigned int* word = nullptr;        // device address of g_status
  unsigned int* flag_host = nullptr;   // pinned, mapped
  unsigned int* flag_dev = nullptr;    // the same word as the device sees it
  unsigned int epoch = 0;
};
DeviceState g_state[kMaxDevices];
std::mutex g_mutex;
thread_local int g_no_host_alloc = 0;

int current_state(DeviceState** out) {
  int dev = -1;
  SA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SA_ERR_UNSUPPORTED;
  *out = &g_state[dev];
  return SA_OK;
}

__global__ void wait_probe_kernel(WaitCtx ctx) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
    mbar_wait(&bar, 0, ctx, 900);      // nobody arrives: runs out after ctx.limit_kcycles
  }
}

}  // namespace

NoHostAllocScope::NoHostAllocScope() { ++g_no_host_alloc; }
NoHostAllocScope::~NoHostAllocScope() { --g_no_host_alloc; }

int wait_ctx(WaitCtx* out, bool may_create_host_flag) {
  if (g_no_host_alloc > 0) may_create_host_flag = false;
  DeviceState* st = nullptr;
  int rc = current_state(&st);
  if (rc != SA_OK) return rc;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (st->word == nullptr) {
    void* p = nullptr;
    SA_CUDA_CHECK(cudaGetSymbolAddress(&p, g_status));
    st->word = static_cast<unsigned int*>(p);
  }
  if (st->flag_host == nullptr && may_create_host_flag) {
    void* h = nullptr;
    SA_CUDA_CHECK(cudaHostAlloc(&h, sizeof(unsigned int), cudaHostAllocMapped | cudaHostAllocPortable));
    *static_cast<volatile unsigned int*>(h) = 0u;
    void* d = nullptr;
    if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
      cudaFreeHost(h);
      return SA_ERR_CUDA;
    }
    st->flag_host = static_cast<unsigned int*>(h);
    st->flag_dev = static_cast<unsigned int*>(d);
  }
  if (++st->epoch == 0u) st->epoch = 1u;
  out->word = st->word;
  out->host_flag = st->flag_dev;
  out->epoch = st->epoch;
  out->limit_kcycles = kWaitLimitKCycles;
  return SA_OK;
}

unsigned int timeout_pending() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0u;
  const unsigned int* flag = g_state[dev].flag_host;
  return flag ? *reinterpret_cast<const volatile unsigned int*>(flag) : 0u;
}

int read_status(unsigned int* host_value, bool clear) {
  WaitCtx ctx;
  int rc = wait_ctx(&ctx, false);
  if (rc != SA_OK) return rc;
  unsigned int words[2] = {0u, 0u};
  SA_CUDA_CHECK(cudaMemcpy(words, ctx.word, sizeof(words), cudaMemcpyDeviceToHost));
  DeviceState* st = nullptr;
  rc = current_state(&st);
  if (rc != SA_OK) return rc;
  unsigned int flag = st->flag_host ? *reinterpret_cast<volatile unsigned int*>(st->flag_host) : 0u;
  *host_value = words[0] ? words[0] : flag;
  if (clear && (words[0] != 0u || words[1] != 0u || flag != 0u)) {
    SA_CUDA_CHECK(cudaMemset(ctx.word, 0, sizeof(words)));
    if (st->flag_host) *reinterpret_cast<volatile unsigned int*>(st->flag_host) = 0u;
  }
  return SA_OK;
}

int selftest_wait_timeout(unsigned int limit_kcycles, cudaStream_t s) {
  WaitCtx ctx;
  int rc = wait_ctx(&ctx);
  if (rc != SA_OK) return rc;
  ctx.limit_kcycles = limit_kcycles;
  wait_probe_kernel<<<1, 32, 0, s>>>(ctx);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
