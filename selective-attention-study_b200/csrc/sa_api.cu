// extern "C" boundary of the Selective Attention library: argument checks, workspace carving and the
// launch sequences of the two engines.  Declarations and the reference code each entry point replaces
// are in include/selective_attention_b200.h.
#include <math.h>

#include <atomic>
#include <mutex>

#include "sa_common.cuh"
#include "sa_tc_host.cuh"

namespace sa {

static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(int code) { g_last_cuda_error = code; }

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// Event pairs recorded around the enabled kernel; created on demand, reused after sa_profile_collect.
namespace {
constexpr int kMaxProfile = 512;
int g_profile_kernel = 0;
int g_profile_count = 0;
int g_profile_created = 0;
cudaEvent_t g_profile_start[kMaxProfile], g_profile_stop[kMaxProfile];
}  // namespace

ProfileScope::ProfileScope(int kernel_id, cudaStream_t s) : slot(-1), stream(s) {
  if (kernel_id != g_profile_kernel || g_profile_count >= kMaxProfile) return;
  if (g_profile_count >= g_profile_created) {
    if (cudaEventCreate(&g_profile_start[g_profile_created]) != cudaSuccess) return;
    if (cudaEventCreate(&g_profile_stop[g_profile_created]) != cudaSuccess) return;
    ++g_profile_created;
  }
  slot = g_profile_count++;
  cudaEventRecord(g_profile_start[slot], stream);
}
ProfileScope::~ProfileScope() {
  if (slot >= 0) cudaEventRecord(g_profile_stop[slot], stream);
}

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

bool dim_ok(int d) { return d == 16 || d == 32 || d == 64 || d == 128; }
bool dtype_ok(int t) { return t == SA_F32 || t == SA_BF16 || t == SA_F16; }
size_t dtype_bytes(int t) { return t == SA_F32 ? 4 : 2; }

int to_problem(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel, Problem* p) {
  if (in == nullptr || in->struct_bytes != (int32_t)sizeof(sa_problem)) return SA_ERR_BAD_ARGUMENT;
  if (!dtype_ok(in->dtype)) return SA_ERR_BAD_ARGUMENT;
  if (in->engine != SA_ENGINE_SIMT && in->engine != SA_ENGINE_TCGEN05) return SA_ERR_BAD_ARGUMENT;
  if (in->batch < 1 || in->heads < 1 || in->seq < 1 || in->exempt < 1) return SA_ERR_BAD_ARGUMENT;
  if (!dim_ok(in->head_dim)) return SA_ERR_UNSUPPORTED;
  if (in->damp < SA_DAMP_NONE || in->damp > SA_DAMP_SQRT) return SA_ERR_BAD_ARGUMENT;
  if (in->damp != SA_DAMP_NONE && in->train_len < 1) return SA_ERR_BAD_ARGUMENT;
  // the CUDA-core kernels put (batch, head) rows on grid.y; the tensor-core kernels use 1-D grids
  if (in->engine == SA_ENGINE_SIMT && (int64_t)in->batch * in->heads > 65535) return SA_ERR_UNSUPPORTED;
  if ((int64_t)in->batch * in->heads * ((in->seq + 127) / 128) > 0x7fffffffLL) return SA_ERR_UNSUPPORTED;
  if (sel != nullptr && (sel->struct_bytes != (int32_t)sizeof(sa_selector) || !sel->q0 || !sel->k0))
    return SA_ERR_BAD_ARGUMENT;
  p->batch = in->batch;
  p->heads = in->heads;
  p->seq = in->seq;
  p->head_dim = in->head_dim;
  p->exempt = in->exempt;
  p->damp = in->damp;
  p->train_len = in->train_len;
  p->dtype = in->dtype;
  p->scale = (float)(1.0 / sqrt((double)in->head_dim));
  p->q = Strided{q, in->q_stride[0], in->q_stride[1], in->q_stride[2]};
  p->k = Strided{k, in->k_stride[0], in->k_stride[1], in->k_stride[2]};
  p->v = Strided{v, in->v_stride[0], in->v_stride[1], in->v_stride[2]};
  p->q_offset = 0;
  p->carry_init = nullptr;
  p->carry_init_stride = 0;
  p->tile_table = nullptr;
  p->out_lowp = nullptr;
  p->out_lowp_rows = contiguous_rows(in->heads, in->seq, in->head_dim);
  p->dv_rows = contiguous_rows(in->heads, in->seq, in->head_dim);
  p->external_selector = (sel != nullptr);
  if (sel != nullptr) {
    p->q0 = Strided{sel->q0, sel->q0_stride[0], 0, sel->q0_stride[1]};
    p->k0 = Strided{sel->k0, sel->k0_stride[0], 0, sel->k0_stride[1]};
  } else {
    p->q0 = Strided{q, in->q_stride[0], 0, in->q_stride[2]};          // head 0 of q / k
    p->k0 = Strided{k, in->k_stride[0], 0, in->k_stride[2]};
  }
  return SA_OK;
}

struct BackwardWorkspace {
  size_t dq_acc, dk_acc, dq0, dk0, dbar, d_out_lowp, total;
};

BackwardWorkspace carve(const sa_problem* in) {
  const size_t rows = (size_t)in->batch * in->heads * in->seq;
  const size_t elems = rows * in->head_dim;
  const size_t elems0 = (size_t)in->batch * in->seq * in->head_dim;
  BackwardWorkspace w{};
  size_t off = 0;
  w.dq_acc = off; off = align_up(off + elems * 4, 256);
  w.dk_acc = off; off = align_up(off + elems * 4, 256);
  w.dq0 = off; off = align_up(off + elems0 * 4, 256);
  w.dk0 = off; off = align_up(off + elems0 * 4, 256);
  w.dbar = off; off = align_up(off + rows * 4, 256);
  w.d_out_lowp = off;   // d_out converted for the engine: bf16/fp16 (tensor-core) or fp32 (CUDA-core)
  off = align_up(off + elems * (in->engine == SA_ENGINE_TCGEN05 ? 2 : 4), 256);
  w.total = off;
  return w;
}

}  // namespace
}  // namespace sa

using namespace sa;

extern "C" {

int sa_abi_version(void) { return 3; }

const char* sa_status_string(int status) {
  switch (status) {
    case SA_OK: return "ok";
    case SA_ERR_BAD_ARGUMENT: return "bad argument";
    case SA_ERR_UNSUPPORTED: return "unsupported shape, dtype or engine";
    case SA_ERR_ALIGNMENT: return "pointer or stride alignment";
    case SA_ERR_WORKSPACE: return "workspace too small";
    case SA_ERR_CUDA: return "CUDA call failed";
    case SA_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case SA_ERR_TOO_LARGE: return "problem exceeds the fixed capacity";
  }
  return "unknown status";
}

int sa_last_cuda_error(void) { return g_last_cuda_error; }

int sa_engine_available(int engine) {
  if (engine == SA_ENGINE_SIMT) return 1;
  if (engine == SA_ENGINE_TCGEN05) return tc_available();
  return 0;
}

int sa_engine_supports(int engine, int dtype, int head_dim, int with_backward) {
  if (!dtype_ok(dtype) || !dim_ok(head_dim)) return 0;
  if (engine == SA_ENGINE_SIMT) return 1;
  if (engine != SA_ENGINE_TCGEN05 || !tc_available()) return 0;
  Problem p{};
  p.dtype = dtype;
  p.head_dim = head_dim;
  p.damp = SA_DAMP_NONE;
  return (with_backward ? tc_backward_supported(p) : tc_supported(p)) == SA_OK;
}

int sa_carry_rows(int engine) {
  if (engine == SA_ENGINE_SIMT) return kSimtCarryRows;
  if (engine == SA_ENGINE_TCGEN05) return kTcCarryRows;
  return 0;
}

int sa_carry_checkpoints(int engine, int seq) {
  if (seq < 1) return 0;
  if (engine == SA_ENGINE_SIMT) return (seq + kSimtCarryRows - 1) / kSimtCarryRows;
  if (engine == SA_ENGINE_TCGEN05) return (seq + kTcCarryRows - 1) / kTcCarryRows + 1;   // + the grand total
  return 0;
}

namespace {
// A caller-layout tensor of the layout-fused entry points: element type of the problem, 16-byte aligned rows.
int rows_of(const sa_tensor* t, int dtype, RowLayout* rows) {
  if (t == nullptr || t->ptr == nullptr || t->dtype != dtype) return SA_ERR_BAD_ARGUMENT;
  const int64_t es = (dtype == SA_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(t->ptr) & 15) != 0) return SA_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if ((t->stride[i] * es) & 15) return SA_ERR_ALIGNMENT;
  *rows = RowLayout{t->stride[0], t->stride[1], t->stride[2]};
  return SA_OK;
}
}  // namespace

int sa_forward_fused(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                     float* out, const sa_tensor* out_lowp, float* lse2, float* carry, float* total, void* stream);

int sa_forward_selector(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                        float* out, float* lse2, float* carry, float* total, void* stream) {
  return sa_forward_fused(in, q, k, v, sel, out, nullptr, lse2, carry, total, stream);
}

int sa_forward_fused(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                     float* out, const sa_tensor* out_lowp, float* lse2, float* carry, float* total, void* stream) {
  return sa_forward_live_tiles(in, q, k, v, sel, out, out_lowp, lse2, carry, total, nullptr, 0, stream);
}

size_t sa_tile_table_bytes(const sa_problem* in) {
  Problem p;
  if (to_problem(in, nullptr, nullptr, nullptr, nullptr, &p) != SA_OK || in->engine != SA_ENGINE_TCGEN05) return 0;
  return tc::tile_table_bytes(p);
}

int sa_forward_live_tiles(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                          float* out, const sa_tensor* out_lowp, float* lse2, float* carry, float* total,
                          void* tile_table, size_t tile_table_bytes, void* stream) {
  Problem p;
  int st = to_problem(in, q, k, v, sel, &p);
  if (st != SA_OK) return st;
  if (!q || !k || !v || !out || !lse2 || !carry || !total) return SA_ERR_BAD_ARGUMENT;
  if (tile_table != nullptr) {
    const size_t need = (in->engine == SA_ENGINE_TCGEN05) ? tc::tile_table_bytes(p) : 0;
    if (need == 0) return SA_ERR_UNSUPPORTED;
    if (tile_table_bytes < need) return SA_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(tile_table) & 255) != 0) return SA_ERR_ALIGNMENT;
    p.tile_table = tile_table;
  }
  if (out_lowp != nullptr) {
    if (in->engine != SA_ENGINE_TCGEN05) return SA_ERR_UNSUPPORTED;
    st = rows_of(out_lowp, in->dtype, &p.out_lowp_rows);
    if (st != SA_OK) return st;
    p.out_lowp = out_lowp->ptr;
  }
  if (tc::timeout_pending()) return SA_ERR_DEVICE_TIMEOUT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in->engine == SA_ENGINE_SIMT) return simt_forward(p, out, lse2, carry, total, s);
  st = tc_supported(p);
  if (st != SA_OK) return st;
  return tc_forward(p, out, lse2, carry, total, s);
}

int sa_selection_carry(const sa_problem* in, const void* q, const void* k, const sa_selector* sel, float* carry,
                       float* total, void* stream) {
  Problem p;
  int st = to_problem(in, q, k, q, sel, &p);
  if (st != SA_OK) return st;
  if (!q || !k || !carry || !total) return SA_ERR_BAD_ARGUMENT;
  if (in->engine != SA_ENGINE_SIMT) return SA_ERR_UNSUPPORTED;
  return simt_carry(p, carry, total, static_cast<cudaStream_t>(stream));
}

int sa_forward(const sa_problem* in, const void* q, const void* k, const void* v, float* out, float* lse2,
               float* carry, float* total, void* stream) {
  return sa_forward_selector(in, q, k, v, nullptr, out, lse2, carry, total, stream);
}

int sa_prefill_extend(const sa_problem* in, int cached, const void* q_new, const void* k_cache, const void* v_cache,
                      const float* selected, int64_t selected_stride, float* out, float* lse2, float* carry, float* total,
                      void* stream) {
  return sa_prefill_extend_live_tiles(in, cached, q_new, k_cache, v_cache, selected, selected_stride, out, lse2, carry, total,
                                      nullptr, 0, stream);
}

int sa_prefill_extend_live_tiles(const sa_problem* in, int cached, const void* q_new, const void* k_cache,
                                 const void* v_cache, const float* selected, int64_t selected_stride, float* out,
                                 float* lse2, float* carry, float* total, void* tile_table, size_t tile_table_bytes,
                                 void* stream) {
  Problem p;
  int st = to_problem(in, q_new, k_cache, v_cache, nullptr, &p);
  if (st != SA_OK) return st;
  if (!q_new || !k_cache || !v_cache || !selected || !out || !lse2 || !carry || !total) return SA_ERR_BAD_ARGUMENT;
  if (cached < 0 || cached >= in->seq || selected_stride < in->seq) return SA_ERR_BAD_ARGUMENT;
  if (in->engine != SA_ENGINE_TCGEN05) return SA_ERR_UNSUPPORTED;
  st = tc_supported(p);
  if (st != SA_OK) return st;
  if (tc::timeout_pending()) return SA_ERR_DEVICE_TIMEOUT;
  if (tile_table != nullptr) {
    const size_t need = tc::tile_table_bytes(p);
    if (need == 0) return SA_ERR_UNSUPPORTED;
    if (tile_table_bytes < need) return SA_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(tile_table) & 255) != 0) return SA_ERR_ALIGNMENT;
    p.tile_table = tile_table;
  }
  p.q_offset = cached;
  p.carry_init = selected;
  p.carry_init_stride = selected_stride;
  return tc_forward(p, out, lse2, carry, total, static_cast<cudaStream_t>(stream));
}

// ---- forward with library-owned scratch (no allocation anywhere on the call path) ----------------------
// The running-selection checkpoints (`carry`) are the forward's only scratch.  Here they live in a
// file-scope device array.  Its name is only a host-side handle; the device address is looked up once
// per device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) float g_static_carry[SA_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_carry_ptr[kMaxDevices] = {};
std::mutex g_static_carry_mutex;

int static_carry_for_current_device(float** out) {
  int dev = -1;
  SA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_carry_mutex);
  if (g_static_carry_ptr[dev] == nullptr) {
    void* p = nullptr;
    SA_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_carry));
    g_static_carry_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_carry_ptr[dev];
  return SA_OK;
}
}  // namespace

size_t sa_static_scratch_floats(void) { return (size_t)SA_STATIC_SCRATCH_FLOATS; }

int sa_forward_static_scratch(const sa_problem* in, const void* q, const void* k, const void* v, float* out,
                              float* lse2, float* total, void* stream) {
  Problem p;
  int st = to_problem(in, q, k, v, nullptr, &p);
  if (st != SA_OK) return st;
  if (!q || !k || !v || !out || !lse2 || !total) return SA_ERR_BAD_ARGUMENT;
  if (tc::timeout_pending()) return SA_ERR_DEVICE_TIMEOUT;
  tc::NoHostAllocScope no_alloc;   // the bounded waits then use the timeout flag only if an earlier call made it
  const size_t need = (size_t)p.batch * (size_t)sa_carry_checkpoints(in->engine, p.seq) * (size_t)p.seq;
  if (need > (size_t)SA_STATIC_SCRATCH_FLOATS) return SA_ERR_TOO_LARGE;
  if (in->engine == SA_ENGINE_TCGEN05) {
    st = tc_supported(p);
    if (st != SA_OK) return st;
  }
  float* carry = nullptr;
  st = static_carry_for_current_device(&carry);
  if (st != SA_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Nothing in the array has to start at zero: both engines write every checkpoint they later read.
  if (in->engine == SA_ENGINE_SIMT) return simt_forward(p, out, lse2, carry, total, s);
  return tc_forward(p, out, lse2, carry, total, s);
}

size_t sa_backward_workspace_bytes(const sa_problem* in) {
  Problem p;
  if (to_problem(in, nullptr, nullptr, nullptr, nullptr, &p) != SA_OK) return 0;
  return carve(in).total;
}

namespace {
int backward_common(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                    const float* out, const float* lse2, const float* carry, const void* d_out, int d_out_dtype,
                    const RowLayout* d_out_rows, void* dq, void* dk, void* dv, const RowLayout* dq_rows,
                    const RowLayout* dk_rows, const RowLayout* dv_rows, float* dq0_out, float* dk0_out, void* workspace,
                    size_t workspace_bytes, const void* tile_table, void* stream);
}  // namespace

int sa_backward_selector(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                         const float* out, const float* lse2, const float* carry, const void* d_out, int d_out_dtype,
                         void* dq, void* dk, void* dv, float* dq0_out, float* dk0_out, void* workspace,
                         size_t workspace_bytes, void* stream) {
  return backward_common(in, q, k, v, sel, out, lse2, carry, d_out, d_out_dtype, nullptr, dq, dk, dv, nullptr, nullptr,
                         nullptr, dq0_out, dk0_out, workspace, workspace_bytes, nullptr, stream);
}

int sa_backward_fused(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                      const float* out, const float* lse2, const float* carry, const sa_tensor* d_out,
                      const sa_tensor* dq, const sa_tensor* dk, const sa_tensor* dv, float* dq0_out, float* dk0_out,
                      void* workspace, size_t workspace_bytes, void* stream) {
  return sa_backward_live_tiles(in, q, k, v, sel, out, lse2, carry, d_out, dq, dk, dv, dq0_out, dk0_out, workspace,
                                workspace_bytes, nullptr, stream);
}

int sa_backward_live_tiles(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                           const float* out, const float* lse2, const float* carry, const sa_tensor* d_out,
                           const sa_tensor* dq, const sa_tensor* dk, const sa_tensor* dv, float* dq0_out, float* dk0_out,
                           void* workspace, size_t workspace_bytes, const void* tile_table, void* stream) {
  if (in == nullptr || in->engine != SA_ENGINE_TCGEN05) return in ? SA_ERR_UNSUPPORTED : SA_ERR_BAD_ARGUMENT;
  RowLayout r_do, r_dq, r_dk, r_dv;
  if (d_out == nullptr || !dtype_ok(d_out->dtype)) return SA_ERR_BAD_ARGUMENT;
  int st = rows_of(d_out, d_out->dtype, &r_do);        // the cotangent may be of any supported element type
  if (st == SA_OK) st = rows_of(dq, in->dtype, &r_dq);
  if (st == SA_OK) st = rows_of(dk, in->dtype, &r_dk);
  if (st == SA_OK) st = rows_of(dv, in->dtype, &r_dv);
  if (st != SA_OK) return st;
  return backward_common(in, q, k, v, sel, out, lse2, carry, d_out->ptr, d_out->dtype, &r_do, dq->ptr, dk->ptr, dv->ptr,
                         &r_dq, &r_dk, &r_dv, dq0_out, dk0_out, workspace, workspace_bytes, tile_table, stream);
}

namespace {
int backward_common(const sa_problem* in, const void* q, const void* k, const void* v, const sa_selector* sel,
                    const float* out, const float* lse2, const float* carry, const void* d_out, int d_out_dtype,
                    const RowLayout* d_out_rows, void* dq, void* dk, void* dv, const RowLayout* dq_rows,
                    const RowLayout* dk_rows, const RowLayout* dv_rows, float* dq0_out, float* dk0_out, void* workspace,
                    size_t workspace_bytes, const void* tile_table, void* stream) {
  Problem p;
  int st = to_problem(in, q, k, v, sel, &p);
  if (st != SA_OK) return st;
  if (dv_rows != nullptr) p.dv_rows = *dv_rows;
  if (tile_table != nullptr) {                         // the table the forward of this call filled
    if (in->engine != SA_ENGINE_TCGEN05 || tc::tile_table_bytes(p) == 0) return SA_ERR_UNSUPPORTED;
    p.tile_table = const_cast<void*>(tile_table);
  }
  if (!q || !k || !v || !out || !lse2 || !carry || !d_out || !dq || !dk || !dv || !workspace) return SA_ERR_BAD_ARGUMENT;
  if (sel != nullptr && (!dq0_out || !dk0_out)) return SA_ERR_BAD_ARGUMENT;
  if (!dtype_ok(d_out_dtype) || in->damp != SA_DAMP_NONE) return SA_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return SA_ERR_ALIGNMENT;
  if (sel != nullptr && ((reinterpret_cast<uintptr_t>(dq0_out) | reinterpret_cast<uintptr_t>(dk0_out)) & 15) != 0)
    return SA_ERR_ALIGNMENT;
  const BackwardWorkspace w = carve(in);
  if (workspace_bytes < w.total) return SA_ERR_WORKSPACE;
  if (tc::timeout_pending()) return SA_ERR_DEVICE_TIMEOUT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(workspace);
  float* dq_acc = reinterpret_cast<float*>(base + w.dq_acc);
  float* dk_acc = reinterpret_cast<float*>(base + w.dk_acc);
  float* dq0 = reinterpret_cast<float*>(base + w.dq0);
  float* dk0 = reinterpret_cast<float*>(base + w.dk0);
  float* dbar = reinterpret_cast<float*>(base + w.dbar);
  const int64_t rows = (int64_t)p.batch * p.heads * p.seq;
  const int64_t per_head = (int64_t)p.seq * p.head_dim;
  const size_t elems = (size_t)rows * p.head_dim;
  const size_t elems0 = (size_t)p.batch * per_head;

  // dq_acc, dq0 and dk0 are accumulated with atomics and start at zero (the workspace's dq0/dk0 pair is contiguous).
  SA_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, elems * 4, s));
  if (sel != nullptr) {            // the selector's gradients go to the caller, unfolded
    dq0 = dq0_out;
    dk0 = dk0_out;
    SA_CUDA_CHECK(cudaMemsetAsync(dq0, 0, elems0 * 4, s));
    SA_CUDA_CHECK(cudaMemsetAsync(dk0, 0, elems0 * 4, s));
  } else {
    SA_CUDA_CHECK(cudaMemsetAsync(dq0, 0, (w.dk0 - w.dq0) + elems0 * 4, s));
  }
  const float* fold_q = sel ? nullptr : dq0;
  const float* fold_k = sel ? nullptr : dk0;

  if (in->engine == SA_ENGINE_SIMT) {
    const float* d_out_f32 = static_cast<const float*>(d_out);
    void* copy = nullptr;
    if (d_out_dtype != SA_F32) {
      copy = base + w.d_out_lowp;
      d_out_f32 = static_cast<const float*>(copy);
    }
    st = launch_dbar(out, d_out, d_out_dtype, rows, p.head_dim, dbar, copy, SA_F32, nullptr, p.heads, p.seq, s);
    if (st != SA_OK) return st;
    st = simt_backward(p, lse2, carry, dbar, d_out_f32, dq_acc, dk_acc, dq0, dk0, dv, s);
    if (st != SA_OK) return st;
    st = launch_fold_cast(dk_acc, fold_k, dk, p.dtype, p.batch, p.heads, per_head, nullptr, p.head_dim, s);
    if (st != SA_OK) return st;
    return launch_fold_cast(dq_acc, fold_q, dq, p.dtype, p.batch, p.heads, per_head, nullptr, p.head_dim, s);
  }
  st = tc_backward_supported(p);
  if (st != SA_OK) return st;
  void* d_out_lowp = base + w.d_out_lowp;
  st = launch_dbar(out, d_out, d_out_dtype, rows, p.head_dim, dbar, d_out_lowp, p.dtype, d_out_rows, p.heads, p.seq, s);
  if (st != SA_OK) return st;
  st = tc_backward(p, lse2, carry, dbar, d_out_lowp, dq_acc, dk_acc, dq0, dk0, dv, s);
  if (st != SA_OK) return st;
  st = launch_fold_cast(dk_acc, fold_k, dk, p.dtype, p.batch, p.heads, per_head, dk_rows, p.head_dim, s);
  if (st != SA_OK) return st;
  return launch_fold_cast(dq_acc, fold_q, dq, p.dtype, p.batch, p.heads, per_head, dq_rows, p.head_dim, s);
}
}  // namespace

int sa_backward(const sa_problem* in, const void* q, const void* k, const void* v, const float* out,
                const float* lse2, const float* carry, const void* d_out, int d_out_dtype, void* dq, void* dk,
                void* dv, void* workspace, size_t workspace_bytes, void* stream) {
  return sa_backward_selector(in, q, k, v, nullptr, out, lse2, carry, d_out, d_out_dtype, dq, dk, dv, nullptr, nullptr,
                              workspace, workspace_bytes, stream);
}

unsigned long long sa_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int sa_profile_enable(int kernel_id) {
  if (kernel_id < 0 || kernel_id > SA_KERNEL_DECODE) return SA_ERR_BAD_ARGUMENT;
  g_profile_kernel = kernel_id;
  g_profile_count = 0;
  return SA_OK;
}

int sa_profile_collect(float* ms_host, int capacity) {
  if (!ms_host || capacity < 0) return -1;
  int n = g_profile_count < capacity ? g_profile_count : capacity;
  for (int i = 0; i < n; ++i) {
    if (cudaEventSynchronize(g_profile_stop[i]) != cudaSuccess) return -1;
    if (cudaEventElapsedTime(&ms_host[i], g_profile_start[i], g_profile_stop[i]) != cudaSuccess) return -1;
  }
  g_profile_count = 0;
  return n;
}

int sa_device_status(unsigned int* value_host, int clear) {
  if (!value_host) return SA_ERR_BAD_ARGUMENT;
  return tc::read_status(value_host, clear != 0);
}

int sa_selftest_wait_timeout(unsigned int limit_kcycles, void* stream) {
  if (limit_kcycles < 1u || limit_kcycles > 100000u) return SA_ERR_BAD_ARGUMENT;   // at most ~0.05 s
  return tc::selftest_wait_timeout(limit_kcycles, static_cast<cudaStream_t>(stream));
}

int sa_selftest_tcgen05(void* scratch, float* result, void* stream) {
  if (!scratch || !result) return SA_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(scratch) & 1023) != 0) return SA_ERR_ALIGNMENT;
  return tc::selftest(scratch, result, static_cast<cudaStream_t>(stream));
}

size_t sa_decode_workspace_bytes(int batch, int heads, int groups, int length, int head_dim) {
  if (batch < 1 || heads < 1 || groups < 1 || length < 0 || !dim_ok(head_dim)) return 0;
  return decode_workspace_floats(batch, heads, groups, length, head_dim) * sizeof(float);
}

int sa_decode_step(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim, int exempt,
                   const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache, float* selected,
                   float* y, void* workspace, size_t workspace_bytes, void* stream) {
  return sa_decode_step_live_keys(dtype, batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, k_cache,
                                  v_cache, selected, nullptr, y, workspace, workspace_bytes, stream);
}

int sa_decode_step_live_keys(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim,
                             int exempt, const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                             float* selected, float* key_norms, float* y, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (!dtype_ok(dtype) || batch < 1 || heads < 1 || groups < 1 || heads % groups != 0 || length < 0 || exempt < 1)
    return SA_ERR_BAD_ARGUMENT;
  if (!dim_ok(head_dim)) return SA_ERR_UNSUPPORTED;
  if (length >= capacity) return SA_ERR_BAD_ARGUMENT;
  if (!q1 || !k1 || !v1 || !k_cache || !v_cache || !selected || !y || !workspace) return SA_ERR_BAD_ARGUMENT;
  if ((int64_t)batch * heads * ((length + 512) / 512) > 0x7fffffffLL) return SA_ERR_TOO_LARGE;   // 1-D grid
  for (const void* ptr : {q1, k1, v1, (const void*)k_cache, (const void*)v_cache})            // 16-byte loads, bulk copies
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return SA_ERR_ALIGNMENT;
  if (workspace_bytes < sa_decode_workspace_bytes(batch, heads, groups, length, head_dim)) return SA_ERR_WORKSPACE;
  if (tc::timeout_pending()) return SA_ERR_DEVICE_TIMEOUT;
  return decode_step(dtype, batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, k_cache, v_cache,
                     selected, y, static_cast<float*>(workspace), key_norms, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
