// Bandwidth-bound helpers of the Selective Attention operator (sm_100a):
//   dbar      dbar[row] = sum_d dO[row, d] * out[row, d], optionally also dO rounded to bf16 / fp16
//             (reference: src/selective_attention/kernels.py:635-636)
//   fold/cast dq = cast(dq_acc + [head 0] dq0)            (reference: kernels.py:662-666)
//   decode    one cached decode step                       (reference: src/selective_attention/mixers.py:115-130)
#include "sa_common.cuh"

namespace sa {
namespace {

// ---- dbar -----------------------------------------------------------------------------------------
// A group of D / 4 consecutive lanes owns one row; every lane handles 4 consecutive elements.
template <typename TDO, typename TLOW, int D, bool kWriteLow>
__global__ void __launch_bounds__(256) dbar_kernel(const float* __restrict__ out, const TDO* __restrict__ d_out,
                                                   int64_t rows, float* __restrict__ dbar,
                                                   TLOW* __restrict__ d_out_low) {
  constexpr int kLanes = D / 4;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / kLanes;
  const int lane = (int)(gid % kLanes);
  float sum = 0.f;
  if (row < rows) {
    const int64_t off = row * D + lane * 4;
    float4 o = *reinterpret_cast<const float4*>(out + off);
    float g[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) g[e] = to_float<TDO>(d_out[off + e]);
    sum = g[0] * o.x + g[1] * o.y + g[2] * o.z + g[3] * o.w;
    if (kWriteLow) {
#pragma unroll
      for (int e = 0; e < 4; ++e) d_out_low[off + e] = from_float<TLOW>(g[e]);
    }
  }
#pragma unroll
  for (int s = kLanes / 2; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  if (row < rows && lane == 0) dbar[row] = sum;
}

template <typename TDO, typename TLOW, bool kWriteLow>
int dbar_by_dim(const float* out, const void* d_out, int64_t rows, int head_dim, float* dbar, void* low,
                cudaStream_t s) {
  const int64_t threads = rows * (head_dim / 4);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  const TDO* g = static_cast<const TDO*>(d_out);
  TLOW* l = static_cast<TLOW*>(low);
  ProfileScope prof(SA_KERNEL_DBAR, s);
  switch (head_dim) {
    case 16: dbar_kernel<TDO, TLOW, 16, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l); break;
    case 32: dbar_kernel<TDO, TLOW, 32, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l); break;
    case 64: dbar_kernel<TDO, TLOW, 64, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l); break;
    case 128: dbar_kernel<TDO, TLOW, 128, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l); break;
    default: return SA_ERR_UNSUPPORTED;
  }
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

template <typename TDO>
int dbar_by_low(const float* out, const void* d_out, int64_t rows, int head_dim, float* dbar, void* low,
                int low_dtype, cudaStream_t s) {
  if (low == nullptr) return dbar_by_dim<TDO, float, false>(out, d_out, rows, head_dim, dbar, nullptr, s);
  if (low_dtype == SA_BF16) return dbar_by_dim<TDO, __nv_bfloat16, true>(out, d_out, rows, head_dim, dbar, low, s);
  if (low_dtype == SA_F16) return dbar_by_dim<TDO, __half, true>(out, d_out, rows, head_dim, dbar, low, s);
  if (low_dtype == SA_F32) return dbar_by_dim<TDO, float, true>(out, d_out, rows, head_dim, dbar, low, s);
  return SA_ERR_BAD_ARGUMENT;
}

// ---- fold + cast ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) fold_cast_kernel(const float* __restrict__ acc, const float* __restrict__ acc0,
                                                        T* __restrict__ dst, int heads, int64_t per_head,
                                                        int64_t total4) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total4) return;
  int64_t e = idx * 4;
  int64_t row = e / per_head;                 // (batch, head) row
  int64_t within = e - row * per_head;
  int b = (int)(row / heads), h = (int)(row - (int64_t)b * heads);
  float4 a = *reinterpret_cast<const float4*>(acc + e);
  if (h == 0 && acc0 != nullptr) {
    float4 z = *reinterpret_cast<const float4*>(acc0 + (int64_t)b * per_head + within);
    a.x += z.x; a.y += z.y; a.z += z.z; a.w += z.w;
  }
  dst[e + 0] = from_float<T>(a.x);
  dst[e + 1] = from_float<T>(a.y);
  dst[e + 2] = from_float<T>(a.z);
  dst[e + 3] = from_float<T>(a.w);
}

// ---- decode -----------------------------------------------------------------------------------------
constexpr int kDecThreads = 128;
constexpr int kDecSplitMin = 512;             // keys per CTA: a multiple of 512, chosen per call so that the grid
constexpr int kDecSplitMax = 4096;            //   has a few waves of CTAs and the combine pass stays short

// Keys per CTA for `t` cached keys and `rows` = batch * heads query rows.
static int decode_split_keys(int t, int rows) {
  const int target_splits = (148 * 8 + rows - 1) / rows;            // about eight CTAs per SM in total
  int keys = (t + target_splits - 1) / target_splits;
  keys = (keys + kDecSplitMin - 1) / kDecSplitMin * kDecSplitMin;
  if (keys < kDecSplitMin) keys = kDecSplitMin;
  if (keys > kDecSplitMax) keys = kDecSplitMax;
  return keys;
}

template <typename T>
__global__ void append_kernel(const T* __restrict__ k1, const T* __restrict__ v1, T* __restrict__ kc,
                              T* __restrict__ vc, int rows, int capacity, int length, int D) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * D) return;
  int n = idx / D, d = idx - n * D;
  int64_t dst = ((int64_t)n * capacity + length) * D + d;
  kc[dst] = k1[idx];
  vc[dst] = v1[idx];
}

// 16-byte load of 8 (bf16 / fp16) or two 16-byte loads of 8 fp32 elements, converted to fp32.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = to_float<T>(h[e]);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 c = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = c.x; x[5] = c.y; x[6] = c.z; x[7] = c.w;
  }
}

// grid (splits, batch * heads).  A group of D / 8 lanes owns one key per step; every thread keeps kUnroll
// 16-byte loads in flight so that a CTA streams its 512 keys of K, then of V, at memory speed.
template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads) decode_attend_kernel(
    const T* __restrict__ q1, const T* __restrict__ kc, const T* __restrict__ vc, const float* __restrict__ selected,
    float* __restrict__ partial, float* __restrict__ sel_new, int heads, int groups, int t, int capacity,
    int exempt, float scale, int split_keys) {
  constexpr int kLanes = D / 8;                       // lanes per key
  constexpr int kKeysPerStep = kDecThreads / kLanes;  // keys the CTA covers per step
  constexpr int kUnroll = 4;
  __shared__ float zs[kDecSplitMax];
  __shared__ float red[kDecThreads];
  __shared__ float accs[kKeysPerStep][D];

  const int n = blockIdx.y, split = blockIdx.x;
  const int b = n / heads, h = n - b * heads;
  const int per = heads / groups, g = h / per;
  const bool selector = (h - g * per) == 0;
  const int c0 = split * split_keys, c1 = min(t, c0 + split_keys);
  const int grp = threadIdx.x / kLanes, lane = threadIdx.x % kLanes;

  float qv[8];
  load8<T>(q1 + (int64_t)n * D + lane * 8, qv);
  const T* kb = kc + (int64_t)n * capacity * D;
  const T* vb = vc + (int64_t)n * capacity * D;
  const float* selb = selected + ((int64_t)b * groups + g) * capacity;
  float* selnb = sel_new + ((int64_t)b * groups + g) * t;

  float local_max = -INFINITY;
  for (int base = c0; base < c1; base += kKeysPerStep * kUnroll) {   // uniform trip count: the shuffles need whole warps
    float dot[kUnroll];
    float kx[kUnroll][8];
    const bool full = base + kKeysPerStep * kUnroll <= c1;       // CTA-uniform: loads without per-key guards
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int j = base + u * kKeysPerStep + grp;
      if (full || j < c1) {
        load8<T>(kb + (int64_t)j * D + lane * 8, kx[u]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) kx[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      dot[u] = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) dot[u] = fmaf(qv[e], kx[u][e], dot[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int s = kLanes / 2; s > 0; s >>= 1) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], s);
      const int j = base + u * kKeysPerStep + grp;
      if (j < c1) {
        const float raw = dot[u] * scale;
        const float z = (raw - selb[j]) * kLog2e;
        if (lane == 0) {
          zs[j - c0] = z;
          if (selector) selnb[j] = (j >= exempt && j != t - 1 && raw > 0.f) ? raw : 0.f;
        }
        local_max = fmaxf(local_max, z);
      }
    }
  }
  red[threadIdx.x] = local_max;
  __syncthreads();
  for (int s = kDecThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + s]);
    __syncthreads();
  }
  const float m = red[0];
  __syncthreads();

  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  float den = 0.f;
  for (int base = c0; base < c1; base += kKeysPerStep * kUnroll) {
    float vx[kUnroll][8], w[kUnroll];
    const bool full = base + kKeysPerStep * kUnroll <= c1;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int j = base + u * kKeysPerStep + grp;
      if (full || j < c1) {
        load8<T>(vb + (int64_t)j * D + lane * 8, vx[u]);
        w[u] = exp2f(zs[j - c0] - m);
      } else {
        w[u] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) vx[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      den += w[u];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(w[u], vx[u][e], acc[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) accs[grp][lane * 8 + e] = acc[e];
  red[threadIdx.x] = (lane == 0) ? den : 0.f;
  __syncthreads();
  for (int s = kDecThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
    __syncthreads();
  }
  float* prow = partial + ((int64_t)n * gridDim.x + split) * (D + 2);
  for (int d = threadIdx.x; d < D; d += kDecThreads) {
    float sum = 0.f;
    for (int gg = 0; gg < kKeysPerStep; ++gg) sum += accs[gg][d];
    prow[d] = sum;
  }
  if (threadIdx.x == 0) {
    prow[D] = m;
    prow[D + 1] = red[0];
  }
}

// grid (batch * heads), 128 threads: merges the per-split partial softmaxes.  The global maximum is found
// first so that the weighted sums over splits have no serial dependence: warp w folds splits w, w + 4, ...
// (lane l owns output columns l, l + 32, ...), then the four warps are added through shared memory.
__global__ void __launch_bounds__(128) decode_combine_kernel(const float* __restrict__ partial, float* __restrict__ y,
                                                             int splits, int D) {
  __shared__ float part[4][128 + 1];
  __shared__ float red[128];
  const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* prow = partial + (int64_t)n * splits * (D + 2);
  float m = -INFINITY;
  for (int s = threadIdx.x; s < splits; s += 128) m = fmaxf(m, prow[(int64_t)s * (D + 2) + D]);
  red[threadIdx.x] = m;
  __syncthreads();
  for (int st = 64; st > 0; st >>= 1) {
    if (threadIdx.x < st) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + st]);
    __syncthreads();
  }
  m = red[0];
  float den = 0.f, num[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int s = warp; s < splits; s += 4) {
    const float* p = prow + (int64_t)s * (D + 2);
    const float c = exp2f(p[D] - m);
    den = fmaf(p[D + 1], c, den);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int d = lane + 32 * u;
      if (d < D) num[u] = fmaf(p[d], c, num[u]);
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int d = lane + 32 * u;
    if (d < D) part[warp][d] = num[u];
  }
  if (lane == 0) part[warp][128] = den;
  __syncthreads();
  const int d = threadIdx.x;
  if (d < D) {
    const float nn = part[0][d] + part[1][d] + part[2][d] + part[3][d];
    const float dd = part[0][128] + part[1][128] + part[2][128] + part[3][128];
    y[(int64_t)n * D + d] = nn / dd;
  }
}

__global__ void decode_update_kernel(float* __restrict__ selected, const float* __restrict__ sel_new, int rows, int t,
                                     int capacity) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * t) return;
  int r = (int)(idx / t), j = (int)(idx - (int64_t)r * t);
  selected[(int64_t)r * capacity + j] += sel_new[idx];
}

template <typename T>
int decode_impl(int batch, int heads, int groups, int length, int capacity, int D, int exempt, const void* q1,
                const void* k1, const void* v1, void* kc, void* vc, float* selected, float* y, float* ws,
                cudaStream_t s) {
  const int rows = batch * heads, t = length + 1;
  const int split_keys = decode_split_keys(t, rows);
  const int splits = (t + split_keys - 1) / split_keys;
  float* partial = ws;
  float* sel_new = ws + (size_t)rows * splits * (D + 2);
  append_kernel<T><<<(rows * D + 255) / 256, 256, 0, s>>>(static_cast<const T*>(k1), static_cast<const T*>(v1),
                                                         static_cast<T*>(kc), static_cast<T*>(vc), rows, capacity,
                                                         length, D);
  SA_CUDA_CHECK(cudaGetLastError());
  dim3 grid(splits, rows);
  ProfileScope prof(SA_KERNEL_DECODE, s);   // the whole step: append, attend, combine, update
  const float scale = 1.0f / sqrtf((float)D);
  const T* q = static_cast<const T*>(q1);
  const T* kk = static_cast<const T*>(kc);
  const T* vv = static_cast<const T*>(vc);
#define SA_DECODE_LAUNCH(DIM)                                                                                   \
  decode_attend_kernel<T, DIM><<<grid, kDecThreads, 0, s>>>(q, kk, vv, selected, partial, sel_new, heads, groups, \
                                                            t, capacity, exempt, scale, split_keys)
  switch (D) {
    case 16: SA_DECODE_LAUNCH(16); break;
    case 32: SA_DECODE_LAUNCH(32); break;
    case 64: SA_DECODE_LAUNCH(64); break;
    case 128: SA_DECODE_LAUNCH(128); break;
    default: return SA_ERR_UNSUPPORTED;
  }
#undef SA_DECODE_LAUNCH
  SA_CUDA_CHECK(cudaGetLastError());
  decode_combine_kernel<<<rows, 128, 0, s>>>(partial, y, splits, D);
  SA_CUDA_CHECK(cudaGetLastError());
  const int64_t upd = (int64_t)batch * groups * t;
  decode_update_kernel<<<(unsigned)((upd + 255) / 256), 256, 0, s>>>(selected, sel_new, batch * groups, t, capacity);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace

int launch_dbar(const float* out, const void* d_out, int d_out_dtype, int64_t rows, int head_dim, float* dbar,
                void* d_out_lowp, int lowp_dtype, cudaStream_t s) {
  switch (d_out_dtype) {
    case SA_F32: return dbar_by_low<float>(out, d_out, rows, head_dim, dbar, d_out_lowp, lowp_dtype, s);
    case SA_BF16: return dbar_by_low<__nv_bfloat16>(out, d_out, rows, head_dim, dbar, d_out_lowp, lowp_dtype, s);
    case SA_F16: return dbar_by_low<__half>(out, d_out, rows, head_dim, dbar, d_out_lowp, lowp_dtype, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}

int launch_fold_cast(const float* acc, const float* acc0, void* dst, int dtype, int batch, int heads,
                     int64_t seq_times_dim, cudaStream_t s) {
  const int64_t total4 = (int64_t)batch * heads * seq_times_dim / 4;
  const unsigned blocks = (unsigned)((total4 + 255) / 256);
  switch (dtype) {
    case SA_F32:
      fold_cast_kernel<float><<<blocks, 256, 0, s>>>(acc, acc0, static_cast<float*>(dst), heads, seq_times_dim, total4);
      break;
    case SA_BF16:
      fold_cast_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(acc, acc0, static_cast<__nv_bfloat16*>(dst), heads,
                                                             seq_times_dim, total4);
      break;
    case SA_F16:
      fold_cast_kernel<__half><<<blocks, 256, 0, s>>>(acc, acc0, static_cast<__half*>(dst), heads, seq_times_dim,
                                                      total4);
      break;
    default: return SA_ERR_BAD_ARGUMENT;
  }
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

size_t decode_workspace_floats(int batch, int heads, int groups, int length, int head_dim) {
  const int t = length + 1;
  const size_t splits = (size_t)(t + kDecSplitMin - 1) / kDecSplitMin;       // upper bound: the smallest split size
  return (size_t)batch * heads * splits * (head_dim + 2) + (size_t)batch * groups * t;
}

int decode_step(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim, int exempt,
                const void* q1, const void* k1, const void* v1, void* kc, void* vc, float* selected, float* y,
                float* ws, cudaStream_t s) {
  switch (dtype) {
    case SA_F32:
      return decode_impl<float>(batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, kc, vc, selected,
                                y, ws, s);
    case SA_BF16:
      return decode_impl<__nv_bfloat16>(batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, kc, vc,
                                        selected, y, ws, s);
    case SA_F16:
      return decode_impl<__half>(batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, kc, vc, selected,
                                 y, ws, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}

}  // namespace sa
