// Bandwidth-bound helpers of the Selective Attention operator (sm_100a):
//   dbar      dbar[row] = sum_d dO[row, d] * out[row, d], optionally also dO rounded to bf16 / fp16
//             (reference: src/selective_attention/kernels.py:635-636)
//   fold/cast dq = cast(dq_acc + [head 0] dq0)            (reference: kernels.py:662-666)
//   decode    one cached decode step                       (reference: src/selective_attention/mixers.py:115-130)
#include "sa_common.cuh"
#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace {

// ---- dbar -----------------------------------------------------------------------------------------
// A group of D / 4 consecutive lanes owns one row; every lane handles 4 consecutive elements.
template <typename TDO, typename TLOW, int D, bool kWriteLow>
__global__ void __launch_bounds__(256) dbar_kernel(const float* __restrict__ out, const TDO* __restrict__ d_out,
                                                   int64_t rows, float* __restrict__ dbar,
                                                   TLOW* __restrict__ d_out_low, bool strided, RowLayout in_rows, int heads,
                                                   int seq) {
  constexpr int kLanes = D / 4;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / kLanes;
  const int lane = (int)(gid % kLanes);
  float sum = 0.f;
  if (row < rows) {
    const int64_t off = row * D + lane * 4;
    int64_t off_in = off;
    if (strided) {                            // d_out rows sit in the caller's (batch, seq, heads, head_dim) activation gradient
      const int64_t bh = row / seq;
      const int64_t t = row - bh * seq;
      const int b = (int)(bh / heads), h = (int)(bh - (int64_t)b * heads);
      off_in = in_rows.at(b, h, t) + lane * 4;
    }
    float4 o = *reinterpret_cast<const float4*>(out + off);
    float g[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) g[e] = to_float<TDO>(d_out[off_in + e]);
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
                const RowLayout* in_rows, int heads, int seq, cudaStream_t s) {
  const bool strided = in_rows != nullptr;
  const RowLayout rl = strided ? *in_rows : RowLayout{0, 0, 0};
  const int64_t threads = rows * (head_dim / 4);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  const TDO* g = static_cast<const TDO*>(d_out);
  TLOW* l = static_cast<TLOW*>(low);
  ProfileScope prof(SA_KERNEL_DBAR, s);
  switch (head_dim) {
    case 16: count_launch(), dbar_kernel<TDO, TLOW, 16, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l, strided, rl, heads, seq); break;
    case 32: count_launch(), dbar_kernel<TDO, TLOW, 32, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l, strided, rl, heads, seq); break;
    case 64: count_launch(), dbar_kernel<TDO, TLOW, 64, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l, strided, rl, heads, seq); break;
    case 128: count_launch(), dbar_kernel<TDO, TLOW, 128, kWriteLow><<<blocks, 256, 0, s>>>(out, g, rows, dbar, l, strided, rl, heads, seq); break;
    default: return SA_ERR_UNSUPPORTED;
  }
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

template <typename TDO>
int dbar_by_low(const float* out, const void* d_out, int64_t rows, int head_dim, float* dbar, void* low,
                int low_dtype, const RowLayout* in_rows, int heads, int seq, cudaStream_t s) {
  if (low == nullptr) return dbar_by_dim<TDO, float, false>(out, d_out, rows, head_dim, dbar, nullptr, in_rows, heads, seq, s);
  if (low_dtype == SA_BF16) return dbar_by_dim<TDO, __nv_bfloat16, true>(out, d_out, rows, head_dim, dbar, low, in_rows, heads, seq, s);
  if (low_dtype == SA_F16) return dbar_by_dim<TDO, __half, true>(out, d_out, rows, head_dim, dbar, low, in_rows, heads, seq, s);
  if (low_dtype == SA_F32) return dbar_by_dim<TDO, float, true>(out, d_out, rows, head_dim, dbar, low, in_rows, heads, seq, s);
  return SA_ERR_BAD_ARGUMENT;
}

// ---- fold + cast ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) fold_cast_kernel(const float* __restrict__ acc, const float* __restrict__ acc0,
                                                        T* __restrict__ dst, int heads, int64_t per_head,
                                                        int64_t total4, bool strided, RowLayout dst_rows, int head_dim) {
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
  int64_t o = e;
  if (strided) {                              // rows go into the caller's (batch, seq, ..., heads, head_dim) gradient buffer
    const int64_t t = within / head_dim;
    o = dst_rows.at(b, h, t) + (within - t * head_dim);
  }
  dst[o + 0] = from_float<T>(a.x);
  dst[o + 1] = from_float<T>(a.y);
  dst[o + 2] = from_float<T>(a.z);
  dst[o + 3] = from_float<T>(a.w);
}

// ---- decode -----------------------------------------------------------------------------------------
constexpr int kDecThreads = 128;
constexpr int kDecSplitMin = 512;             // keys per CTA: a multiple of 512, at least 512
constexpr int kDecCtasPerSm = 4;              // attend CTAs resident per SM (48 KB of stages each)

// Keys per CTA for `t` cached keys and `rows` = batch * heads query rows: the grid is about one full wave of
// resident CTAs, so no SM is left with a straggler and the combine pass stays short.
static int decode_split_keys(int t, int rows) {
  int target_splits = 148 * kDecCtasPerSm / rows;
  if (target_splits < 1) target_splits = 1;
  int keys = (t + target_splits - 1) / target_splits;
  keys = (keys + kDecSplitMin - 1) / kDecSplitMin * kDecSplitMin;
  if (keys < kDecSplitMin) keys = kDecSplitMin;
  return keys;
}

// Writes the new key and value into the cache and clears the tickets the attend kernel counts CTAs with.
// With `knorm` (the per-key norms a decode that leaves out dead keys relies on) also stores the new key's norm.
template <typename T>
__global__ void append_kernel(const T* __restrict__ k1, const T* __restrict__ v1, T* __restrict__ kc,
                              T* __restrict__ vc, int rows, int capacity, int length, int D,
                              unsigned int* __restrict__ tickets, int n_tickets, float* __restrict__ knorm) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n_tickets) tickets[idx] = 0u;
  if (knorm != nullptr && idx < rows) {
    float ss = 0.f;
    for (int d = 0; d < D; ++d) {
      const float x = to_float<T>(k1[(int64_t)idx * D + d]);
      ss = fmaf(x, x, ss);
    }
    knorm[(int64_t)idx * capacity + length] = sqrtf(ss);
  }
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

// 16-byte load of 8 (bf16 / fp16) or two 16-byte loads of 8 fp32 elements from shared memory, converted to fp32.
template <typename T>
__device__ __forceinline__ void load8_shared(const uint8_t* p, float (&x)[8]) {
  load8<T>(reinterpret_cast<const T*>(p), x);
}

// Untiled bulk copy global -> shared memory, completion counted in bytes on an mbarrier.  Both addresses and the
// size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

constexpr int kDecStages = 3;                   // stages of 8 KB of K + 8 KB of V
constexpr int kDecStageBytes = 8192;            // per tensor
constexpr size_t kDecSmemBytes = (size_t)kDecStages * 2 * kDecStageBytes + 128;
constexpr int kDecMaxLive = 512;                // stages (of 8 KB) of a CTA's key range when dead stages are left out
constexpr float kDecDeadMargin = 150.f;         // binades below the newest key's logit at which a key counts as dead

// Merges the per-split partial softmaxes of one query row; called by all 128 threads of a CTA.  The global
// maximum is found first so that the weighted sums over splits have no serial dependence: warp w folds splits
// w, w + 4, ... (lane l owns output columns l, l + 32, ...), then the four warps are added through shared memory.
// The partials were written by other CTAs: they are read past the L1 cache.
__device__ __forceinline__ void decode_combine_row(const float* prow, float* yrow, int splits, int D,
                                                   float (*part)[128 + 1], float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float m = -INFINITY;
  for (int s = threadIdx.x; s < splits; s += 128) m = fmaxf(m, __ldcg(prow + (int64_t)s * (D + 2) + D));
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
    const float c = exp2f(__ldcg(p + D) - m);
    den = fmaf(__ldcg(p + D + 1), c, den);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int d = lane + 32 * u;
      if (d < D) num[u] = fmaf(__ldcg(p + d), c, num[u]);
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
    yrow[d] = nn / dd;
  }
}

// grid = batch * heads * splits CTAs (a row's splits are neighbours).  One thread streams the CTA's keys of K and V through a ring of shared-memory
// stages with bulk copies, kDecStages - 1 stages (32 KB) ahead of the arithmetic, so the bytes in flight do not
// depend on how the arithmetic is scheduled.  A group of D / 8 lanes owns every (128 / lanes)-th key of a stage
// and keeps its own running maximum, denominator and weighted sum (one pass, rescaled when its maximum grows);
// the groups are merged at the end.
//
// LIVE (optional, needs the per-key norms `knorm`): the history term of a key only grows, so most of a long cache
// can be dead for the new query -- its weight exp2(z - m) is below 2^-150 and adds nothing to fp32 sums of order one.
// A key is dead when  c1 |q| |k_j| - log2e selected[j]  <  z_new - 150, z_new being the logit of the newest key (its
// history term is zero, and the row maximum is at least that).  A CTA first marks the 64-key stages of its range that
// hold a live key (it reads 8 bytes per key for that instead of the 2 x 128 or 256 of K and V) and then streams
// only those.  The CTAs of a selecting head stay dense: the new query's selection is needed for every key.
template <typename T, int D, bool LIVE>
__global__ void __launch_bounds__(kDecThreads) decode_attend_kernel(
    const T* __restrict__ q1, const T* __restrict__ kc, const T* __restrict__ vc, float* selected,
    float* __restrict__ partial, float* __restrict__ sel_new, int heads, int groups, int t, int capacity,
    int exempt, float scale, int split_keys, tc::WaitCtx status, float* __restrict__ y, unsigned int* __restrict__ row_tickets, unsigned int* __restrict__ split_tickets, int splits,
    const float* __restrict__ knorm) {
  constexpr int kLanes = D / 8;                                   // lanes per key
  constexpr int kGroups = kDecThreads / kLanes;                   // keys the CTA covers per step
  constexpr int kRowBytes = D * (int)sizeof(T);
  constexpr int kStageKeys = kDecStageBytes / kRowBytes;
  constexpr int kPer = kStageKeys / kGroups;                      // keys per group per stage (4, fp32: 2)
  static_assert(kPer >= 1 && kPer * kGroups == kStageKeys, "stage layout");
  extern __shared__ uint8_t dec_smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dec_smem_raw) + 127) & ~uintptr_t(127));
  __shared__ uint64_t full[kDecStages];
  __shared__ float red[kDecThreads];
  __shared__ float gmax[kGroups];
  __shared__ float accs[kGroups][D];
  __shared__ float part[4][128 + 1];
  __shared__ unsigned int ticket_s[2];
  __shared__ uint16_t live_s[LIVE ? kDecMaxLive : 1];             // LIVE: the stages of this CTA's range that hold a live key
  __shared__ unsigned int live_bits[LIVE ? kDecMaxLive / 32 : 1];
  __shared__ int live_n_s;

  const int n = (int)(blockIdx.x / (unsigned)splits), split = (int)(blockIdx.x % (unsigned)splits);
  const int b = n / heads, h = n - b * heads;
  const int per = heads / groups, g = h / per;
  const bool selector = (h - g * per) == 0;
  const int c0 = split * split_keys, c1 = min(t, c0 + split_keys);
  const int n_stages = (c1 - c0 + kStageKeys - 1) / kStageKeys;
  const int grp = threadIdx.x / kLanes, lane = threadIdx.x % kLanes;
  const uint8_t* kb = reinterpret_cast<const uint8_t*>(kc + (int64_t)n * capacity * D);
  const uint8_t* vb = reinterpret_cast<const uint8_t*>(vc + (int64_t)n * capacity * D);

  const bool sparse = LIVE && !selector;                          // this CTA leaves out dead stages
  auto stage_of = [&](int it) { return sparse ? (int)live_s[it] : it; };
  auto issue = [&](int it) {                                      // thread 0 only; `it` counts the stages this CTA streams
    const int st = it;
    const int j0 = c0 + stage_of(it) * kStageKeys;
    const uint32_t bytes = (uint32_t)(min(kStageKeys, c1 - j0) * kRowBytes);
    uint8_t* dst = ring + (size_t)(st % kDecStages) * 2 * kDecStageBytes;
    uint64_t* bar = &full[st % kDecStages];
    tc::mbar_expect_tx(bar, 2 * bytes);
    bulk_load(dst, kb + (int64_t)j0 * kRowBytes, bytes, bar);
    bulk_load(dst + kDecStageBytes, vb + (int64_t)j0 * kRowBytes, bytes, bar);
  };
  float qv[8];
  load8<T>(q1 + (int64_t)n * D + lane * 8, qv);
  const float* selb = selected + ((int64_t)b * groups + g) * capacity;
  float* selnb = sel_new + ((int64_t)b * groups + g) * t;
  int n_iter = n_stages;
  if (sparse) {
    // |q| and the newest key's logit, by every group of lanes (each holds the whole of q between its lanes)
    float kx[8], ss = 0.f, dot = 0.f;
    load8<T>(kc + ((int64_t)n * capacity + (t - 1)) * D + lane * 8, kx);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      ss = fmaf(qv[e], qv[e], ss);
      dot = fmaf(qv[e], kx[e], dot);
    }
#pragma unroll
    for (int sft = kLanes / 2; sft > 0; sft >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, sft);
      dot += __shfl_xor_sync(0xffffffffu, dot, sft);
    }
    const float thr = (dot * scale - selb[t - 1]) * kLog2e - kDecDeadMargin;
    const float cq = scale * kLog2e * sqrtf(ss);
    const float* kn = knorm + (int64_t)n * capacity;
    for (int w = threadIdx.x; w < (n_stages + 31) / 32; w += kDecThreads) live_bits[w] = 0u;
    __syncthreads();
    constexpr int kAhead = 4;                                      // independent loads in flight per thread
    for (int base = c0 + threadIdx.x; base < c1; base += kDecThreads * kAhead) {
      float nrm[kAhead], sel[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int j = base + u * kDecThreads;
        nrm[u] = (j < c1) ? __ldg(kn + j) : 0.f;
        sel[u] = (j < c1) ? __ldcg(selb + j) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int j = base + u * kDecThreads;
        if (j < c1 && cq * nrm[u] - kLog2e * sel[u] >= thr) {
          const int st = (j - c0) / kStageKeys;
          atomicOr(&live_bits[st >> 5], 1u << (st & 31));
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {                                        // compact the marked stages, in order
      int count = 0;
      for (int w0 = 0; w0 < (n_stages + 31) / 32; w0 += 32) {
        const int w = w0 + threadIdx.x;
        const unsigned int bits = (w < (n_stages + 31) / 32) ? live_bits[w] : 0u;
        int mine = __popc(bits), before = mine;
#pragma unroll
        for (int sft = 1; sft < 32; sft <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, before, sft);
          if ((int)threadIdx.x >= sft) before += v;
        }
        const int total = __shfl_sync(0xffffffffu, before, 31);
        int pos = count + before - mine;
        for (unsigned int rest = bits; rest != 0u; rest &= rest - 1u) live_s[pos++] = (uint16_t)(w * 32 + __ffs(rest) - 1);
        count += total;
      }
      if (threadIdx.x == 0) live_n_s = count;
    }
    __syncthreads();
    n_iter = live_n_s;
  }
  if (threadIdx.x == 0) {
    for (int st = 0; st < kDecStages; ++st) tc::mbar_init(&full[st], 1);
    tc::mbar_init_fence();
    for (int st = 0; st < min(kDecStages - 1, n_iter); ++st) issue(st);
  }
  __syncthreads();                                                // barriers initialised before anyone waits

  float m = -INFINITY, den = 0.f, acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int st = 0; st < n_iter; ++st) {
    const int j0 = c0 + stage_of(st) * kStageKeys;
    float sv[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u) {                              // the history sums arrive while the stage is awaited
      const int j = j0 + u * kGroups + grp;
      sv[u] = (j < c1) ? selb[j] : 0.f;
    }
    // the slot that stage st + kDecStages - 1 uses was read in iteration st - 1; every thread is past it
    if (threadIdx.x == 0 && st + kDecStages - 1 < n_iter) issue(st + kDecStages - 1);
    tc::mbar_wait(&full[st % kDecStages], (st / kDecStages) & 1, status, 600);
    const uint8_t* ks = ring + (size_t)(st % kDecStages) * 2 * kDecStageBytes;
    const uint8_t* vs = ks + kDecStageBytes;

    float z[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      float kx[8];
      load8_shared<T>(ks + (u * kGroups + grp) * kRowBytes + lane * 8 * (int)sizeof(T), kx);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) dot = fmaf(qv[e], kx[e], dot);
      z[u] = dot;
    }
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
#pragma unroll
      for (int sft = kLanes / 2; sft > 0; sft >>= 1) z[u] += __shfl_xor_sync(0xffffffffu, z[u], sft);
    }
    float mx = m;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int j = j0 + u * kGroups + grp;
      const float raw = z[u] * scale;
      if (j < c1) {
        if (selector && lane == 0) selnb[j] = (j >= exempt && j != t - 1 && raw > 0.f) ? raw : 0.f;
        z[u] = (raw - sv[u]) * kLog2e;
      } else {
        z[u] = -INFINITY;                                         // past the end: the stage holds no data there
      }
      mx = fmaxf(mx, z[u]);
    }
    if (mx > m) {                                                 // the group's maximum grew: rescale its sums
      const float c = exp2f(m - mx);                              // m = -inf on the first keys: c = 0
      den *= c;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= c;
      m = mx;
    }
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      if (z[u] != -INFINITY) {
        const float w = exp2f(z[u] - m);
        float vx[8];
        load8_shared<T>(vs + (u * kGroups + grp) * kRowBytes + lane * 8 * (int)sizeof(T), vx);
        den += w;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, vx[e], acc[e]);
      }
    }
    __syncthreads();                                              // stage read by everyone: its slot may be refilled
  }

  // merge the groups: common maximum, then rescaled sums
  if (lane == 0) gmax[grp] = m;
  __syncthreads();
  float cta_max = -INFINITY;
#pragma unroll 4
  for (int gg = 0; gg < kGroups; ++gg) cta_max = fmaxf(cta_max, gmax[gg]);
  const float c = (m == -INFINITY) ? 0.f : exp2f(m - cta_max);   // a group that saw no key contributes nothing
#pragma unroll
  for (int e = 0; e < 8; ++e) accs[grp][lane * 8 + e] = acc[e] * c;
  red[threadIdx.x] = (lane == 0) ? den * c : 0.f;
  __syncthreads();
  for (int sft = kDecThreads / 2; sft > 0; sft >>= 1) {
    if (threadIdx.x < sft) red[threadIdx.x] += red[threadIdx.x + sft];
    __syncthreads();
  }
  float* prow = partial + ((int64_t)n * splits + split) * (D + 2);
  for (int d = threadIdx.x; d < D; d += kDecThreads) {
    float sum = 0.f;
    for (int gg = 0; gg < kGroups; ++gg) sum += accs[gg][d];
    prow[d] = sum;
  }
  if (threadIdx.x == 0) {
    prow[D] = cta_max;
    prow[D + 1] = red[0];
  }

  // The last CTA of a query row merges the row's partials into y; the last of the `per` heads that share a
  // history vector to finish a key range adds the new selection of that range to it (every reader is done).
  __threadfence();                                                // partials and sel_new visible before the ticket
  __syncthreads();
  if (threadIdx.x == 0) {
    ticket_s[0] = atomicAdd(&row_tickets[n], 1u);
    ticket_s[1] = atomicAdd(&split_tickets[((int64_t)b * groups + g) * splits + split], 1u);
  }
  __syncthreads();
  const bool last_of_row = ticket_s[0] == (unsigned)splits - 1;
  const bool last_of_range = ticket_s[1] == (unsigned)per - 1;
  if (!last_of_row && !last_of_range) return;
  __threadfence();
  if (last_of_range) {
    float* sel_rw = selected + ((int64_t)b * groups + g) * capacity;
    constexpr int kBatch = 8;                                     // independent loads in flight per thread
    for (int base = c0 + threadIdx.x; base < c1; base += kDecThreads * kBatch) {
      float old_v[kBatch], new_v[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int j = base + u * kDecThreads;
        old_v[u] = (j < c1) ? __ldcg(sel_rw + j) : 0.f;
        new_v[u] = (j < c1) ? __ldcg(selnb + j) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int j = base + u * kDecThreads;
        if (j < c1) sel_rw[j] = old_v[u] + new_v[u];
      }
    }
  }
  if (last_of_row)
    decode_combine_row(partial + (int64_t)n * splits * (D + 2), y + (int64_t)n * D, splits, D, part, red);
}

template <typename T>
int decode_impl(int batch, int heads, int groups, int length, int capacity, int D, int exempt, const void* q1,
                const void* k1, const void* v1, void* kc, void* vc, float* selected, float* y, float* ws,
                float* knorm, cudaStream_t s) {
  const int rows = batch * heads, t = length + 1;
  // With key norms most CTAs find nothing to stream and only the selecting heads stay dense: short key ranges (1024
  // keys; 512 and 2048 measured slower) then spread those heads over the whole GPU.
  const int split_keys = (knorm != nullptr) ? 2 * kDecSplitMin : decode_split_keys(t, rows);
  const int splits = (t + split_keys - 1) / split_keys;
  float* partial = ws;
  float* sel_new = partial + (size_t)rows * splits * (D + 2);
  unsigned int* row_tickets = reinterpret_cast<unsigned int*>(sel_new + (size_t)batch * groups * t);
  unsigned int* split_tickets = row_tickets + rows;
  const int n_tickets = rows + batch * groups * splits;
  const int append_threads = rows * D > n_tickets ? rows * D : n_tickets;
  ProfileScope prof(SA_KERNEL_DECODE, s);   // the whole step: append, then attend with its merge and update
  count_launch();
  append_kernel<T><<<(append_threads + 255) / 256, 256, 0, s>>>(
      static_cast<const T*>(k1), static_cast<const T*>(v1), static_cast<T*>(kc), static_cast<T*>(vc), rows, capacity,
      length, D, row_tickets, n_tickets, knorm);
  SA_CUDA_CHECK(cudaGetLastError());
  const unsigned grid = (unsigned)rows * (unsigned)splits;
  const float scale = 1.0f / sqrtf((float)D);
  const T* q = static_cast<const T*>(q1);
  const T* kk = static_cast<const T*>(kc);
  const T* vv = static_cast<const T*>(vc);
  tc::WaitCtx status;
  if (int st = tc::wait_ctx(&status)) return st;
  // dead stages are left out when the norms are given and a CTA's range fits the stage list
  const bool live = knorm != nullptr && split_keys / (kDecStageBytes / (D * (int)sizeof(T))) <= kDecMaxLive;
#define SA_DECODE_LAUNCH_ONE(DIM, LIVE_)                                                                           \
  do {                                                                                                             \
    SA_CUDA_CHECK(cudaFuncSetAttribute(decode_attend_kernel<T, DIM, LIVE_>,                                        \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDecSmemBytes));          \
    count_launch();                                                                                                \
    decode_attend_kernel<T, DIM, LIVE_><<<grid, kDecThreads, kDecSmemBytes, s>>>(                                  \
        q, kk, vv, selected, partial, sel_new, heads, groups, t, capacity, exempt, scale, split_keys, status,      \
        y, row_tickets, split_tickets, splits, knorm);                                                            \
  } while (0)
#define SA_DECODE_LAUNCH(DIM)                                                                                      \
  do {                                                                                                             \
    if (live) SA_DECODE_LAUNCH_ONE(DIM, true);                                                                     \
    else SA_DECODE_LAUNCH_ONE(DIM, false);                                                                         \
  } while (0)
  switch (D) {
    case 16: SA_DECODE_LAUNCH(16); break;
    case 32: SA_DECODE_LAUNCH(32); break;
    case 64: SA_DECODE_LAUNCH(64); break;
    case 128: SA_DECODE_LAUNCH(128); break;
    default: return SA_ERR_UNSUPPORTED;
  }
#undef SA_DECODE_LAUNCH
#undef SA_DECODE_LAUNCH_ONE
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace

int launch_dbar(const float* out, const void* d_out, int d_out_dtype, int64_t rows, int head_dim, float* dbar,
                void* d_out_lowp, int lowp_dtype, const RowLayout* d_out_rows, int heads, int seq, cudaStream_t s) {
  switch (d_out_dtype) {
    case SA_F32: return dbar_by_low<float>(out, d_out, rows, head_dim, dbar, d_out_lowp, lowp_dtype, d_out_rows, heads, seq, s);
    case SA_BF16: return dbar_by_low<__nv_bfloat16>(out, d_out, rows, head_dim, dbar, d_out_lowp, lowp_dtype, d_out_rows, heads, seq, s);
    case SA_F16: return dbar_by_low<__half>(out, d_out, rows, head_dim, dbar, d_out_lowp, lowp_dtype, d_out_rows, heads, seq, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}

int launch_fold_cast(const float* acc, const float* acc0, void* dst, int dtype, int batch, int heads,
                     int64_t seq_times_dim, const RowLayout* dst_rows, int head_dim, cudaStream_t s) {
  const bool strided = dst_rows != nullptr;
  const RowLayout rl = strided ? *dst_rows : RowLayout{0, 0, 0};
  const int64_t total4 = (int64_t)batch * heads * seq_times_dim / 4;
  const unsigned blocks = (unsigned)((total4 + 255) / 256);
  switch (dtype) {
    case SA_F32:
      count_launch();
      fold_cast_kernel<float><<<blocks, 256, 0, s>>>(acc, acc0, static_cast<float*>(dst), heads, seq_times_dim, total4, strided, rl, head_dim);
      break;
    case SA_BF16:
      count_launch();
      fold_cast_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(acc, acc0, static_cast<__nv_bfloat16*>(dst), heads,
                                                             seq_times_dim, total4, strided, rl, head_dim);
      break;
    case SA_F16:
      count_launch();
      fold_cast_kernel<__half><<<blocks, 256, 0, s>>>(acc, acc0, static_cast<__half*>(dst), heads, seq_times_dim,
                                                      total4, strided, rl, head_dim);
      break;
    default: return SA_ERR_BAD_ARGUMENT;
  }
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

size_t decode_workspace_floats(int batch, int heads, int groups, int length, int head_dim) {
  const int t = length + 1;
  const size_t splits = (size_t)(t + kDecSplitMin - 1) / kDecSplitMin;       // upper bound: the smallest split size
  return (size_t)batch * heads * splits * (head_dim + 2) + (size_t)batch * groups * t   // partials, new selection
         + (size_t)batch * heads + (size_t)batch * groups * splits;                       // tickets
}

int decode_step(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim, int exempt,
                const void* q1, const void* k1, const void* v1, void* kc, void* vc, float* selected, float* y,
                float* ws, float* knorm, cudaStream_t s) {
  switch (dtype) {
    case SA_F32:
      return decode_impl<float>(batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, kc, vc, selected,
                                y, ws, knorm, s);
    case SA_BF16:
      return decode_impl<__nv_bfloat16>(batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, kc, vc,
                                        selected, y, ws, knorm, s);
    case SA_F16:
      return decode_impl<__half>(batch, heads, groups, length, capacity, head_dim, exempt, q1, k1, v1, kc, vc, selected,
                                 y, ws, knorm, s);
  }
  return SA_ERR_BAD_ARGUMENT;
}

}  // namespace sa
