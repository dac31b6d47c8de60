// CUDA-core (fp32 FFMA) engine of the Selective Attention operator.
//
// Exact fp32 products ("ieee"), every supported head_dim and dtype, any sequence length.  It is the
// accuracy path behind the fp32 parity bar and the path for shapes the tensor-core engine does not
// take; it is not the throughput path.
//
// Three kernels mirror the structure of the operator (reference: src/selective_attention/kernels.py):
//   carry    per key block, query blocks in causal order, running per-key selection sum written on
//            entry to every 32-query block                         (:111-138)
//   forward  per 32-query block of one head, online softmax over 64-key tiles of (L_h - F) (:140-194)
//   backward per 32-key block of one head, query blocks last to first; dV, dK in registers; dQ and the
//            head-0 selection gradients through fp32 atomics       (:196-268)
#pragma once
#include "sa_common.cuh"

namespace sa {
namespace simt {

constexpr int kThreads = 256;
constexpr int kQ = 32;         // query rows per tile (== kSimtCarryRows)
constexpr int kKF = 64;        // keys per tile, carry and forward kernels
constexpr int kKB = 32;        // keys per block, backward kernel

template <typename T>
__device__ __forceinline__ const T* row_ptr(const Strided& s, int b, int h) {
  return static_cast<const T*>(s.ptr) + b * s.sb + h * s.sh;
}

// Loads `rows` rows of D elements starting at token t0 into dst[rows][D + 1] as fp32, zero past seq.
template <typename T, int D>
__device__ __forceinline__ void load_tile(float* dst, const T* base, int64_t st, int t0, int rows, int seq) {
  for (int idx = threadIdx.x; idx < rows * D; idx += kThreads) {
    int r = idx / D, d = idx - r * D;
    int t = t0 + r;
    dst[r * (D + 1) + d] = (t < seq) ? to_float<T>(base[(int64_t)t * st + d]) : 0.f;
  }
}

// ---------------------------------------------------------------------------------------------------
// carry: grid (key blocks of 64, batch)
// ---------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) carry_kernel(Problem p, float* __restrict__ carry_out,
                                                         float* __restrict__ total_out, int nblocks) {
  extern __shared__ float smem[];
  float* k0s = smem;                       // [64][D + 1]
  float* q0s = k0s + kKF * (D + 1);        // [32][D + 1]
  float* part = q0s + kQ * (D + 1);        // [4][64]

  const int b = blockIdx.y;
  const int j0 = blockIdx.x * kKF;
  const T* q0 = row_ptr<T>(p.q0, b, 0);
  const T* k0 = row_ptr<T>(p.k0, b, 0);
  load_tile<T, D>(k0s, k0, p.k0.st, j0, kKF, p.seq);

  const int jl = threadIdx.x & 63;         // key within the block
  const int rg = threadIdx.x >> 6;         // row group: rows rg * 8 .. rg * 8 + 7
  const int j = j0 + jl;
  float running = 0.f;                     // meaningful in threads < 64
  float* carry_b = carry_out + (int64_t)b * nblocks * p.seq;

  for (int rb = j0 / kQ; rb < nblocks; ++rb) {
    __syncthreads();                       // previous iteration done with q0s / part
    load_tile<T, D>(q0s, q0, p.q0.st, rb * kQ, kQ, p.seq);
    __syncthreads();
    float colsum = 0.f;
    const float* kr = k0s + jl * (D + 1);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      int rl = rg * 8 + u;
      int i = rb * kQ + rl;
      const float* qr = q0s + rl * (D + 1);
      float acc = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) acc = fmaf(qr[d], kr[d], acc);
      float l0 = acc * p.scale;
      bool gate = (j < i) && (j >= p.exempt) && (i < p.seq) && (j < p.seq) && (l0 > 0.f);
      colsum += gate ? l0 : 0.f;
    }
    part[rg * kKF + jl] = colsum;
    __syncthreads();
    if (threadIdx.x < kKF) {
      if (j < p.seq) carry_b[(int64_t)rb * p.seq + j] = running;
      running += part[jl] + part[kKF + jl] + part[2 * kKF + jl] + part[3 * kKF + jl];
    }
  }
  if (threadIdx.x < kKF && j < p.seq) total_out[(int64_t)b * p.seq + j] = running;
}

// ---------------------------------------------------------------------------------------------------
// forward: grid (query tiles of 32 [heaviest first], batch * heads)
// ---------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) forward_kernel(Problem p, const float* __restrict__ carry,
                                                           float* __restrict__ out, float* __restrict__ lse2,
                                                           int nblocks) {
  extern __shared__ float smem[];
  float* qs = smem;                        // [32][D + 1]
  float* q0s = qs + kQ * (D + 1);          // [32][D + 1]
  float* ks = q0s + kQ * (D + 1);          // [64][D + 1]
  float* k0s = ks + kKF * (D + 1);         // [64][D + 1]
  float* vs = k0s + kKF * (D + 1);         // [64][D + 1]
  float* ss = vs + kKF * (D + 1);          // [32][65]  selection, then exclusive prefix
  float* ps = ss + kQ * (kKF + 1);         // [32][65]  exp2 tile

  constexpr int kDD = D / 8;               // output columns per thread
  const int mi = gridDim.x - 1 - blockIdx.x;
  const int n = blockIdx.y;
  const int b = n / p.heads, h = n - b * p.heads;
  const int m0 = mi * kQ;
  const T* qh = row_ptr<T>(p.q, b, h);
  const T* kh = row_ptr<T>(p.k, b, h);
  const T* vh = row_ptr<T>(p.v, b, h);
  const T* q0 = row_ptr<T>(p.q0, b, 0);
  const T* k0 = row_ptr<T>(p.k0, b, 0);

  load_tile<T, D>(qs, qh, p.q.st, m0, kQ, p.seq);
  load_tile<T, D>(q0s, q0, p.q0.st, m0, kQ, p.seq);

  const int r = threadIdx.x >> 3;          // query row in the tile
  const int cg = threadIdx.x & 7;          // column group
  const int i = m0 + r;
  float damp = 1.f;
  if (p.damp == SA_DAMP_LINEAR) damp = fminf(1.f, (float)p.train_len / (float)(i + 1));
  if (p.damp == SA_DAMP_SQRT) damp = fminf(1.f, sqrtf((float)p.train_len / (float)(i + 1)));

  float run_max = -INFINITY, run_den = 0.f;
  float acc[kDD];
#pragma unroll
  for (int dd = 0; dd < kDD; ++dd) acc[dd] = 0.f;
  const float* carry_row = carry + ((int64_t)b * nblocks + mi) * p.seq;
  const int last_key = min(m0 + kQ, p.seq);  // keys < last_key can be visible

  for (int n0 = 0; n0 < last_key; n0 += kKF) {
    __syncthreads();
    load_tile<T, D>(ks, kh, p.k.st, n0, kKF, p.seq);
    load_tile<T, D>(k0s, k0, p.k0.st, n0, kKF, p.seq);
    load_tile<T, D>(vs, vh, p.v.st, n0, kKF, p.seq);
    __syncthreads();
    float aff[8], sel[8];
    const float* qr = qs + r * (D + 1);
    const float* q0r = q0s + r * (D + 1);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int jl = cg + 8 * c, j = n0 + jl;
      const float* kr = ks + jl * (D + 1);
      const float* k0r = k0s + jl * (D + 1);
      float a = 0.f, a0 = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) {
        a = fmaf(qr[d], kr[d], a);
        a0 = fmaf(q0r[d], k0r[d], a0);
      }
      aff[c] = a * p.scale;
      float l0 = a0 * p.scale;
      bool gate = (j < i) && (j >= p.exempt) && (i < p.seq) && (j < p.seq) && (l0 > 0.f);
      sel[c] = gate ? l0 : 0.f;
      ss[r * (kKF + 1) + jl] = sel[c];
    }
    __syncthreads();
    if (threadIdx.x < kKF) {                // exclusive prefix down the 32 query rows, one key per thread
      float run = 0.f;
      for (int rr = 0; rr < kQ; ++rr) {
        float x = ss[rr * (kKF + 1) + threadIdx.x];
        ss[rr * (kKF + 1) + threadIdx.x] = run;
        run += x;
      }
    }
    __syncthreads();
    float z[8], tile_max = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int jl = cg + 8 * c, j = n0 + jl;
      bool causal = (j <= i) && (j < p.seq) && (i < p.seq);
      float hist = 0.f;
      if (causal) hist = (carry_row[j] + ss[r * (kKF + 1) + jl]) * damp;
      z[c] = causal ? (aff[c] - hist) * kLog2e : -INFINITY;
      tile_max = fmaxf(tile_max, z[c]);
    }
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
    float new_max = fmaxf(run_max, tile_max);
    float alpha = (new_max == -INFINITY) ? 1.f : exp2f(run_max - new_max);
    float rowsum = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float e = (z[c] == -INFINITY) ? 0.f : exp2f(z[c] - new_max);
      ps[r * (kKF + 1) + cg + 8 * c] = e;
      rowsum += e;
    }
    rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 1);
    rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 2);
    rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 4);
    run_den = run_den * alpha + rowsum;
    run_max = new_max;
#pragma unroll
    for (int dd = 0; dd < kDD; ++dd) acc[dd] *= alpha;
    __syncthreads();
    const float* pr = ps + r * (kKF + 1);
    for (int jl = 0; jl < kKF; ++jl) {
      float e = pr[jl];
      const float* vr = vs + jl * (D + 1) + cg;
#pragma unroll
      for (int dd = 0; dd < kDD; ++dd) acc[dd] = fmaf(e, vr[8 * dd], acc[dd]);
    }
  }
  if (i < p.seq) {
    float inv = 1.f / run_den;
    float* orow = out + ((int64_t)n * p.seq + i) * D;
#pragma unroll
    for (int dd = 0; dd < kDD; ++dd) orow[cg + 8 * dd] = acc[dd] * inv;
    if (cg == 0) lse2[(int64_t)n * p.seq + i] = run_max + log2f(run_den);
  }
}

// ---------------------------------------------------------------------------------------------------
// backward: grid (key blocks of 32, batch * heads); query blocks last to first
// ---------------------------------------------------------------------------------------------------
template <typename T, typename TDO, int D>
__global__ void __launch_bounds__(kThreads) backward_kernel(
    Problem p, const float* __restrict__ lse2, const float* __restrict__ carry, const float* __restrict__ dbar,
    const TDO* __restrict__ d_out, float* __restrict__ dq_acc, float* __restrict__ dk_acc,
    float* __restrict__ dq0, float* __restrict__ dk0, T* __restrict__ dv, int nblocks) {
  extern __shared__ float smem[];
  constexpr int P = D + 1, W = kKB + 1;
  float* ks = smem;                 // [32][P] keys of this head
  float* vs = ks + kKB * P;
  float* k0s = vs + kKB * P;
  float* qs = k0s + kKB * P;        // [32][P] query tile of this head
  float* q0s = qs + kQ * P;
  float* dos = q0s + kQ * P;
  float* as = dos + kQ * P;         // [32][W] attention
  float* zs = as + kQ * W;          // [32][W] dz
  float* gs = zs + kQ * W;          // [32][W] selection, prefix, suffix, then g
  float* lse_s = gs + kQ * W;       // [32]
  float* dbar_s = lse_s + kQ;       // [32]

  constexpr int kDD = D / 8;
  const int kb = blockIdx.x;
  const int n = blockIdx.y;
  const int b = n / p.heads, h = n - b * p.heads;
  const int j0 = kb * kKB;
  const T* qh = row_ptr<T>(p.q, b, h);
  const T* kh = row_ptr<T>(p.k, b, h);
  const T* vh = row_ptr<T>(p.v, b, h);
  const T* q0 = row_ptr<T>(p.q0, b, 0);
  const T* k0 = row_ptr<T>(p.k0, b, 0);
  const TDO* doh = d_out + (int64_t)n * p.seq * D;

  load_tile<T, D>(ks, kh, p.k.st, j0, kKB, p.seq);
  load_tile<T, D>(vs, vh, p.v.st, j0, kKB, p.seq);
  load_tile<T, D>(k0s, k0, p.k0.st, j0, kKB, p.seq);

  const int r = threadIdx.x >> 3;   // row index (query row in phase 1, key row / query row in phase 2)
  const int cg = threadIdx.x & 7;
  float dk_r[kDD], dv_r[kDD], dk0_r[kDD];
#pragma unroll
  for (int dd = 0; dd < kDD; ++dd) dk_r[dd] = dv_r[dd] = dk0_r[dd] = 0.f;
  float suffix = 0.f;               // threads < 32: sum of dz over queries in later tiles, key j0 + tid

  for (int rb = nblocks - 1; rb * kQ + kQ > j0 && rb >= 0; --rb) {
    const int m0 = rb * kQ;
    __syncthreads();
    load_tile<T, D>(qs, qh, p.q.st, m0, kQ, p.seq);
    load_tile<T, D>(q0s, q0, p.q0.st, m0, kQ, p.seq);
    for (int idx = threadIdx.x; idx < kQ * D; idx += kThreads) {
      int rr = idx / D, d = idx - rr * D;
      int t = m0 + rr;
      dos[rr * P + d] = (t < p.seq) ? to_float<TDO>(doh[(int64_t)t * D + d]) : 0.f;
    }
    if (threadIdx.x < kQ) {
      int t = m0 + threadIdx.x;
      lse_s[threadIdx.x] = (t < p.seq) ? lse2[(int64_t)n * p.seq + t] : 0.f;
      dbar_s[threadIdx.x] = (t < p.seq) ? dbar[(int64_t)n * p.seq + t] : 0.f;
    }
    __syncthreads();

    const int i = m0 + r;
    float aff[4], dov[4];
    bool gate[4];
    const float* qr = qs + r * P;
    const float* q0r = q0s + r * P;
    const float* dor = dos + r * P;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int jl = cg + 8 * c, j = j0 + jl;
      const float* kr = ks + jl * P;
      const float* k0r = k0s + jl * P;
      const float* vr = vs + jl * P;
      float a = 0.f, a0 = 0.f, dv_ = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) {
        a = fmaf(qr[d], kr[d], a);
        a0 = fmaf(q0r[d], k0r[d], a0);
        dv_ = fmaf(dor[d], vr[d], dv_);
      }
      aff[c] = a * p.scale;
      dov[c] = dv_;
      float l0 = a0 * p.scale;
      gate[c] = (j < i) && (j >= p.exempt) && (i < p.seq) && (j < p.seq) && (l0 > 0.f);
      gs[r * W + jl] = gate[c] ? l0 : 0.f;
    }
    __syncthreads();
    if (threadIdx.x < kKB) {          // exclusive prefix of the selection down the query rows
      float run = 0.f;
      for (int rr = 0; rr < kQ; ++rr) {
        float x = gs[rr * W + threadIdx.x];
        gs[rr * W + threadIdx.x] = run;
        run += x;
      }
    }
    __syncthreads();
    const float* carry_row = carry + ((int64_t)b * nblocks + rb) * p.seq;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int jl = cg + 8 * c, j = j0 + jl;
      bool causal = (j <= i) && (j < p.seq) && (i < p.seq);
      float attn = 0.f, dz = 0.f;
      if (causal) {
        float hist = carry_row[j] + gs[r * W + jl];
        attn = exp2f((aff[c] - hist) * kLog2e - lse_s[r]);
        dz = attn * (dov[c] - dbar_s[r]);
      }
      as[r * W + jl] = attn;
      zs[r * W + jl] = dz;
    }
    __syncthreads();
    if (threadIdx.x < kKB) {          // sum of dz over strictly later queries, per key
      float run = suffix;
      for (int rr = kQ - 1; rr >= 0; --rr) {
        float x = zs[rr * W + threadIdx.x];
        gs[rr * W + threadIdx.x] = run;
        run += x;
      }
      suffix = run;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int jl = cg + 8 * c;
      float later = gs[r * W + jl];
      gs[r * W + jl] = gate[c] ? -later : 0.f;
    }
    __syncthreads();

    // phase 2a: key-row accumulators (r = key row)
    for (int rr = 0; rr < kQ; ++rr) {
      float a = as[rr * W + r], z = zs[rr * W + r], g = gs[rr * W + r];
      const float* dor2 = dos + rr * P + cg;
      const float* qr2 = qs + rr * P + cg;
      const float* q0r2 = q0s + rr * P + cg;
#pragma unroll
      for (int dd = 0; dd < kDD; ++dd) {
        dv_r[dd] = fmaf(a, dor2[8 * dd], dv_r[dd]);
        dk_r[dd] = fmaf(z, qr2[8 * dd], dk_r[dd]);
        dk0_r[dd] = fmaf(g, q0r2[8 * dd], dk0_r[dd]);
      }
    }
    // phase 2b: query-row products (r = query row), accumulated across key blocks with atomics
    if (i < p.seq) {
      float dq_r[kDD], dq0_r[kDD];
#pragma unroll
      for (int dd = 0; dd < kDD; ++dd) dq_r[dd] = dq0_r[dd] = 0.f;
      for (int jl = 0; jl < kKB; ++jl) {
        float z = zs[r * W + jl], g = gs[r * W + jl];
        const float* kr = ks + jl * P + cg;
        const float* k0r = k0s + jl * P + cg;
#pragma unroll
        for (int dd = 0; dd < kDD; ++dd) {
          dq_r[dd] = fmaf(z, kr[8 * dd], dq_r[dd]);
          dq0_r[dd] = fmaf(g, k0r[8 * dd], dq0_r[dd]);
        }
      }
      float* dq_row = dq_acc + ((int64_t)n * p.seq + i) * D + cg;
      float* dq0_row = dq0 + ((int64_t)b * p.seq + i) * D + cg;
#pragma unroll
      for (int dd = 0; dd < kDD; ++dd) {
        atomicAdd(dq_row + 8 * dd, dq_r[dd] * p.scale);
        atomicAdd(dq0_row + 8 * dd, dq0_r[dd] * p.scale);
      }
    }
  }
  const int j = j0 + r;
  if (j < p.seq) {
    float* dk_row = dk_acc + ((int64_t)n * p.seq + j) * D + cg;
    float* dk0_row = dk0 + ((int64_t)b * p.seq + j) * D + cg;
    T* dv_row = dv + ((int64_t)n * p.seq + j) * D + cg;
#pragma unroll
    for (int dd = 0; dd < kDD; ++dd) {
      dk_row[8 * dd] = dk_r[dd] * p.scale;
      dv_row[8 * dd] = from_float<T>(dv_r[dd]);
      atomicAdd(dk0_row + 8 * dd, dk0_r[dd] * p.scale);
    }
  }
}

template <int D> constexpr size_t carry_smem() { return sizeof(float) * ((kKF + kQ) * (D + 1) + 4 * kKF); }
template <int D> constexpr size_t forward_smem() {
  return sizeof(float) * ((2 * kQ + 3 * kKF) * (D + 1) + 2 * kQ * (kKF + 1));
}
template <int D> constexpr size_t backward_smem() {
  return sizeof(float) * ((3 * kKB + 3 * kQ) * (D + 1) + 3 * kQ * (kKB + 1) + 2 * kQ);
}

template <typename T, int D>
int forward_impl(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  const int nb = (p.seq + kQ - 1) / kQ;
  SA_CUDA_CHECK(cudaFuncSetAttribute(carry_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)carry_smem<D>()));
  SA_CUDA_CHECK(cudaFuncSetAttribute(forward_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)forward_smem<D>()));
  dim3 gc((p.seq + kKF - 1) / kKF, p.batch);
  count_launch();
  carry_kernel<T, D><<<gc, kThreads, carry_smem<D>(), s>>>(p, carry, total, nb);
  SA_CUDA_CHECK(cudaGetLastError());
  dim3 gf(nb, p.batch * p.heads);
  count_launch();
  forward_kernel<T, D><<<gf, kThreads, forward_smem<D>(), s>>>(p, carry, out, lse2, nb);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

// The selection pass alone: carry checkpoints every 32 queries and the per-key totals.
template <typename T, int D>
int carry_impl(const Problem& p, float* carry, float* total, cudaStream_t s) {
  const int nb = (p.seq + kQ - 1) / kQ;
  SA_CUDA_CHECK(cudaFuncSetAttribute(carry_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)carry_smem<D>()));
  dim3 gc((p.seq + kKF - 1) / kKF, p.batch);
  count_launch();
  carry_kernel<T, D><<<gc, kThreads, carry_smem<D>(), s>>>(p, carry, total, nb);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

template <typename T, typename TDO, int D>
int backward_impl(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out,
                  float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  const int nb = (p.seq + kQ - 1) / kQ;
  SA_CUDA_CHECK(cudaFuncSetAttribute(backward_kernel<T, TDO, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)backward_smem<D>()));
  dim3 g((p.seq + kKB - 1) / kKB, p.batch * p.heads);
  count_launch();
  backward_kernel<T, TDO, D><<<g, kThreads, backward_smem<D>(), s>>>(
      p, lse2, carry, dbar, static_cast<const TDO*>(d_out), dq_acc, dk_acc, dq0, dk0, static_cast<T*>(dv), nb);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

template <typename T>
int forward_by_dim(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  switch (p.head_dim) {
    case 16: return forward_impl<T, 16>(p, out, lse2, carry, total, s);
    case 32: return forward_impl<T, 32>(p, out, lse2, carry, total, s);
    case 64: return forward_impl<T, 64>(p, out, lse2, carry, total, s);
    case 128: return forward_impl<T, 128>(p, out, lse2, carry, total, s);
  }
  return SA_ERR_UNSUPPORTED;
}

template <typename T>
int carry_by_dim(const Problem& p, float* carry, float* total, cudaStream_t s) {
  switch (p.head_dim) {
    case 16: return carry_impl<T, 16>(p, carry, total, s);
    case 32: return carry_impl<T, 32>(p, carry, total, s);
    case 64: return carry_impl<T, 64>(p, carry, total, s);
    case 128: return carry_impl<T, 128>(p, carry, total, s);
  }
  return SA_ERR_UNSUPPORTED;
}

template <typename T, typename TDO>
int backward_by_dim(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out,
                    float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  switch (p.head_dim) {
    case 16: return backward_impl<T, TDO, 16>(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
    case 32: return backward_impl<T, TDO, 32>(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
    case 64: return backward_impl<T, TDO, 64>(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
    case 128: return backward_impl<T, TDO, 128>(p, lse2, carry, dbar, d_out, dq_acc, dk_acc, dq0, dk0, dv, s);
  }
  return SA_ERR_UNSUPPORTED;
}

}  // namespace simt
}  // namespace sa
