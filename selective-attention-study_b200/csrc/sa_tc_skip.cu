// Tensor-core engine: the table of (query tile, key tile) pairs whose probabilities are all exactly zero.
//
// The history term F[i, j] never decreases with the query index i, so for a key tile that many later queries have
// selected against, every logit of a far query tile sits hundreds of units below its row maximum and ex2 (which
// flushes results below 2^-126 to zero) returns exactly 0 for the whole tile: the tile adds nothing to the output,
// to the row sums, or to any gradient.  Such a tile can be left out without changing a single bit of the result.
// The reference computes every causal tile (src/selective_attention/kernels.py:100-160); this is an option on top.
//
// Bound used, in log2 units, for query tile mi and key tile nj < mi of row n = (b, h):
//     z[i, j] - m[i]  <=  c1 |q_i| (|k_j| + |k_i|) - log2e * F[i, j]
// because z[i, j] = c1 q_i.k_j - log2e F[i, j], and the row maximum m[i] is at least the diagonal logit
// z[i, i] = c1 q_i.k_i (no query before i selects against key i, so F[i, i] = 0) >= -c1 |q_i| |k_i|; the row's
// log-sum-exp, which the backward subtracts, is at least m[i].  F[i, j] >= carry[mi][j], the selection key j has
// received from the queries before tile mi.  With Qn, Kn the largest row norms of a tile and Fmin the smallest
// carry over the key tile, the tile is dead when
//     c1 Qn[mi] (Kn[nj] + Kn[mi]) - log2e Fmin[mi][nj]  <  -kDeadMargin,
// kDeadMargin = 150 leaving 24 units beyond the flush threshold for the rounding of the bf16 products and sums.
// Tiles holding an exempt key (F = 0 there) are never dead; the diagonal tile is always kept.
#include <float.h>

#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {
namespace {

constexpr int kTile = 128;
constexpr float kDeadMargin = 150.f;

// Largest row norm of each 128-row tile of q (z = 0) and k (z = 1): one block per (tile, row n, tensor), one thread
// per token.  Tiles are counted in absolute positions; the query tensor starts at position q_offset (a prefill that
// continues from a cache), the key tensor at 0.
template <int D>
__global__ void __launch_bounds__(kTile) tile_norms_kernel(const __nv_bfloat16* __restrict__ q, RowLayout q_rows,
                                                           const __nv_bfloat16* __restrict__ k, RowLayout k_rows,
                                                           int heads, int seq, int ntiles, int q_offset,
                                                           float* __restrict__ qn, float* __restrict__ kn) {
  const int tile = blockIdx.x, n = blockIdx.y, which = blockIdx.z;
  const int b = n / heads, h = n - b * heads;
  const int t = tile * kTile + threadIdx.x;
  float ss = 0.f;
  if (t < seq && (which == 1 || t >= q_offset)) {
    const __nv_bfloat16* row = which == 0 ? q + q_rows.at(b, h, t - q_offset) : k + k_rows.at(b, h, t);
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(row + c * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
        ss = fmaf(lo, lo, fmaf(hi, hi, ss));
      }
    }
  }
  float m = sqrtf(ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float part[4];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0)
    (which == 0 ? qn : kn)[(int64_t)n * ntiles + tile] = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
}

// alive[n][mi][nj] for nj <= mi: one block per (query tile mi >= mi_first, sequence b); a warp takes every fourth key
// tile, finds the smallest carry over its 128 keys, and its lanes write the verdict for the heads of the sequence.
__global__ void __launch_bounds__(kTile) tile_table_kernel(const float* __restrict__ carry, const float* __restrict__ qn,
                                                           const float* __restrict__ kn, int heads, int seq, int ntiles,
                                                           int mi_first, float c1, uint8_t* __restrict__ alive) {
  const int mi = mi_first + blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* carry_row = carry + ((int64_t)b * (ntiles + 1) + mi) * seq;
  for (int nj = warp; nj <= mi; nj += 4) {
    float fmin = FLT_MAX;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = nj * kTile + c * 32 + lane;
      if (j < seq) fmin = fminf(fmin, carry_row[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) fmin = fminf(fmin, __shfl_xor_sync(0xffffffffu, fmin, o));
    for (int h = lane; h < heads; h += 32) {
      const int64_t n = (int64_t)b * heads + h;
      const float bound = c1 * qn[n * ntiles + mi] * (kn[n * ntiles + nj] + kn[n * ntiles + mi]) - kLog2e * fmin;
      alive[(n * ntiles + mi) * ntiles + nj] = (nj == mi || !(bound < -kDeadMargin)) ? 1 : 0;
    }
  }
}

}  // namespace

// Skipping is offered for bf16 operands at head_dim 64 / 128 up to 1024 tiles (the forward keeps a tile's list of live
// key tiles in shared memory).
size_t tile_table_bytes(const Problem& p) {
  const int64_t ntiles = (p.seq + kTile - 1) / kTile;
  if (p.dtype != SA_BF16 || (p.head_dim != 64 && p.head_dim != 128) || ntiles > 1024 || p.damp != SA_DAMP_NONE) return 0;
  const int64_t nrows = (int64_t)p.batch * p.heads;
  const int64_t table = (nrows * ntiles * ntiles + 255) & ~(int64_t)255;
  return (size_t)(table + 2 * nrows * ntiles * 4);
}


int build_tile_table(const Problem& p, const float* carry, cudaStream_t s) {
  const int ntiles = (p.seq + kTile - 1) / kTile;
  const int64_t nrows = (int64_t)p.batch * p.heads;
  if (tile_table_bytes(p) == 0 || p.tile_table == nullptr) return SA_ERR_UNSUPPORTED;
  uint8_t* alive = static_cast<uint8_t*>(p.tile_table);
  float* qn = reinterpret_cast<float*>(alive + ((nrows * ntiles * ntiles + 255) & ~(int64_t)255));
  float* kn = qn + nrows * ntiles;
  const RowLayout q_rows{p.q.sb, p.q.sh, p.q.st}, k_rows{p.k.sb, p.k.sh, p.k.st};
  const dim3 gn(ntiles, (unsigned)nrows, 2);
  count_launch();
  if (p.head_dim == 64)
    tile_norms_kernel<64><<<gn, kTile, 0, s>>>(static_cast<const __nv_bfloat16*>(p.q.ptr), q_rows,
                                               static_cast<const __nv_bfloat16*>(p.k.ptr), k_rows, p.heads, p.seq, ntiles,
                                               p.q_offset, qn, kn);
  else
    tile_norms_kernel<128><<<gn, kTile, 0, s>>>(static_cast<const __nv_bfloat16*>(p.q.ptr), q_rows,
                                                static_cast<const __nv_bfloat16*>(p.k.ptr), k_rows, p.heads, p.seq, ntiles,
                                                p.q_offset, qn, kn);
  SA_CUDA_CHECK(cudaGetLastError());
  count_launch();
  const int mi_first = p.q_offset / kTile;                // a continued prefill computes the query tiles from here on
  tile_table_kernel<<<dim3(ntiles - mi_first, p.batch), kTile, 0, s>>>(carry, qn, kn, p.heads, p.seq, ntiles, mi_first,
                                                                       p.scale * kLog2e, alive);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
