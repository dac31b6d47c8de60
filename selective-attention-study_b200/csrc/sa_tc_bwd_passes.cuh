// Tensor-core engine, backward: the per-half arithmetic shared by the two backward kernels (head_dim 64 in
// sa_tc_bwd.cu, head_dim 128 in sa_tc_bwd_wide.cu).  One thread owns one key row (a TMEM lane) and 16 of the half's
// 64 query columns; see sa_tc_bwd.cu for the whole scheme.
#pragma once

#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {
namespace bwd {

constexpr int kTile = 128;
constexpr int kRowTile = 16384;      // bytes of a [128][64] bf16 operand tile
constexpr int kHalfTile = 8192;      // bytes of a [64][64] bf16 operand tile
constexpr int kGroups = 4;           // arithmetic warpgroups; each owns 16 of a half's 64 query columns
constexpr int kChunk = 64 / kGroups;
constexpr int kComputeThreads = 128 * kGroups;
constexpr int kThreads = kComputeThreads + 32;
constexpr int kComputeBarrier = 1;   // hardware barrier id of the arithmetic warps

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float load_ahead(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// Which (row n = batch x head, key tile nj) a CTA takes.  Dense: one row after the other, key tile 0 (the longest
// walk) first.  With a table of live tiles most walks are a few tiles long, except those of the key tiles that hold an
// exempt key, which stay live for every query tile: all rows' key tile 0 go first so that the long walks start together.
__device__ __forceinline__ void tile_of_block(unsigned block, int ntiles, int nrows, bool sparse, int& n, int& nj) {
  if (!sparse) {
    n = (int)(block / ntiles);
    nj = (int)(block % ntiles);
  } else if ((int)block < nrows) {
    n = (int)block;
    nj = 0;
  } else {
    const unsigned r = block - nrows;
    n = (int)(r / (ntiles - 1));
    nj = 1 + (int)(r % (ntiles - 1));
  }
}

// The last query tile from which key tile nj of row n gets anything: ntiles - 1, or with a table of live tiles
// (alive[n][mi][nj], sa_tc_skip.cu) the largest live mi; the diagonal tile is always live.  One warp.
__device__ __forceinline__ void find_top_tile(const uint8_t* alive, int n, int nj, int ntiles, int lane, int* top) {
  int found = ntiles - 1;
  if (alive != nullptr) {
    const uint8_t* col = alive + (int64_t)n * ntiles * ntiles + nj;
    found = nj;
    for (int base = ntiles - 1; base >= nj; base -= 32) {
      const int mi = base - lane;
      const bool f = mi >= nj && col[(int64_t)mi * ntiles] != 0;
      const unsigned m = __ballot_sync(0xffffffffu, f);
      if (m != 0) {
        found = base - (__ffs(m) - 1);
        break;
      }
    }
  }
  if (lane == 0) *top = found;
}

// TMEM columns of the three score-shaped tiles (the same in both kernels)
constexpr uint32_t kColZ = 256, kColX = 320, kColY = 384;

__device__ __forceinline__ void put_words(uint8_t* base, int row, int c0, const uint32_t* w) {
  *reinterpret_cast<uint4*>(base + (c0 >> 6) * kRowTile + swz_off(row, (c0 & 63) >> 3)) = make_uint4(w[0], w[1], w[2], w[3]);
}

struct HalfState {
  float gate[16];      // 1 where the (query, key) pair is selected, else 0
  float lx[16];        // NEGATED exclusive suffix sums of dz inside this thread's chunk (the g pass wants -U)
  float dz[16];        // one head per selector only: dz, which the g pass adds to g before the products
};

struct Ctx {
  uint8_t* dz_tile;    // [128 keys][128 queries] bf16 as two query-half tiles: dz (one head per selector: dz + g)
  uint8_t* g_tile;     // the same shape for g
  uint32_t tmem, lane_base;
  int row, wg;
  bool selectable;
  float c1;
  const float* lse_s;
  const float* dbar_s;
  float (*sel_tot)[kTile];
  float (*dz_tot)[kTile];
  WaitCtx status;
};

// First part of a half: selection pass, probabilities, dz.  Leaves P^T and dz^T in this thread's columns of Y (bf16
// pairs), the dz half tile in shared memory, and returns what the g pass needs.
// `keep_dz`: whether the dz half tile is also needed in shared memory (an MMA of this CTA reads it from there).
template <bool DIAG, bool SELF>
__device__ __forceinline__ void half_scores(const Ctx& c, int hf, uint32_t phase, float cnl, float& sel_state,
                                            HalfState& st, uint64_t* bar_l0, uint64_t* bar_sel, uint64_t* bar_s,
                                            uint64_t* bar_dp, uint64_t* bar_early, bool drain_reduce, bool keep_dz) {
  const int colw = c.wg * kChunk;
  const int col0 = hf * 64 + colw;
  uint32_t r[16];
  float ls[16], p[16];

  if (SELF) {                                               // the selection logits are the head's own: S^T serves both
    mbar_wait(bar_s, phase, c.status, 416);
    tc_fence_after_sync();
    tmem_ld16(c.lane_base + kColY + colw, r);
  } else {
    mbar_wait(bar_l0, phase, c.status, 410);
    tc_fence_after_sync();
    tmem_ld16(c.lane_base + kColZ + colw, r);               // L0^T
  }
  tmem_ld_wait();
#pragma unroll
  for (int e = 0; e < 16; ++e) {                            // the gate as 1 / 0: one compare-and-set per element ...
    const float l0 = __uint_as_float(r[e]);
    bool on = c.selectable && (l0 > 0.f);
    if (DIAG) on = on && (c.row < col0 + e);                // key strictly before the query
    st.gate[e] = on ? 1.f : 0.f;
  }
#pragma unroll
  for (int e = 0; e < 16; e += 2) {                         // ... and the selected logits as a packed product
    const float2 v = __fmul2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])),
                                make_float2(st.gate[e], st.gate[e + 1]));
    ls[e] = v.x; ls[e + 1] = v.y;
  }
#pragma unroll
  for (int e = 6; e >= 0; --e) {                            // inclusive suffix sums, two chains
    ls[e] += ls[e + 1];
    ls[e + 8] += ls[e + 9];
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) ls[e] += ls[8];
  c.sel_tot[c.wg][c.row] = ls[0];
  tc_fence_before_sync();
  named_barrier(kComputeBarrier, kComputeThreads);          // every thread has read L0^T
  if (!SELF && threadIdx.x == 0) mbar_arrive(bar_sel);      // Z may now receive the next half's L0^T
  float later = 0.f, all = 0.f;
#pragma unroll
  for (int w = 0; w < kGroups; ++w) {
    const float t = c.sel_tot[w][c.row];
    all += t;
    if (w > c.wg) later += t;
  }
  // F * log2e = cnl - c1 * (sel_state + later + ls[e]);   z = S * c1 - F * log2e - lse
  const float cb = cnl - c.c1 * (sel_state + later);
  sel_state += all;

  if (!SELF) {
    mbar_wait(bar_s, phase, c.status, 416);
    tc_fence_after_sync();
    tmem_ld16(c.lane_base + kColY + colw, r);               // S^T
    tmem_ld_wait();
  }
  const float2 cc = make_float2(c.c1, c.c1);
  const float2 ncb = make_float2(-cb, -cb);
#pragma unroll
  for (int e4 = 0; e4 < 16; e4 += 4) {
    const float4 st4 = *reinterpret_cast<const float4*>(c.lse_s + col0 + e4);
    const float2 sv[2] = {make_float2(st4.x, st4.y), make_float2(st4.z, st4.w)};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = e4 + 2 * k;
      const float2 t2 = __ffma2_rn(cc, make_float2(ls[e], ls[e + 1]), __fadd2_rn(sv[k], ncb));     // c1 ls - (cb + lse)
      const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), cc, t2);
      p[e] = ex2(x.x);
      p[e + 1] = ex2(x.y);
      if (DIAG) {                                           // key after the query
        if (c.row > col0 + e) p[e] = 0.f;
        if (c.row > col0 + e + 1) p[e + 1] = 0.f;
      }
    }
  }
  {                                                         // P^T as bf16 pairs over the first half of this thread's S^T
    uint32_t w8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w8[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
    tmem_st8(c.lane_base + kColY + colw, w8);
  }

  mbar_wait(bar_dp, phase, c.status, 411);
  tc_fence_after_sync();
  tmem_ld16(c.lane_base + kColX + colw, r);                 // dP^T
  tmem_ld_wait();
#pragma unroll
  for (int e4 = 0; e4 < 16; e4 += 4) {
    const float4 st4 = *reinterpret_cast<const float4*>(c.dbar_s + col0 + e4);
    const float2 d0 = __fmul2_rn(make_float2(p[e4], p[e4 + 1]),                                   // dz = P (dP - dbar)
                                 __fadd2_rn(make_float2(__uint_as_float(r[e4]), __uint_as_float(r[e4 + 1])),
                                            make_float2(st4.x, st4.y)));
    const float2 d1 = __fmul2_rn(make_float2(p[e4 + 2], p[e4 + 3]),
                                 __fadd2_rn(make_float2(__uint_as_float(r[e4 + 2]), __uint_as_float(r[e4 + 3])),
                                            make_float2(st4.z, st4.w)));
    p[e4] = d0.x; p[e4 + 1] = d0.y; p[e4 + 2] = d1.x; p[e4 + 3] = d1.y;
  }
  if (SELF) {                                               // dz + g leaves in the g pass
#pragma unroll
    for (int e = 0; e < 16; ++e) st.dz[e] = p[e];
  } else {                                                  // dz: bf16 once, to TMEM (A of dK) and shared memory (A of dQ)
    uint32_t w8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w8[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
    tmem_st8(c.lane_base + kColY + colw + 8, w8);           //   over the second half of this thread's S^T
    if (keep_dz) {
      put_words(c.dz_tile, c.row, col0, w8);
      put_words(c.dz_tile, c.row, col0 + 8, w8 + 4);
    }
  }

  st.lx[15] = 0.f;                                          // NEGATED exclusive suffix sums of dz, two chains
  st.lx[7] = 0.f;
#pragma unroll
  for (int e = 6; e >= 0; --e) {
    st.lx[e] = st.lx[e + 1] - p[e + 1];
    st.lx[e + 8] = st.lx[e + 9] - p[e + 9];
  }
  const float tot_hi = st.lx[8] - p[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) st.lx[e] += tot_hi;
  c.dz_tot[c.wg][c.row] = p[0] - st.lx[0];
  fence_async_smem();                                       // dz half tile -> visible to the MMAs
  tmem_st_wait();                                           // P^T and dz^T in TMEM
  tc_fence_before_sync();
  if (drain_reduce && threadIdx.x == 0) bulk_wait_read();   // the staging tile's last reduce-add has read it
  named_barrier(kComputeBarrier, kComputeThreads);          // every thread is done with S^T and dP^T
  if (threadIdx.x == 0) mbar_arrive(bar_early);
}

// Second part of a half: g = gate ? -(sum of dz over later queries, all in this head) : 0 into shared memory.
// `keep`: whether the g (one head per selector: dz + g) half tile is also needed in shared memory.
template <bool SELF>
__device__ __forceinline__ void half_gate(const Ctx& c, int hf, float& dz_state, HalfState& st, bool keep) {
  const int col0 = hf * 64 + c.wg * kChunk;
  float later = 0.f, all = 0.f;
#pragma unroll
  for (int w = 0; w < kGroups; ++w) {
    const float t = c.dz_tot[w][c.row];
    all += t;
    if (w > c.wg) later += t;
  }
  const float base = dz_state + later;
  dz_state += all;
  const float2 bb = make_float2(-base, -base);                   // lx holds negated sums: gate * (-(sum + base))
#pragma unroll
  for (int e = 0; e < 16; e += 2) {
    float2 x;
    if (SELF)                                                    // dz + g: Q0 = Q and K0 = K, so the two gradient paths add
      x = __ffma2_rn(make_float2(st.gate[e], st.gate[e + 1]), __fadd2_rn(make_float2(st.lx[e], st.lx[e + 1]), bb),
                     make_float2(st.dz[e], st.dz[e + 1]));
    else
      x = __fmul2_rn(make_float2(st.gate[e], st.gate[e + 1]), __fadd2_rn(make_float2(st.lx[e], st.lx[e + 1]), bb));
    st.lx[e] = x.x; st.lx[e + 1] = x.y;
  }
  uint32_t w8[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) w8[e] = pack_bf16(st.lx[2 * e], st.lx[2 * e + 1]);
  tmem_st8(c.lane_base + kColX + c.wg * kChunk, w8);             // g^T (or (dz + g)^T) over this thread's dP^T columns
  if (keep) {                                                    // g: operand of dQ0 (dz + g: operand of dQ)
    put_words(SELF ? c.dz_tile : c.g_tile, c.row, col0, w8);
    put_words(SELF ? c.dz_tile : c.g_tile, c.row, col0 + 8, w8 + 4);
  }
  tmem_st_wait();
}

}  // namespace bwd
}  // namespace tc
}  // namespace sa
