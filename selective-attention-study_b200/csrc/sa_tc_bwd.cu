// Tensor-core engine, backward (sm_100a: TMA loads and reduce-adds, tcgen05 MMAs, fp32 accumulators in TMEM).
//
// One CTA owns one 128-key tile of one head and walks the 128-query tiles LAST TO FIRST.  All
// score-shaped tiles are computed transposed, KEYS on the TMEM lanes: S^T = K Q^T, dP^T = V dO^T,
// L0^T = K0 Q0^T, so one thread owns one key and sees that key's queries along its registers.  The
// two running sums down the query axis are then thread-local fp32 recurrences walked from the last
// query to the first:
//     F[i]  = carry_after_tile - sum_{r >= i} sel[r]          (history term rebuilt per key)
//     U[i]  = suffix + sum_{i' > i} dz[i']                      (logit gradient of later queries)
// with  P = exp2(z - lse),  dz = P (dP - dbar),  g = gate ? -U : 0.
//
// Roles.  Warps 0-15 (four warpgroups) do the arithmetic: a query tile is handled as two 64-query
// halves, and within a half each warpgroup takes 16 query columns of every key row; chunk totals are
// exchanged through shared memory so the recurrences chain across chunks, halves and tiles.  Warp 16 is
// the control warp: one lane issues every TMA load and every MMA, so MMA issue never stalls arithmetic.
//
// Products per query tile (all on tcgen05, fp32 accumulation in TMEM):
//     per half : S^T, dP^T, L0^T (N = 64);  dV += P^T dO with P^T read from TMEM as bf16;
//                dK += dz^T Q;  dK0 += g^T Q0
//     per tile : dQ = dz K;  dQ0 = g K0  (dz, g read from shared memory M-major) -> scaled, staged in
//                shared memory and added to the fp32 global accumulators with TMA reduce-add.
//
// SELF variant (one head per selector, i.e. the per-head form reshaped to (B H, 1, T, D)): the selection logits
// are the head's own logits, so L0^T is S^T, and since Q0 = Q and K0 = K the two gradient paths add before the
// MMAs: dK += (dz + g)^T Q and dQ = (dz + g) K.  40 MMAs per query tile instead of 64, no Q0 / K0 tiles, one
// read-out per tile.
//
// Only the SELF variant is launched from this file.  A selector shared by several heads (or given separately) runs
// backward_shared_kernel (sa_tc_bwd_shared.cu), which keeps this kernel's arithmetic and changes where the MMA
// operands live and when the products are issued; the !SELF branches below are that kernel's starting point.
// Reference for the arithmetic: src/selective_attention/kernels.py:196-268.
#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {
namespace {

constexpr int kTile = 128;
constexpr int kRowTile = 16384;     // bytes of a [128][64] bf16 operand tile
constexpr int kGroups = 4;          // arithmetic warpgroups; each owns 16 of a half's 64 query columns
constexpr int kChunk = 64 / kGroups;
constexpr int kComputeThreads = 128 * kGroups;
constexpr int kThreads = kComputeThreads + 32;
constexpr int kComputeBarrier = 1;  // hardware barrier id of the arithmetic warps

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A global load the compiler must issue where it is written (volatile asm keeps its place among the other
// volatile asm statements), so a value fetched one tile ahead is really in flight during that tile.
__device__ __forceinline__ float load_ahead(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

struct BwdSmem {
  static constexpr int k = 0;                       // [128 keys][64], stationary
  static constexpr int v = k + kRowTile;
  static constexpr int k0 = v + kRowTile;
  static constexpr int stage = k0 + kRowTile;       // 2 stages x (Q, Q0, dO) tiles [128 queries][64]
  static constexpr int dz = stage + 6 * kRowTile;   // [128 keys][128 queries] bf16 as two query-half tiles;
  static constexpr int g = dz + 2 * kRowTile;       //   after the tile's MMAs: fp32 staging of dQ / dQ0
  static constexpr int total = g + 2 * kRowTile;
};

// TMEM columns.  L0T doubles as the home of P^T (bf16 pairs, 32 columns) once L0^T has been read.
constexpr uint32_t kColST = 0, kColDPT = 64, kColL0T = 128, kColDV = 192, kColDK = 256, kColDK0 = 320, kColDQ = 384,
                   kColDQ0 = 448;

// Writes 8 consecutive bf16 (query columns c0 .. c0 + 7 of key row `row`) of a [128][128] matrix kept
// as two 64-column tiles.
__device__ __forceinline__ void put8(uint8_t* base, int row, int c0, const float* x) {
  uint4 w = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
  *reinterpret_cast<uint4*>(base + (c0 >> 6) * kRowTile + swz_off(row, (c0 & 63) >> 3)) = w;
}

struct HalfCtx {
  uint8_t* smem;
  uint32_t lane_base;
  int row;                 // key row of this thread inside the tile (its TMEM lane)
  int wg;                  // warpgroup: which 16-column chunk of the half
  int hf;                  // which half of the query tile
  bool selectable;         // key >= exempt
  float cnl;               // log2(e) * selection received through the END of this query tile
  float c1;                // scale * log2(e)
  const float* lse_s;      // -lse2 of the tile's queries (padded queries: -inf)
  const float* dbar_s;     // -dbar
  float (*sel_tot)[kTile];
  float (*dz_tot)[kTile];
  uint64_t* bar_early;     // arrived once per half when P^T and dz are in place and the score columns are free
  bool drain_reduce;       // first half of a tile: the previous tile's reduce-adds still read the dz / g buffers
};

// One 64-query half of a (key tile, query tile) pair; this thread handles 16 of its query columns for
// its key row.  The two running sums run from the last query to the first; a chunk computes them
// locally (two independent chains of 8) and picks up the totals of the chunks to its right, and the
// carried state, through shared memory.
template <bool DIAG, bool SELF>
__device__ __forceinline__ void process_half(const HalfCtx& c, float& sel_state, float& dz_state) {
  using L = BwdSmem;
  const int colw = c.wg * kChunk;
  const int col0 = c.hf * 64 + colw;
  uint32_t r[16];
  float negon[16], ls[16], p[16], lx[16];

  tmem_ld16(c.lane_base + (SELF ? kColST : kColL0T) + colw, r);
  tmem_ld_wait();
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const float l0 = __uint_as_float(r[e]);
    bool on = c.selectable && (l0 > 0.f);
    if (DIAG) on = on && (c.row < col0 + e);          // key strictly before the query
    negon[e] = on ? -1.f : 0.f;
    ls[e] = on ? l0 : 0.f;
  }
#pragma unroll
  for (int e = 6; e >= 0; --e) {                        // inclusive suffix sums, two chains
    ls[e] += ls[e + 1];
    ls[e + 8] += ls[e + 9];
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) ls[e] += ls[8];
  c.sel_tot[c.wg][c.row] = ls[0];
  tc_fence_before_sync();
  if (c.drain_reduce && threadIdx.x == 0) bulk_wait_read();
  named_barrier(kComputeBarrier, kComputeThreads);      // also: every thread has finished reading L0^T
  tc_fence_after_sync();
  float later = 0.f, all = 0.f;
#pragma unroll
  for (int w = 0; w < kGroups; ++w) {
    const float t = c.sel_tot[w][c.row];
    all += t;
    if (w > c.wg) later += t;
  }
  // F * log2e = cnl - c1 * (sel_state + later + ls[e]);   z = S * c1 - F * log2e - lse
  const float cb = c.cnl - c.c1 * (sel_state + later);
  sel_state += all;

  tmem_ld16(c.lane_base + kColST + colw, r);
  tmem_ld_wait();
  // Packed fp32x2 arithmetic (two results per issue slot) for the elementwise parts.
  const float2 cc = make_float2(c.c1, c.c1);
  const float2 ncb = make_float2(-cb, -cb);
#pragma unroll
  for (int e4 = 0; e4 < 16; e4 += 4) {                  // row statistics: one 16-byte broadcast load per 4 queries
    const float4 st4 = *reinterpret_cast<const float4*>(c.lse_s + col0 + e4);
    const float2 st[2] = {make_float2(st4.x, st4.y), make_float2(st4.z, st4.w)};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = e4 + 2 * k;
      const float2 t2 = __ffma2_rn(cc, make_float2(ls[e], ls[e + 1]), __fadd2_rn(st[k], ncb));     // c1 ls - (cb + lse)
      const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), cc, t2);
      p[e] = ex2(x.x);
      p[e + 1] = ex2(x.y);
      if (DIAG) {                                       // key after the query
        if (c.row > col0 + e) p[e] = 0.f;
        if (c.row > col0 + e + 1) p[e + 1] = 0.f;
      }
    }
  }
  {                                                     // P^T as bf16 pairs into the (consumed) L0^T columns
    uint32_t w8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w8[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
    tmem_st8(c.lane_base + kColL0T + (colw >> 1), w8);
  }

  tmem_ld16(c.lane_base + kColDPT + colw, r);
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
  if (!SELF) {
    put8(c.smem + L::dz, c.row, col0, p);
    put8(c.smem + L::dz, c.row, col0 + 8, p + 8);
  }

  lx[15] = 0.f;                                          // exclusive suffix sums of dz, two chains
  lx[7] = 0.f;
#pragma unroll
  for (int e = 6; e >= 0; --e) {
    lx[e] = lx[e + 1] + p[e + 1];
    lx[e + 8] = lx[e + 9] + p[e + 9];
  }
  const float tot_hi = lx[8] + p[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) lx[e] += tot_hi;
  c.dz_tot[c.wg][c.row] = lx[0] + p[0];
  fence_async_smem();                                    // dz tile half -> visible to the MMAs
  tmem_st_wait();                                        // P^T in TMEM
  tc_fence_before_sync();
  named_barrier(kComputeBarrier, kComputeThreads);      // every thread is done with S^T, dP^T and L0^T
  if (threadIdx.x == 0) mbar_arrive(c.bar_early);
  later = 0.f;
  all = 0.f;
#pragma unroll
  for (int w = 0; w < kGroups; ++w) {
    const float t = c.dz_tot[w][c.row];
    all += t;
    if (w > c.wg) later += t;
  }
  const float base = dz_state + later;
  dz_state += all;
  const float2 bb = make_float2(base, base);
  if (SELF) {
#pragma unroll
    for (int e = 0; e < 16; e += 2) {                                                              // dz + g
      const float2 x = __ffma2_rn(make_float2(negon[e], negon[e + 1]), __fadd2_rn(make_float2(lx[e], lx[e + 1]), bb),
                                  make_float2(p[e], p[e + 1]));
      lx[e] = x.x; lx[e + 1] = x.y;
    }
    put8(c.smem + L::dz, c.row, col0, lx);
    put8(c.smem + L::dz, c.row, col0 + 8, lx + 8);
  } else {
#pragma unroll
    for (int e = 0; e < 16; e += 2) {                                                              // g
      const float2 x = __fmul2_rn(make_float2(negon[e], negon[e + 1]), __fadd2_rn(make_float2(lx[e], lx[e + 1]), bb));
      lx[e] = x.x; lx[e + 1] = x.y;
    }
    put8(c.smem + L::g, c.row, col0, lx);
    put8(c.smem + L::g, c.row, col0 + 8, lx + 8);
  }
}

template <bool SELF>
__global__ void __launch_bounds__(kThreads, 1) backward_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ CUtensorMap map_dq0,
    const __grid_constant__ CUtensorMap map_q0, const __grid_constant__ CUtensorMap map_k0,
    const float* __restrict__ lse2, const float* __restrict__ carry, const float* __restrict__ dbar,
    float* __restrict__ dk_acc, float* __restrict__ dk0, __nv_bfloat16* __restrict__ dv, int heads, int seq,
    int ntiles, int exempt, float scale, WaitCtx status, RowLayout dv_rows) {
  using L = BwdSmem;
  constexpr int D = 64;
  const int nrows = gridDim.x / ntiles;                  // batch * heads
  const int nj = (int)(blockIdx.x / nrows);              // key tiles with the most query tiles first
  const int n = blockIdx.x % nrows;
  const int b = n / heads, h = n - b * heads;
  const int n_iter = ntiles - nj;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_kv, bar_ld[2], bar_a, bar_b, bar_dq, bar_half[2], bar_early;
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float lse_s[kTile];
  __shared__ __align__(16) float dbar_s[kTile];
  __shared__ float sel_tot[kGroups][kTile];
  __shared__ float dz_tot[kGroups][kTile];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&bar_kv, 1);
    mbar_init(&bar_ld[0], 1);
    mbar_init(&bar_ld[1], 1);
    mbar_init(&bar_a, 1);
    mbar_init(&bar_b, 1);
    mbar_init(&bar_dq, 1);
    // bar_half: one per half, each used once per tile, so the waiter can never see one complete two phases between
    // two of its polls.  bar_early needs no such split: each arrival needs scores that are issued after the
    // previous arrival was observed.
    mbar_init(&bar_half[0], kComputeThreads / 32);
    mbar_init(&bar_half[1], kComputeThreads / 32);
    mbar_init(&bar_early, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t sa = smem_u32(smem);

  if (warp == kComputeThreads / 32) {
    // =============================== control warp: TMA loads and MMA issue ===============================
    if (lane == 0) {
      const uint32_t idesc_t = instr_desc_bf16(128, 64, false, false);     // keys x 64 queries, K = D
      const uint32_t idesc_acc = instr_desc_bf16(128, 64, false, true);    // A K-major (keys x queries), B MN-major
      const uint32_t idesc_dq = instr_desc_bf16(128, 64, true, true);      // A MN-major (queries x keys), B MN-major
      auto load_stage = [&](int it) {
        const int mi = ntiles - 1 - it;
        uint8_t* st = smem + L::stage + (it & 1) * 3 * kRowTile;
        mbar_expect_tx(&bar_ld[it & 1], (SELF ? 2 : 3) * kRowTile);
        tma_load_4d(st, &map_q, &bar_ld[it & 1], 0, mi * kTile, h, b);
        if (!SELF) tma_load_4d(st + kRowTile, &map_q0, &bar_ld[it & 1], 0, mi * kTile, 0, b);
        tma_load_4d(st + 2 * kRowTile, &map_do, &bar_ld[it & 1], 0, mi * kTile, n, 0);
      };
      // Operand descriptors are built once; an MMA's descriptor is a base plus a byte offset / 16, so the
      // issuing thread spends a couple of integer adds per MMA instead of rebuilding 64-bit descriptors.
      auto at = [](uint64_t desc, uint32_t byte_off) { return desc + (uint64_t)(byte_off >> 4); };
      const uint64_t kK = smem_desc(sa + L::k, 16, 1024), kV = smem_desc(sa + L::v, 16, 1024),
                     kK0 = smem_desc(sa + L::k0, 16, 1024);                                   // K-major A (scores)
      const uint64_t mK = smem_desc(sa + L::k, kRowTile, 1024), mK0 = smem_desc(sa + L::k0, kRowTile, 1024);
      const uint64_t kDZ = smem_desc(sa + L::dz, 16, 1024), kG = smem_desc(sa + L::g, 16, 1024);   // K-major A
      const uint64_t mDZ = smem_desc(sa + L::dz, kRowTile, 1024), mG = smem_desc(sa + L::g, kRowTile, 1024);
      const uint64_t kStage = smem_desc(sa + L::stage, 16, 1024);            // Q, Q0, dO of stage 0, K-major B
      const uint64_t mStage = smem_desc(sa + L::stage, kRowTile, 1024);      // the same tiles as "K rows" operands
      // S^T, dP^T, L0^T of one 64-query half
      auto issue_scores = [&](int it, int hf) {
        const uint32_t st = (it & 1) * 3 * kRowTile + hf * 8192;                   // rows 64 hf .. 64 hf + 63
        if (!SELF) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tmem + kColL0T, at(kK0, ks * 32), at(kStage, st + kRowTile + ks * 32), idesc_t, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColST, at(kK, ks * 32), at(kStage, st + ks * 32), idesc_t, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColDPT, at(kV, ks * 32), at(kStage, st + 2 * kRowTile + ks * 32), idesc_t, ks > 0);
        mma_commit(&bar_a);
      };
      // dV += P^T dO over the half's 64 queries, P^T from TMEM
      auto issue_dv = [&](int it, int hf, bool first) {
        const uint32_t st = (it & 1) * 3 * kRowTile + hf * 8192;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDV, tmem + kColL0T + ks * 8, at(mStage, st + 2 * kRowTile + ks * 2048), idesc_acc,
                 (first && ks == 0) ? 0u : 1u);
      };
      // dK += dz^T Q and dK0 += g^T Q0 over the half's 64 queries
      auto issue_dk_only = [&](int it, int hf, bool first) {
        const uint32_t st = (it & 1) * 3 * kRowTile + hf * 8192;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColDK, at(kDZ, hf * kRowTile + ks * 32), at(mStage, st + ks * 2048), idesc_acc,
                 (first && ks == 0) ? 0u : 1u);
      };
      auto issue_dk0_only = [&](int it, int hf, bool first) {
        const uint32_t st = (it & 1) * 3 * kRowTile + hf * 8192;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColDK0, at(kG, hf * kRowTile + ks * 32), at(mStage, st + kRowTile + ks * 2048), idesc_acc,
                 (first && ks == 0) ? 0u : 1u);
      };

      mbar_expect_tx(&bar_kv, (SELF ? 2 : 3) * kRowTile);
      tma_load_4d(smem + L::k, &map_k, &bar_kv, 0, nj * kTile, h, b);
      tma_load_4d(smem + L::v, &map_v, &bar_kv, 0, nj * kTile, h, b);
      if (!SELF) tma_load_4d(smem + L::k0, &map_k0, &bar_kv, 0, nj * kTile, 0, b);
      load_stage(0);
      if (n_iter > 1) load_stage(1);
      mbar_wait(&bar_kv, 0, status, 400);
      mbar_wait(&bar_ld[0], 0, status, 401);
      tc_fence_after_sync();
      issue_scores(0, 1);

      uint32_t early_phase = 0;
      for (int it = 0; it < n_iter; ++it) {
        // half 1: P^T and dz are ready and the score columns are free while the g pass still runs
        const uint32_t ph = it & 1;
        mbar_wait(&bar_early, early_phase, status, 402);
        early_phase ^= 1;
        tc_fence_after_sync();
        issue_dv(it, 1, it == 0);                             // reads P^T before the next scores overwrite it
        issue_scores(it, 0);
        if (!SELF) issue_dk_only(it, 1, it == 0);
        mbar_wait(&bar_half[1], ph, status, 403);            // half 1: g (SELF: dz + g) written
        tc_fence_after_sync();
        if (SELF) issue_dk_only(it, 1, it == 0);
        else issue_dk0_only(it, 1, it == 0);
        // half 0
        mbar_wait(&bar_early, early_phase, status, 406);
        early_phase ^= 1;
        tc_fence_after_sync();
        if (SELF) {
          issue_dv(it, 0, false);
          if (it + 1 < n_iter) {                              // nothing else can run until the g pass ends
            mbar_wait(&bar_ld[(it + 1) & 1], ((it + 1) >> 1) & 1, status, 404);
            tc_fence_after_sync();
            issue_scores(it + 1, 1);
          }
          mbar_wait(&bar_half[0], ph, status, 407);          // half 0: dz + g written
          tc_fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)                      // dQ = (dz + g) K: A M-major, K = key index
            mma_ss(tmem + kColDQ, at(mDZ, ks * 2048), at(mK, ks * 2048), idesc_dq, ks > 0);
          issue_dk_only(it, 0, false);
          mma_commit(&bar_dq);
          mma_commit(&bar_b);
        } else {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)                      // dQ = dz K: A M-major, K = key index
            mma_ss(tmem + kColDQ, at(mDZ, ks * 2048), at(mK, ks * 2048), idesc_dq, ks > 0);
          issue_dk_only(it, 0, false);
          mma_commit(&bar_dq);                                // dQ done and every MMA reading the dz tiles is done:
          issue_dv(it, 0, false);                             //   its read-out overlaps the MMAs from here on
          mbar_wait(&bar_half[0], ph, status, 407);          // half 0: g written
          tc_fence_after_sync();
          issue_dk0_only(it, 0, false);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)                      // dQ0 = g K0
            mma_ss(tmem + kColDQ0, at(mG, ks * 2048), at(mK0, ks * 2048), idesc_dq, ks > 0);
          mma_commit(&bar_b);
          if (it + 1 < n_iter) {
            mbar_wait(&bar_ld[(it + 1) & 1], ((it + 1) >> 1) & 1, status, 404);
            tc_fence_after_sync();
            issue_scores(it + 1, 1);
          }
        }
        mbar_wait(&bar_b, it & 1, status, 405);               // every MMA reading stage (it & 1) has completed
        if (it + 2 < n_iter) load_stage(it + 2);
      }
    }
    __syncwarp();
  } else {
    // ======================================= arithmetic warps ============================================
    const int row = tid & 127, wg = tid >> 7;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // a warp reaches lanes 32 (warp % 4) ..
    const int j = nj * kTile + row;
    float dz_state = 0.f;            // sum of dz over the queries already visited (later queries), this key
    uint32_t a_phase = 0;

    HalfCtx ctx;
    ctx.smem = smem;
    ctx.lane_base = lane_base;
    ctx.row = row;
    ctx.wg = wg;
    ctx.selectable = (j >= exempt);
    ctx.c1 = scale * kLog2e;
    ctx.lse_s = lse_s;
    ctx.dbar_s = dbar_s;
    ctx.sel_tot = sel_tot;
    ctx.dz_tot = dz_tot;
    ctx.bar_early = &bar_early;

    // per-tile row statistics and carry, fetched one tile ahead
    auto fetch_lse = [&](int mi) {
      const int i = mi * kTile + tid;
      return (tid < kTile && i < seq) ? load_ahead(lse2 + (int64_t)n * seq + i) : INFINITY;   // +inf: P = 0 for padded queries
    };
    auto fetch_dbar = [&](int mi) {
      const int i = mi * kTile + tid;
      return (tid < kTile && i < seq) ? load_ahead(dbar + (int64_t)n * seq + i) : 0.f;
    };
    auto fetch_carry = [&](int mi) {
      return (j < seq) ? load_ahead(carry + ((int64_t)b * (ntiles + 1) + mi + 1) * seq + j) : 0.f;
    };
    float next_lse = fetch_lse(ntiles - 1), next_dbar = fetch_dbar(ntiles - 1), next_carry = fetch_carry(ntiles - 1);

    for (int it = 0; it < n_iter; ++it) {
      const int mi = ntiles - 1 - it;
      const int i0 = mi * kTile;
      const bool diag = (mi == nj);
      if (tid < kTile) {
        lse_s[tid] = -next_lse;                                // negated: both enter packed adds directly
        dbar_s[tid] = -next_dbar;
      }
      ctx.cnl = next_carry * kLog2e;
      if (it + 1 < n_iter) {
        next_lse = fetch_lse(mi - 1);
        next_dbar = fetch_dbar(mi - 1);
        next_carry = fetch_carry(mi - 1);
      }
      float sel_state = 0.f;         // selection of the tile's queries already visited, this key (raw logit units)

#pragma unroll 1
      for (int hf = 1; hf >= 0; --hf) {
        mbar_wait(&bar_a, a_phase, status, 410);
        a_phase ^= 1;
        tc_fence_after_sync();
        ctx.hf = hf;
        ctx.drain_reduce = (hf == 1) && (it > 0);
        if (diag) process_half<true, SELF>(ctx, sel_state, dz_state);
        else process_half<false, SELF>(ctx, sel_state, dz_state);
        fence_async_smem();                                    // g tile half -> visible to the MMAs
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_half[hf]);
      }

      // ---- dQ, then dQ0, of this query tile: TMEM -> scaled fp32 staging in shared memory (the dz / g tiles,
      // which no MMA reads any more) -> TMA reduce-add.  dQ is staged while the dK0 / dQ0 MMAs still run.
      auto stage_tile = [&](uint32_t col, uint8_t* dst) {
        const int c0 = wg * kChunk;                           // here the lane is a QUERY row, columns are d
        uint32_t r[16];
        tmem_ld16(lane_base + col + c0, r);
        tmem_ld_wait();
        uint8_t* sq = dst + (wg >> 1) * kRowTile;             // [128 queries][32 floats] tiles, 128-byte swizzle
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<float4*>(sq + swz_off(row, (wg & 1) * 4 + c)) =
              make_float4(__uint_as_float(r[4 * c]) * scale, __uint_as_float(r[4 * c + 1]) * scale,
                          __uint_as_float(r[4 * c + 2]) * scale, __uint_as_float(r[4 * c + 3]) * scale);
        fence_async_smem();
        tc_fence_before_sync();
        named_barrier(kComputeBarrier, kComputeThreads);
      };
      mbar_wait(&bar_dq, it & 1, status, 412);
      tc_fence_after_sync();
      stage_tile(kColDQ, smem + L::dz);
      if (tid == 0) {
        tma_reduce_add_4d(&map_dq, smem + L::dz, 0, i0, n, 0);
        tma_reduce_add_4d(&map_dq, smem + L::dz + kRowTile, 32, i0, n, 0);
        bulk_commit();
      }
      if (SELF) continue;                                      // dQ already carries the selection path
      mbar_wait(&bar_b, it & 1, status, 411);
      tc_fence_after_sync();
      stage_tile(kColDQ0, smem + L::g);
      if (tid == 0) {
        tma_reduce_add_4d(&map_dq0, smem + L::g, 0, i0, b, 0);
        tma_reduce_add_4d(&map_dq0, smem + L::g + kRowTile, 32, i0, b, 0);
        bulk_commit();
      }
    }

    // ---- epilogue: dV, dK (this head) and this head's share of dK0 ------------------------------------------
    {
      const int c0 = wg * kChunk;
      __nv_bfloat16* dv_row = dv + dv_rows.at(b, h, j) + c0;
      float* dk_row = dk_acc + ((int64_t)n * seq + j) * D + c0;
      float* dk0_row = dk0 + ((int64_t)b * seq + j) * D + c0;
      uint32_t rv[16], rk[16], r0[16];
      tmem_ld16(lane_base + kColDV + c0, rv);
      tmem_ld16(lane_base + kColDK + c0, rk);
      if (!SELF) tmem_ld16(lane_base + kColDK0 + c0, r0);
      tmem_ld_wait();
      if (j < seq) {
#pragma unroll
        for (int e = 0; e < 16; e += 8) {
          uint4 w = make_uint4(pack_bf16(__uint_as_float(rv[e]), __uint_as_float(rv[e + 1])),
                               pack_bf16(__uint_as_float(rv[e + 2]), __uint_as_float(rv[e + 3])),
                               pack_bf16(__uint_as_float(rv[e + 4]), __uint_as_float(rv[e + 5])),
                               pack_bf16(__uint_as_float(rv[e + 6]), __uint_as_float(rv[e + 7])));
          *reinterpret_cast<uint4*>(dv_row + e) = w;
        }
#pragma unroll
        for (int e = 0; e < 16; e += 4) {
          *reinterpret_cast<float4*>(dk_row + e) =
              make_float4(__uint_as_float(rk[e]) * scale, __uint_as_float(rk[e + 1]) * scale,
                          __uint_as_float(rk[e + 2]) * scale, __uint_as_float(rk[e + 3]) * scale);
          if (!SELF)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dk0_row + e),
                         "f"(__uint_as_float(r0[e]) * scale), "f"(__uint_as_float(r0[e + 1]) * scale),
                         "f"(__uint_as_float(r0[e + 2]) * scale), "f"(__uint_as_float(r0[e + 3]) * scale)
                         : "memory");
        }
      }
    }
    if (tid == 0) bulk_wait_all();                            // the last reduce-adds must land before the CTA exits
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

int backward_shared(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_bf16,
                    float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s);

int backward(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_bf16,
             float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  if (p.head_dim != 64) return SA_ERR_UNSUPPORTED;
  // A selector shared by several heads (or given separately) has its own kernel (sa_tc_bwd_shared.cu); the kernel of
  // this file runs the one-head-per-selector form.
  const bool self = (p.heads == 1) && !p.external_selector;
  if (!self) return backward_shared(p, lse2, carry, dbar, d_out_bf16, dq_acc, dk_acc, dq0, dk0, dv, s);
  const int ntiles = (p.seq + kTile - 1) / kTile;
  const int nrows = p.batch * p.heads;
  CUtensorMap map_q, map_k, map_v, map_do, map_dq, map_dq0;
  int st = make_map_16bit(&map_q, p.q.ptr, 64, p.seq, p.heads, p.batch, p.q.st, p.q.sh, p.q.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k, p.k.ptr, 64, p.seq, p.heads, p.batch, p.k.st, p.k.sh, p.k.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_v, p.v.ptr, 64, p.seq, p.heads, p.batch, p.v.st, p.v.sh, p.v.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_do, d_out_bf16, 64, p.seq, nrows, 1, 64, (int64_t)p.seq * 64, (int64_t)nrows * p.seq * 64,
                      kTile);
  if (st != SA_OK) return st;
  st = make_map_f32_rows(&map_dq, dq_acc, p.seq, nrows);
  if (st != SA_OK) return st;
  st = make_map_f32_rows(&map_dq0, dq0, p.seq, p.batch);
  if (st != SA_OK) return st;
  CUtensorMap map_q0, map_k0;                            // the selector's rows: (d, token, 1, batch)
  st = make_map_16bit(&map_q0, p.q0.ptr, 64, p.seq, 1, p.batch, p.q0.st, 0, p.q0.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k0, p.k0.ptr, 64, p.seq, 1, p.batch, p.k0.st, 0, p.k0.sb, kTile);
  if (st != SA_OK) return st;
  WaitCtx status;
  st = wait_ctx(&status);
  if (st != SA_OK) return st;
  const int smem = BwdSmem::total + 1024;
  // One head per selector (the per-head form): the selection logits are the head's own, and the kernel merges the
  // two gradient paths before the MMAs.
  SA_CUDA_CHECK(cudaFuncSetAttribute(backward_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  {
    ProfileScope prof(SA_KERNEL_TC_BACKWARD, s);
    count_launch();
    backward_kernel<true><<<(unsigned)ntiles * nrows, kThreads, smem, s>>>(
        map_q, map_k, map_v, map_do, map_dq, map_dq0, map_q0, map_k0, lse2, carry, dbar, dk_acc, dk0,
        static_cast<__nv_bfloat16*>(dv), p.heads, p.seq, ntiles, p.exempt, p.scale, status, p.dv_rows);
  }
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
