// Tensor-core engine, forward side (sm_100a: TMA loads, tcgen05 MMAs, fp32 accumulators in TMEM).
//
//   colsum_kernel   selection pass: for one 128-key tile and a run of 128-query tiles, the product
//                   K0 Q0^T with KEYS on the TMEM lanes, so a thread owns one key and the column sum of
//                   relu'd, masked logits over the tile's queries is a register reduction.  Writes
//                   COLSUM[b][query tile][key].
//   scan_kernel     exclusive prefix of COLSUM across query tiles, in place (-> CARRY), plus one extra
//                   row holding the grand total.  One thread per key column; bandwidth-bound.
//   forward_wide_kernel  flash-style forward for one 128-query tile of one head over 128-key steps, taken from
//                   the diagonal back to key 0: S = Q K^T and L0 = Q0 K0^T by MMA (Q, Q0 in TMEM); relu(L0) under
//                   the selection mask is written to shared memory as bf16 and the in-tile exclusive running
//                   sum over queries is one more MMA, (-strictly-lower-triangular ones) x selection,
//                   accumulated into S; then online softmax in the log2 domain with the cross-tile carry
//                   subtracted per key, and O += P V in TMEM.  Four arithmetic warpgroups and a control warp
//                   that issues every load and MMA; steps software-pipelined so the tensor pipe works under
//                   the exponentials.  head_dim 64 and 128.
//
// Reference for the arithmetic: src/selective_attention/kernels.py:100-194 (selection, carry, forward).
#include <type_traits>

#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {
namespace {

constexpr int kTile = 128;          // query rows per CTA; also the carry checkpoint spacing
constexpr int kRowTile = 16384;     // bytes of a [128][64] bf16 operand tile

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A global load the compiler must issue where it is written (volatile asm keeps its place among the other
// volatile asm statements), so a value fetched one step ahead is really in flight during that step.
__device__ __forceinline__ float load_ahead(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// ---------------------------------------------------------------------------------------------------
// selection column sums
// ---------------------------------------------------------------------------------------------------
constexpr int kColsumChunk = 8;     // query tiles per CTA

template <int D>
__global__ void __launch_bounds__(128) colsum_kernel(const __grid_constant__ CUtensorMap map_q,
                                                     const __grid_constant__ CUtensorMap map_k, float* __restrict__ carry,
                                                     int seq, int ntiles, int exempt, float scale,
                                                     WaitCtx status, int q_offset, int mi_first) {
  constexpr int DK = D / 64;
  const int nj = blockIdx.x, b = blockIdx.z;
  // Query tiles from the key tile's own (the diagonal) on; in a prefill continuation from the first tile that holds a
  // new query on (rows before q_offset are not in the query tensor: TMA fills them with zeros, which select nothing).
  const int mi0 = max(nj, mi_first) + blockIdx.y * kColsumChunk;
  if (mi0 >= ntiles) return;
  const int count = min(kColsumChunk, ntiles - mi0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k0s = smem;                               // DK tiles [128 keys][64]
  uint8_t* q0s = smem + DK * kRowTile;               // 2 stages x DK tiles [128 queries][64]
  __shared__ uint64_t bar_k, bar_q[2], bar_mma[2];
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar_k, 1);
    mbar_init(&bar_q[0], 1);
    mbar_init(&bar_q[1], 1);
    mbar_init(&bar_mma[0], 1);
    mbar_init(&bar_mma[1], 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t idesc = instr_desc_bf16(128, 128, false, false);
  const uint32_t k0a = smem_u32(k0s), q0a = smem_u32(q0s);

  auto load_q = [&](int it) {
    uint64_t* bar = &bar_q[it & 1];
    mbar_expect_tx(bar, DK * kRowTile);
    for (int s = 0; s < DK; ++s)
      tma_load_4d(q0s + ((it & 1) * DK + s) * kRowTile, &map_q, bar, s * 64, (mi0 + it) * kTile - q_offset, 0, b);
  };
  auto issue = [&](int it) {
    mbar_wait(&bar_q[it & 1], (it >> 1) & 1, status, 200);
    tc_fence_after_sync();
    for (int ks = 0; ks < 4 * DK; ++ks)
      mma_ss(tmem + (it & 1) * 128, smem_desc(k0a + (ks >> 2) * kRowTile + (ks & 3) * 32, 16, 1024),
             smem_desc(q0a + ((it & 1) * DK + (ks >> 2)) * kRowTile + (ks & 3) * 32, 16, 1024), idesc, ks > 0);
    mma_commit(&bar_mma[it & 1]);
  };

  if (tid == 0) {
    mbar_expect_tx(&bar_k, DK * kRowTile);
    for (int s = 0; s < DK; ++s) tma_load_4d(k0s + s * kRowTile, &map_k, &bar_k, s * 64, nj * kTile, 0, b);
    load_q(0);
    if (count > 1) load_q(1);
    mbar_wait(&bar_k, 0, status, 201);
    issue(0);
  }
  const int j = nj * kTile + tid;
  for (int it = 0; it < count; ++it) {
    if (tid == 0 && it + 1 < count) issue(it + 1);
    mbar_wait(&bar_mma[it & 1], (it >> 1) & 1, status, 202);
    tc_fence_after_sync();
    if (tid == 0 && it + 2 < count) load_q(it + 2);     // stage (it & 1) is free: its MMA has completed
    const int mi = mi0 + it;
    const int i0 = mi * kTile;
    const bool diag = (mi == nj);
    float sum = 0.f;
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(lane_base + (it & 1) * 128 + c0, r);
      tmem_ld_wait();
      if (diag) {
#pragma unroll
        for (int e = 0; e < 32; ++e) sum += (j < i0 + c0 + e) ? fmaxf(__uint_as_float(r[e]), 0.f) : 0.f;
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) sum += fmaxf(__uint_as_float(r[e]), 0.f);
      }
    }
    if (j < exempt) sum = 0.f;
    if (j < seq) carry[((int64_t)b * (ntiles + 1) + mi) * seq + j] = sum * scale;
    tc_fence_before_sync();
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// One thread per key column: CARRY[b][mi][j] = sum of COLSUM[b][m'][j] over m' < mi, in place; row `ntiles`
// and total[b][j] receive the sum over all query tiles.  Only rows mi >= j / 128 exist.
__global__ void __launch_bounds__(256) scan_kernel(float* __restrict__ carry, float* __restrict__ total, int seq,
                                                   int ntiles, int mi_first, const float* __restrict__ init,
                                                   int64_t init_stride) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (j >= seq) return;
  float* col = carry + (int64_t)b * (ntiles + 1) * seq + j;
  float run = init ? init[(int64_t)b * init_stride + j] : 0.f;   // what the key received before the first query given
  int mi = max(j / kTile, mi_first);
  for (; mi + 8 <= ntiles; mi += 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = col[(int64_t)(mi + u) * seq];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      col[(int64_t)(mi + u) * seq] = run;
      run += x[u];
    }
  }
  for (; mi < ntiles; ++mi) {
    float x = col[(int64_t)mi * seq];
    col[(int64_t)mi * seq] = run;
    run += x;
  }
  col[(int64_t)ntiles * seq] = run;
  total[(int64_t)b * seq + j] = run;
}

// ---------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------
template <int N>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 16) tmem_ld16(taddr, r);
  else tmem_ld32(taddr, r);
}
template <int N>
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[N]) {
  if constexpr (N == 8) tmem_st8(taddr, r);
  else if constexpr (N == 16) tmem_st16(taddr, r);
  else tmem_st32(taddr, r);
}

// ---------------------------------------------------------------------------------------------------
// forward: 128-query tile x 128-key steps, one CTA per SM
// ---------------------------------------------------------------------------------------------------
// One 128-query tile of one head.  Key steps of 128 run from the diagonal back to key 0: the keys nearest the query
// carry the least history, so the running maximum settles within the first steps and the output accumulator,
// which stays in TMEM for the whole loop, is rescaled only while the maximum still moves.  One CTA keeps the tensor
// pipe and four warpgroups busy without a second resident CTA: a step covers 128 keys (N = 128 MMAs run at the full tensor rate and the per-step barriers
// are paid half as often), a control warp issues every load and MMA, and the steps are software-pipelined: after
// the logits and the row maximum of step t the arithmetic warps write the selection tile of step t + 1 (its L0 was
// issued right behind the running sum of step t), and only then do the exponentials of step t, so S and the
// triangular running sum of step t + 1 run on the tensor pipe under the exponentials instead of being waited for.
// head_dim 64 keeps two stages of K, K0 and V in shared memory; head_dim 128 has room for one and refills a
// tile as soon as the MMA that read it has completed.
template <int D>
struct WideSmem {
  static constexpr int DK = D / 64;
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kTileBytes = DK * kRowTile;     // one [128 keys][D] operand
  static constexpr int q = 0;                          // landing tiles of Q (and Q0 at head_dim 64), then the triangular ones
  static constexpr int sel = q + 2 * kRowTile;         // [128 queries][128 keys] bf16 as two key tiles (B of the running sum);
                                                       //   head_dim 128: first the landing tiles of Q0
  static constexpr int p = sel + 2 * kRowTile;         // the same shape: P (A of P V)
  static constexpr int k = p + 2 * kRowTile;
  static constexpr int k0 = k + kStages * kTileBytes;
  static constexpr int v = k0 + kStages * kTileBytes;
  static constexpr int total = v + kStages * kTileBytes;   // 192 KB for both head dims
  static constexpr int q0_landing = (D == 64) ? q + kRowTile : sel;
};
constexpr int kWideCompute = 512;                      // four warpgroups: 32 of a step's 128 key columns, D / 4 of the d each
constexpr int kWideThreads = kWideCompute + 32;        // + the control warp: one lane issues every TMA load and MMA
constexpr int kWideBarrier = 1;                        // hardware barrier id of the arithmetic warps
constexpr int kMaxLiveTiles = 1024;                    // key tiles of a sequence when dead tiles are left out (sa_tc_skip.cu)

template <int D, bool SELF, bool LIVE>   // LIVE: a table of live key tiles is given and the dead ones are left out
__global__ void __launch_bounds__(kWideThreads, 1)
    forward_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_q0,
                        const __grid_constant__ CUtensorMap map_k0, const float* __restrict__ carry,
                        float* __restrict__ out, float* __restrict__ lse2, int heads, int seq, int ntiles, int exempt,
                        float scale, WaitCtx status, __nv_bfloat16* __restrict__ out_lowp, RowLayout out_lowp_rows,
                        int q_offset, const uint8_t* __restrict__ alive) {
  using L = WideSmem<D>;
  constexpr int DK = D / 64, DH = D / 4, NC = 32, ST = L::kStages;
  // TMEM columns: S and L0 (fp32, 128 each), the output accumulator (D), Q and Q0 as bf16 pairs (D / 2 each)
  constexpr uint32_t kColS = 0, kColL = 128, kColO = 256, kColQ = kColO + D, kColQ0 = kColQ + D / 2;
  // head_dim 64 leaves 128 columns: the triangular matrix and P live there as bf16 pairs (64 columns each), so the
  // running-sum and P V MMAs fetch only their B operands from shared memory.  head_dim 128 keeps both in shared memory.
  constexpr bool kTmemAB = (D == 64);
  constexpr uint32_t kColTri = 384, kColP = 448;

  const int nrows = gridDim.x / (ntiles - q_offset / kTile);  // batch * heads (the grid covers the query tiles with rows to compute)
  const int mi = ntiles - 1 - (int)(blockIdx.x / nrows);      // heaviest query tiles first
  const int n = blockIdx.x % nrows;
  const int b = n / heads, h = n - b * heads;
  const int i0 = mi * kTile;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Completion barriers (one MMA commit each): bar_l0 L0 of a step; bar_tri S and running sum of a step; bar_pv
  // P V of a step; bar_fin the last P V.  Arrival barriers (one arrival per arithmetic warp and step): bar_sel
  // selection tile written and the previous step's logits read; bar_p P written and O rescaled.
  __shared__ uint64_t bar_q, bar_k[2], bar_k0[2], bar_v[2], bar_l0, bar_tri, bar_pv, bar_fin, bar_sel, bar_p, bar_setup;
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float carry_s[2][kTile];
  __shared__ float rmax_s[4][kTile];
  __shared__ uint16_t live_s[kMaxLiveTiles + 1];              // with a table of live tiles: this query tile's key tiles,
  __shared__ int live_count_s;                                //   nearest first

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (LIVE && warp == 1) {
    const uint8_t* live_row = alive + ((int64_t)n * ntiles + mi) * ntiles;
    int cnt = 0;
    for (int base = mi; base >= 0; base -= 32) {
      const int nj = base - lane;
      const bool f = nj >= 0 && live_row[nj] != 0;
      const unsigned m = __ballot_sync(0xffffffffu, f);
      if (f) live_s[cnt + __popc(m & ((1u << lane) - 1u))] = (uint16_t)nj;
      cnt += __popc(m);
    }
    if (lane == 0) live_count_s = cnt;
  }
  if (tid == 0) {
    mbar_init(&bar_q, 1);
    for (int u = 0; u < 2; ++u) {
      mbar_init(&bar_k[u], 1);
      mbar_init(&bar_k0[u], 1);
      mbar_init(&bar_v[u], 1);
    }
    mbar_init(&bar_l0, 1);
    mbar_init(&bar_tri, 1);
    mbar_init(&bar_pv, 1);
    mbar_init(&bar_fin, 1);
    mbar_init(&bar_sel, kWideCompute / 32);
    mbar_init(&bar_p, kWideCompute / 32);
    mbar_init(&bar_setup, kWideCompute / 32);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t sa = smem_u32(smem);
  // 128-key steps: every key tile up to and including the diagonal one, or the live ones only.  Step index `it`
  // counts from the diagonal (it = 0) back towards key 0; key_tile(it) is the tile it covers.
  const int steps = LIVE ? live_count_s : mi + 1;
  auto key_tile = [&](int it) { return LIVE ? (it < steps ? (int)live_s[it] : 0) : steps - 1 - it; };

  if (warp == kWideCompute / 32) {
    // =============================== control warp: TMA loads and MMA issue ===============================
    if (lane == 0) {
      // A tile of step it lives in stage slot(it); the j-th fill of a stage completes its barrier's phase j.
      auto slot = [](int it) { return ST == 2 ? (it & 1) : 0; };
      auto fill = [](int it) { return (uint32_t)((ST == 2 ? (it >> 1) : it) & 1); };
      auto load_tile = [&](int off, const CUtensorMap* map, uint64_t* bars, int it, int head) {
        uint64_t* bar = &bars[slot(it)];
        mbar_expect_tx(bar, L::kTileBytes);
        for (int s2 = 0; s2 < DK; ++s2)
          tma_load_4d(smem + off + slot(it) * L::kTileBytes + s2 * kRowTile, map, bar, s2 * 64, key_tile(it) * kTile, head, b);
      };
      auto load_k = [&](int it) { load_tile(L::k, &map_k, bar_k, it, h); };
      auto load_k0 = [&](int it) { if (!SELF) load_tile(L::k0, &map_k0, bar_k0, it, 0); };   // SELF: K0 is K
      auto load_v = [&](int it) { load_tile(L::v, &map_v, bar_v, it, h); };
      const uint32_t idesc_s = instr_desc_bf16(128, 128, false, false);
      const uint32_t idesc_tri = instr_desc_bf16(128, 128, false, true, /*negate_a=*/true);
      const uint32_t idesc_pv = instr_desc_bf16(128, D, false, true);
      auto issue_l0 = [&](int it) {                            // L0 = Q0 K0^T
        mbar_wait(SELF ? &bar_k[slot(it)] : &bar_k0[slot(it)], fill(it), status, 311);
        tc_fence_after_sync();
        const uint32_t tile = sa + (SELF ? L::k : L::k0) + slot(it) * L::kTileBytes;
        for (int ks = 0; ks < 4 * DK; ++ks)
          mma_ts(tmem + kColL, tmem + (SELF ? kColQ : kColQ0) + ks * 8,
                 smem_desc(tile + (ks >> 2) * kRowTile + (ks & 3) * 32, 16, 1024), idesc_s, ks > 0);
        mma_commit(&bar_l0);
      };
      auto issue_s_tri = [&](int it) {                         // S = Q K^T, then S -= TRI x selection
        mbar_wait(&bar_k[slot(it)], fill(it), status, 312);
        tc_fence_after_sync();
        const uint32_t tile = sa + L::k + slot(it) * L::kTileBytes;
        for (int ks = 0; ks < 4 * DK; ++ks)
          mma_ts(tmem + kColS, tmem + kColQ + ks * 8, smem_desc(tile + (ks >> 2) * kRowTile + (ks & 3) * 32, 16, 1024),
                 idesc_s, ks > 0);
        for (int ks = 0; ks < 8; ++ks) {
          if (kTmemAB)
            mma_ts(tmem + kColS, tmem + kColTri + ks * 8, smem_desc(sa + L::sel + ks * 2048, kRowTile, 1024), idesc_tri, 1);
          else
            mma_ss(tmem + kColS, smem_desc(sa + L::q + (ks >> 2) * kRowTile + (ks & 3) * 32, 16, 1024),
                   smem_desc(sa + L::sel + ks * 2048, kRowTile, 1024), idesc_tri, 1);
        }
        mma_commit(&bar_tri);
      };
      auto issue_pv = [&](int it, uint64_t* bar) {             // O += P V
        mbar_wait(&bar_v[slot(it)], fill(it), status, 315);
        tc_fence_after_sync();
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t vdesc = smem_desc(sa + L::v + slot(it) * L::kTileBytes + ks * 2048, kRowTile, 1024);
          if (kTmemAB)
            mma_ts(tmem + kColO, tmem + kColP + ks * 8, vdesc, idesc_pv, (it > 0 || ks > 0) ? 1u : 0u);
          else
            mma_ss(tmem + kColO, smem_desc(sa + L::p + (ks >> 2) * kRowTile + (ks & 3) * 32, 16, 1024), vdesc, idesc_pv,
                   (it > 0 || ks > 0) ? 1u : 0u);
        }
        mma_commit(bar);
      };

      mbar_expect_tx(&bar_q, (SELF ? 1 : 2) * DK * kRowTile);
      for (int s2 = 0; s2 < DK; ++s2) {
        tma_load_4d(smem + L::q + s2 * kRowTile, &map_q, &bar_q, s2 * 64, i0 - q_offset, h, b);
        if (!SELF) tma_load_4d(smem + L::q0_landing + s2 * kRowTile, &map_q0, &bar_q, s2 * 64, i0 - q_offset, 0, b);
      }
      load_k0(0);
      load_k(0);
      load_v(0);
      if (ST == 2 && steps > 1) {
        load_k0(1);
        load_k(1);
        load_v(1);
      }
      mbar_wait(&bar_setup, 0, status, 317);                   // Q, Q0 in TMEM and the triangular tile in place
      tc_fence_after_sync();
      issue_l0(0);
#pragma unroll(D == 64 ? 2 : 1)   // head_dim 64: the stage and phase parities become constants (-2.6 %); head_dim 128: +11 %
      for (int it = 0; it < steps; ++it) {
        mbar_wait(&bar_sel, it & 1, status, 318);              // selection of step it written; logits of it - 1 read;
        tc_fence_after_sync();                                 //   L0 of step it consumed: its K0 tile is free
        if (it + ST < steps) load_k0(it + ST);
        issue_s_tri(it);
        const bool l0_now = !(SELF && ST == 1);                // one-stage SELF: K of the next step is not loaded yet
        if (l0_now && it + 1 < steps) issue_l0(it + 1);
        if (it > 0) {
          mbar_wait(&bar_p, (it - 1) & 1, status, 320);        // P of step it - 1 written, O rescaled
          tc_fence_after_sync();
          if (ST == 2 && it >= 2) {                            // before this barrier's next commit: P V of it - 2 done,
            mbar_wait(&bar_pv, it & 1, status, 321);           //   so its V tile may be refilled
            load_v(it);
          }
          issue_pv(it - 1, &bar_pv);
        }
        mbar_wait(&bar_tri, it & 1, status, 319);              // S of step it done: its K tile is free
        if (it + ST < steps) load_k(it + ST);
        if (!l0_now && it + 1 < steps) issue_l0(it + 1);
        if (ST == 1 && it > 0) {                               // the single V tile: refilled with V of step it (for the
          mbar_wait(&bar_pv, (it - 1) & 1, status, 321);       //   P V issued in the next iteration) once P V of step
          load_v(it);                                          //   it - 1 has completed
        }
      }
      mbar_wait(&bar_p, (steps - 1) & 1, status, 322);
      tc_fence_after_sync();
      issue_pv(steps - 1, &bar_fin);
    }
    __syncwarp();
  } else {
    // ======================================= arithmetic warps ============================================
    const int row = tid & 127, wg = tid >> 7;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    auto arrive = [&](uint64_t* bar) {                         // this warp's shared-memory and TMEM accesses are done
      fence_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    // Q and Q0 rows from the landing tiles into TMEM as bf16 pairs; warpgroup wg moves D / 4 of the D columns
    mbar_wait(&bar_q, 0, status, 310);
    {
      constexpr int kChunks = D / 32;                          // 16-byte chunks per thread and matrix
#pragma unroll
      for (int m = 0; m < (SELF ? 1 : 2); ++m) {
        const uint8_t* src = smem + (m == 0 ? L::q : L::q0_landing);
        uint32_t w[kChunks * 4];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          const int chunk = wg * kChunks + c;                  // chunk index along D (8 elements each)
          const uint4 v4 = *reinterpret_cast<const uint4*>(src + (chunk >> 3) * kRowTile + swz_off(row, chunk & 7));
          w[4 * c] = v4.x; w[4 * c + 1] = v4.y; w[4 * c + 2] = v4.z; w[4 * c + 3] = v4.w;
        }
        tmem_st_n<kChunks * 4>(lane_base + (m == 0 ? kColQ : kColQ0) + wg * (kChunks * 4), w);
      }
    }
    tmem_st_wait();
    named_barrier(kWideBarrier, kWideCompute);                 // the landing tiles have been read by everyone
    // strictly-lower-triangular ones TRI[i][r] = 1 for r < i over the landing area: a K-major A operand of two
    // [128][64] tiles; thread (row, wg) writes running-sum indices r = 32 wg .. 32 wg + 31 of its row
    if (kTmemAB) {                                             // 32 running-sum indices = 16 packed columns per thread
      uint32_t w[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int r = wg * 32 + 2 * e;
        w[e] = pack_bf16(r < row ? 1.f : 0.f, (r + 1) < row ? 1.f : 0.f);
      }
      tmem_st16(lane_base + kColTri + wg * 16, w);
      tmem_st_wait();
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int chunk = wg * 4 + c;
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = chunk * 8 + 2 * e;
          w[e] = pack_bf16(r < row ? 1.f : 0.f, (r + 1) < row ? 1.f : 0.f);
        }
        *reinterpret_cast<uint4*>(smem + L::q + (chunk >> 3) * kRowTile + swz_off(row, chunk & 7)) =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    arrive(&bar_setup);

    const float c1 = scale * kLog2e;
    const float* carry_row = carry + ((int64_t)b * (ntiles + 1) + mi) * seq;
    const int i = i0 + row;
    const int cw = wg * NC;                                    // this warpgroup's key columns within a step

    // The carry of a step's keys is fetched from global memory a step before it is staged, so the load's latency
    // is spent under the exponentials of the step before.
    auto fetch_carry = [&](int it) {
      const int j = key_tile(it) * kTile + tid;
      return (tid < kTile && it < steps && j < seq) ? load_ahead(carry_row + j) : 0.f;
    };
    // selection relu(L0) under the mask of step `it` -> bf16 tile, in two halves of 16 columns; also stages the
    // step's carry (scaled) for the logits pass
    auto selection = [&](int it, float carry_value) {
      const int j0 = key_tile(it) * kTile;
      if (tid < kTile) carry_s[it & 1][tid] = -carry_value * kLog2e;   // negated: the logits pass adds it in an FMA
      mbar_wait(&bar_l0, it & 1, status, 313);
      tc_fence_after_sync();
      const bool masked = (j0 + kTile > i0) || (j0 < exempt);
      uint32_t r32[32];
      tmem_ld32(lane_base + kColL + cw, r32);                 // one load and one wait for the step's 32 columns
      tmem_ld_wait();
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        const uint32_t* r = r32 + hc * 16;
        float s[16];
        if (masked) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int j = j0 + cw + hc * 16 + e;
            s[e] = (j < i && j >= exempt) ? __uint_as_float(r[e]) : 0.f;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) s[e] = __uint_as_float(r[e]);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {                          // the relu rides on the bf16 conversion
          uint4 w = make_uint4(pack_bf16_relu(s[c * 8 + 0], s[c * 8 + 1]), pack_bf16_relu(s[c * 8 + 2], s[c * 8 + 3]),
                               pack_bf16_relu(s[c * 8 + 4], s[c * 8 + 5]), pack_bf16_relu(s[c * 8 + 6], s[c * 8 + 7]));
          *reinterpret_cast<uint4*>(smem + L::sel + (wg >> 1) * kRowTile + swz_off(row, (wg & 1) * 4 + hc * 2 + c)) = w;
        }
      }
      arrive(&bar_sel);
    };

    float run_max = -INFINITY, run_den = 0.f;                  // run_den: this warpgroup's share of the denominator
    selection(0, fetch_carry(0));
    float next_carry = fetch_carry(1);
    // One 128-key step.  The diagonal step (it = 0: causal mask inside the tile, nothing to wait for or rescale yet) is
    // peeled off the loop.
    auto step = [&](int it, auto first_tag) {
      constexpr bool kFirst = decltype(first_tag)::value;
      const int j0 = key_tile(it) * kTile;
      // ---- logits z = (S * scale - carry) * log2(e) after S -= TRI x selection, and the row maximum -----------
      mbar_wait(&bar_tri, it & 1, status, 314);
      tc_fence_after_sync();
      // Packed fp32x2 arithmetic (two results per issue slot) for the logits, the shift by the maximum and the row sum.
      float2 z[NC / 2];
      {
        uint32_t r[NC];
        tmem_ld32(lane_base + kColS + cw, r);
        tmem_ld_wait();
        const float4* ncs = reinterpret_cast<const float4*>(carry_s[it & 1] + cw);   // -carry * log2(e), broadcast loads
        const float2 cc = make_float2(c1, c1);
        float tile_max = -INFINITY;
#pragma unroll
        for (int e4 = 0; e4 < NC / 4; ++e4) {
          const float4 nc = ncs[e4];
          float2 a = __ffma2_rn(make_float2(__uint_as_float(r[4 * e4]), __uint_as_float(r[4 * e4 + 1])), cc,
                                make_float2(nc.x, nc.y));
          float2 b2 = __ffma2_rn(make_float2(__uint_as_float(r[4 * e4 + 2]), __uint_as_float(r[4 * e4 + 3])), cc,
                                 make_float2(nc.z, nc.w));
          if (kFirst) {                                        // the diagonal tile
            const int jj = j0 + cw + 4 * e4;
            if (jj > i) a.x = -INFINITY;
            if (jj + 1 > i) a.y = -INFINITY;
            if (jj + 2 > i) b2.x = -INFINITY;
            if (jj + 3 > i) b2.y = -INFINITY;
          }
          tile_max = fmaxf(fmaxf(tile_max, fmaxf(a.x, a.y)), fmaxf(b2.x, b2.y));
          z[2 * e4] = a;
          z[2 * e4 + 1] = b2;
        }
        rmax_s[wg][row] = tile_max;
      }
      named_barrier(kWideBarrier, kWideCompute);
      // every row has its own key in the diagonal tile, so the maximum is finite from the first step on
      const float new_max =
          fmaxf(fmaxf(run_max, fmaxf(rmax_s[0][row], rmax_s[1][row])), fmaxf(rmax_s[2][row], rmax_s[3][row]));
      const float alpha = ex2(run_max - new_max);
      run_max = new_max;

      // ---- the next step's selection tile first: its S and running sum then run under the exponentials --------
      if (it + 1 < steps) selection(it + 1, next_carry);
      next_carry = fetch_carry(it + 2);

      // ---- exponentials, P, and the accumulator rescale ---------------------------------------------------------
      float2 rs = make_float2(0.f, 0.f);
      const float2 nm = make_float2(-new_max, -new_max);
#pragma unroll
      for (int e = 0; e < NC / 2; ++e) {
        const float2 x = __fadd2_rn(z[e], nm);
        z[e] = make_float2(ex2(x.x), ex2(x.y));
        rs = __fadd2_rn(rs, z[e]);
      }
      run_den = run_den * alpha + (rs.x + rs.y);
      if (!kFirst) {
        mbar_wait(&bar_pv, (it - 1) & 1, status, 323);         // P V of the previous step: P tile and O are free
        tc_fence_after_sync();
      }
      if (kTmemAB) {                                           // P as bf16 pairs: keys 32 wg .. at column 16 wg of P
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) w[e] = pack_bf16(z[e].x, z[e].y);
        tmem_st16(lane_base + kColP + wg * 16, w);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 w = make_uint4(pack_bf16(z[c * 4].x, z[c * 4].y), pack_bf16(z[c * 4 + 1].x, z[c * 4 + 1].y),
                               pack_bf16(z[c * 4 + 2].x, z[c * 4 + 2].y), pack_bf16(z[c * 4 + 3].x, z[c * 4 + 3].y));
          *reinterpret_cast<uint4*>(smem + L::p + (wg >> 1) * kRowTile + swz_off(row, (wg & 1) * 4 + c)) = w;
        }
      }
      if (!kFirst && __any_sync(0xffffffffu, alpha != 1.f)) {  // the accumulator follows the maximum while it moves
        uint32_t r[DH];
        tmem_ld_n<DH>(lane_base + kColO + wg * DH, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < DH; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
        tmem_st_n<DH>(lane_base + kColO + wg * DH, r);
      }
      tmem_st_wait();                                          // P (head_dim 64) and the rescaled accumulator are in TMEM
      arrive(&bar_p);
    };
    step(0, std::true_type{});
    for (int it = 1; it < steps; ++it) step(it, std::false_type{});
    mbar_wait(&bar_fin, 0, status, 316);                       // the last P V
    tc_fence_after_sync();

    named_barrier(kWideBarrier, kWideCompute);                 // everyone has read the last row maxima
    rmax_s[wg][row] = run_den;                                 // the warpgroups hold disjoint shares of the denominator
    named_barrier(kWideBarrier, kWideCompute);
    const float den = (rmax_s[0][row] + rmax_s[1][row]) + (rmax_s[2][row] + rmax_s[3][row]);
    const float inv = 1.f / den;
    uint32_t r[DH];
    tmem_ld_n<DH>(lane_base + kColO + wg * DH, r);
    tmem_ld_wait();
    if (i < seq && i >= q_offset) {                            // rows before q_offset belong to an earlier call
      const int iq = i - q_offset;                             // row inside the query tensor
      const int q_rows = seq - q_offset;
      float4* orow = reinterpret_cast<float4*>(out + ((int64_t)n * q_rows + iq) * D + wg * DH);
#pragma unroll
      for (int d = 0; d < DH; d += 4)
        orow[d >> 2] = make_float4(__uint_as_float(r[d]) * inv, __uint_as_float(r[d + 1]) * inv,
                                   __uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv);
      if (wg == 0) lse2[(int64_t)n * q_rows + iq] = run_max + log2f(den);
      if (out_lowp != nullptr) {                               // the same rows in the operand dtype, in the caller's layout
        uint4* lrow = reinterpret_cast<uint4*>(out_lowp + out_lowp_rows.at(b, h, iq) + wg * DH);
#pragma unroll
        for (int d = 0; d < DH; d += 8)
          lrow[d >> 3] = make_uint4(pack_bf16(__uint_as_float(r[d]) * inv, __uint_as_float(r[d + 1]) * inv),
                                    pack_bf16(__uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv),
                                    pack_bf16(__uint_as_float(r[d + 4]) * inv, __uint_as_float(r[d + 5]) * inv),
                                    pack_bf16(__uint_as_float(r[d + 6]) * inv, __uint_as_float(r[d + 7]) * inv));
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <int D>
int forward_impl(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  const int ntiles = (p.seq + kTile - 1) / kTile;
  const int q_rows = p.seq - p.q_offset;                 // rows of the query tensor (all of them unless continuing a prefill)
  const int mi_first = p.q_offset / kTile;               // first query tile with a row to compute
  CUtensorMap map_q, map_k128, map_v128;                 // boxes of 128 rows x 64 columns
  int st = make_map_16bit(&map_q, p.q.ptr, D, q_rows, p.heads, p.batch, p.q.st, p.q.sh, p.q.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k128, p.k.ptr, D, p.seq, p.heads, p.batch, p.k.st, p.k.sh, p.k.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_v128, p.v.ptr, D, p.seq, p.heads, p.batch, p.v.st, p.v.sh, p.v.sb, kTile);
  if (st != SA_OK) return st;
  CUtensorMap map_q0, map_k0;                            // the selector's rows: (d, token, 1, batch)
  st = make_map_16bit(&map_q0, p.q0.ptr, D, q_rows, 1, p.batch, p.q0.st, 0, p.q0.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k0, p.k0.ptr, D, p.seq, 1, p.batch, p.k0.st, 0, p.k0.sb, kTile);
  if (st != SA_OK) return st;
  WaitCtx status;
  st = wait_ctx(&status);
  if (st != SA_OK) return st;

  constexpr int DK = D / 64;
  const int colsum_smem = 3 * DK * kRowTile + 1024;
  SA_CUDA_CHECK(cudaFuncSetAttribute(colsum_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, colsum_smem));
  dim3 gc(ntiles, (ntiles - mi_first + kColsumChunk - 1) / kColsumChunk, p.batch);
  {
    ProfileScope prof(SA_KERNEL_TC_COLSUM, s);
    count_launch();
    colsum_kernel<D><<<gc, 128, colsum_smem, s>>>(map_q0, map_k0, carry, p.seq, ntiles, p.exempt, p.scale, status,
                                                  p.q_offset, mi_first);
  }
  SA_CUDA_CHECK(cudaGetLastError());
  dim3 gs((p.seq + 255) / 256, p.batch);
  {
    ProfileScope prof(SA_KERNEL_TC_SCAN, s);
    count_launch();
    scan_kernel<<<gs, 256, 0, s>>>(carry, total, p.seq, ntiles, mi_first, p.carry_init, p.carry_init_stride);
  }
  SA_CUDA_CHECK(cudaGetLastError());

  const uint8_t* alive = nullptr;
  if (p.tile_table != nullptr && ntiles <= kMaxLiveTiles) {
    st = build_tile_table(p, carry, s);
    if (st != SA_OK) return st;
    alive = static_cast<const uint8_t*>(p.tile_table);
  }
  const unsigned grid = (unsigned)(ntiles - mi_first) * p.batch * p.heads;
  const bool self = (p.heads == 1) && !p.external_selector;   // one head per selector: the selection logits are the head's own
  const int wide_smem = WideSmem<D>::total + 1024;
  auto launch = [&](auto kernel) -> int {
    SA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide_smem));
    ProfileScope prof(SA_KERNEL_TC_FORWARD, s);
    count_launch();
    kernel<<<grid, kWideThreads, wide_smem, s>>>(map_q, map_k128, map_v128, map_q0, map_k0, carry, out, lse2, p.heads, p.seq,
                                                 ntiles, p.exempt, p.scale, status, static_cast<__nv_bfloat16*>(p.out_lowp),
                                                 p.out_lowp_rows, p.q_offset, alive);
    return SA_OK;
  };
  if (alive != nullptr) st = self ? launch(forward_wide_kernel<D, true, true>) : launch(forward_wide_kernel<D, false, true>);
  else st = self ? launch(forward_wide_kernel<D, true, false>) : launch(forward_wide_kernel<D, false, false>);
  if (st != SA_OK) return st;
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace

int forward(const Problem& p, float* out, float* lse2, float* carry, float* total, cudaStream_t s) {
  if (p.head_dim == 64) return forward_impl<64>(p, out, lse2, carry, total, s);
  if (p.head_dim == 128) return forward_impl<128>(p, out, lse2, carry, total, s);
  return SA_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace sa
