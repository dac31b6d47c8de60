// Tensor-core engine, backward (sm_100a: TMA loads and reduce-adds, tcgen05 MMAs, fp32 accumulators in TMEM).
//
// One CTA owns one 128-key tile of one head and walks the query tiles LAST TO FIRST in 64-query halves.  All
// score-shaped tiles are computed transposed, KEYS on the TMEM lanes (S^T = K Q^T, dP^T = V dO^T, L0^T = K0 Q0^T), so
// one thread owns one key and sees that key's queries along its registers.  The two running sums down the query
// axis are then thread-local fp32 recurrences walked from the last query to the first:
//     F[i]  = carry_after_tile - sum_{r >= i} sel[r]          (history term rebuilt per key)
//     U[i]  = suffix + sum_{i' > i} dz[i']                      (logit gradient of later queries)
// with  P = exp2(z - lse),  dz = P (dP - dbar),  g = gate ? -U : 0.
//
// Roles.  Warps 0-15 (four warpgroups) do the arithmetic: within a half each warpgroup takes 16 query columns of
// every key row; chunk totals are exchanged through shared memory so the recurrences chain across chunks, halves
// and tiles.  Warp 16 is the control warp: one lane issues every TMA load and every MMA.
//
// Operand sources and issue points.  Measured on B200, a head-tile of a form with every operand in shared memory and
// each product issued when its inputs appear costs ~10.5 k cycles of which the arithmetic is ~3 k and the MMAs ~4 k;
// the rest is hand-over latency, because every product the arithmetic warps wait for is issued only after an arrival
// of theirs has travelled to the control warp and the MMA's completion has travelled back.  Here each such product is
// issued one arithmetic pass EARLIER than it is needed, into columns that are free by then:
//     L0^T of half n + 1 -> Z   when the selection pass of half n has read Z
//     S^T  of half n + 1 -> Y   when P^T and dz^T of half n (which live in Y) have been handed to dV and dK
//     dP^T of half n + 1 -> X   when g^T of half n (which lives in X) has been handed to dK0
// K and V sit in TMEM as bf16 pairs (A of S^T and dP^T); P^T, dz^T and g^T are written by each thread as bf16 pairs
// over the score columns that SAME thread has just read (its 16 columns of Y hold P^T then dz^T, 8 packed columns
// each; its 16 columns of X hold g^T), so no barrier is needed between reading a score tile and overwriting it, and
// dV, dK, dK0 read their A operand from TMEM with a stride of 16 columns per 16-query step.  L0^T = K0 Q0^T and the
// per-tile dQ = dz K, dQ0 = g K0 take both operands from shared memory.  TMEM, 512 columns: K, V (32 each) | dV, dK,
// dK0 | Z | X | Y | one accumulator shared by dQ and dQ0 (64 each): dQ is read out at the tile's end, dQ0 in the
// middle of the next tile's first half.  The query-side tiles (Q, Q0, dO) arrive per half through a ring of three
// 24 KB slots; dQ / dQ0 leave through their own fp32 staging tile and TMA reduce-add.
//
// SELF variant (one head per selector, i.e. the per-head form reshaped to (B H, 1, T, D)): the selection logits are the
// head's own logits, so S^T serves as L0^T, and since Q0 = Q and K0 = K the two gradient paths add before the MMAs:
// dK += (dz + g)^T Q and dQ = (dz + g) K, with (dz + g)^T in this thread's X columns.  40 MMAs per query tile instead
// of 64, no Q0 / K0 tiles, no Z, one read-out per tile (deferred into the next tile's first half).
//
// Code shape.  The diagonal tile, the only one that needs the causal mask inside the tile, is the LAST tile of a CTA's
// walk: the loop holds the unmasked form of the per-half arithmetic only and the masked form runs once after it, and
// the two halves of a tile are inlined (constant barrier parities and tile addresses).  That removes no work and 8 % of
// the time.  LIVE: with a table of live tiles (sa_tc_skip.cu) the walk starts at the key tile's last live query tile.
//
// Reference for the arithmetic: src/selective_attention/kernels.py:196-268 (one head), :271-364 (the shared
// selection-gradient products).
#include <type_traits>

#include "sa_tc_bwd_passes.cuh"

namespace sa {
namespace tc {
namespace {

using namespace bwd;

constexpr int kRing = 3;             // half-tile slots of Q, Q0, dO in flight

struct Smem {
  static constexpr int k = 0;                              // [128 keys][64], stationary
  static constexpr int v = k + kRowTile;
  static constexpr int k0 = v + kRowTile;
  static constexpr int ring = k0 + kRowTile;               // kRing x (Q, Q0, dO) half tiles [64 queries][64]
  static constexpr int dz = ring + kRing * 3 * kHalfTile;  // [128 keys][128 queries] bf16 as two query-half tiles
  static constexpr int g = dz + 2 * kRowTile;
  static constexpr int out = g + 2 * kRowTile;             // fp32 [128 queries][64] as two [128][32] boxes
  static constexpr int total = out + 2 * kRowTile;         // 216 KB
};

// TMEM columns (Z, X, Y: sa_tc_bwd_passes.cuh)
constexpr uint32_t kColK = 0, kColV = 32, kColDV = 64, kColDK = 128, kColDK0 = 192, kColDQ = 448;

template <bool SELF, bool LIVE>   // LIVE: a table of live tiles is given (sa_tc_skip.cu)
__global__ void __launch_bounds__(kThreads, 1) backward_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ CUtensorMap map_dq0,
    const __grid_constant__ CUtensorMap map_q0, const __grid_constant__ CUtensorMap map_k0,
    const float* __restrict__ lse2, const float* __restrict__ carry, const float* __restrict__ dbar,
    float* __restrict__ dk_acc, float* __restrict__ dk0, __nv_bfloat16* __restrict__ dv, int heads, int seq,
    int ntiles, int exempt, float scale, WaitCtx status, RowLayout dv_rows, const uint8_t* __restrict__ alive) {
  using L = Smem;
  constexpr int D = 64;
  // One (batch, head) row after the other, and within a row the key tiles with the most query tiles first: the CTAs
  // resident at one time belong to one or two rows and walk the same query tiles from the last one down, so every
  // Q, Q0, dO tile is fetched from DRAM once and then served from L2 to the row's other CTAs.
  int n, nj;
  tile_of_block(blockIdx.x, ntiles, gridDim.x / ntiles, LIVE, n, nj);
  const int b = n / heads, h = n - b * heads;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Completion barriers (MMA commits and TMA loads) and arrival barriers (arithmetic warps).  bar_l0 .. bar_g complete
  // one phase per half; each side reaches its next wait on one of them only after the other side has consumed the
  // previous phase, so a poller can never see two phases complete between two polls.
  __shared__ uint64_t bar_kv, bar_setup, bar_ld[kRing], bar_free[kRing], bar_l0, bar_s, bar_dp, bar_sel, bar_early, bar_g,
      bar_dq, bar_dq0, bar_dqread, bar_dq0read, bar_fin;
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float lse_s[kTile];
  __shared__ __align__(16) float dbar_s[kTile];
  __shared__ float sel_tot[kGroups][kTile];
  __shared__ float dz_tot[kGroups][kTile];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  __shared__ int top_s;
  if (LIVE && warp == 1) find_top_tile(alive, n, nj, ntiles, lane, &top_s);
  if (tid == 0) {
    mbar_init(&bar_kv, 1);
    for (int u = 0; u < kRing; ++u) {
      mbar_init(&bar_ld[u], 1);
      mbar_init(&bar_free[u], 1);
    }
    mbar_init(&bar_setup, kComputeThreads / 32);
    mbar_init(&bar_l0, 1);
    mbar_init(&bar_s, 1);
    mbar_init(&bar_dp, 1);
    mbar_init(&bar_sel, 1);
    mbar_init(&bar_early, 1);
    mbar_init(&bar_g, kComputeThreads / 32);
    mbar_init(&bar_dq, 1);
    mbar_init(&bar_dq0, 1);
    mbar_init(&bar_dqread, 1);
    mbar_init(&bar_dq0read, 1);
    mbar_init(&bar_fin, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t sa = smem_u32(smem);
  const int mi_top = LIVE ? top_s : ntiles - 1;   // the walk starts at the last query tile, or at the last live one
  const int n_iter = mi_top - nj + 1;
  const int n_half = 2 * n_iter;

  if (warp == kComputeThreads / 32) {
    // =============================== control warp: TMA loads and MMA issue ===============================
    if (lane == 0) {
      const uint32_t idesc_t = instr_desc_bf16(128, 64, false, false);     // keys x 64 queries, K = D
      const uint32_t idesc_acc = instr_desc_bf16(128, 64, false, true);    // A K-major (keys x queries), B MN-major
      const uint32_t idesc_dq = instr_desc_bf16(128, 64, true, true);      // A MN-major (queries x keys), B MN-major
      // Half index hn counts from the last query half: tile it = hn / 2 (query tile mi_top - it), upper half of
      // the tile first.  Its operands sit in ring slot hn % kRing.
      auto load_half = [&](int hn) {
        const int it = hn >> 1, hf = 1 - (hn & 1), slot = hn % kRing;
        const int row0 = (mi_top - it) * kTile + hf * 64;
        uint8_t* st = smem + L::ring + slot * 3 * kHalfTile;
        mbar_expect_tx(&bar_ld[slot], (SELF ? 2 : 3) * kHalfTile);
        tma_load_4d(st, &map_q, &bar_ld[slot], 0, row0, h, b);
        if (!SELF) tma_load_4d(st + kHalfTile, &map_q0, &bar_ld[slot], 0, row0, 0, b);
        tma_load_4d(st + 2 * kHalfTile, &map_do, &bar_ld[slot], 0, row0, n, 0);
      };
      auto at = [](uint64_t desc, uint32_t byte_off) { return desc + (uint64_t)(byte_off >> 4); };
      const uint64_t kK0 = smem_desc(sa + L::k0, 16, 1024);                   // K-major A of L0^T
      const uint64_t mK = smem_desc(sa + L::k, kRowTile, 1024), mK0 = smem_desc(sa + L::k0, kRowTile, 1024);
      const uint64_t mDZ = smem_desc(sa + L::dz, kRowTile, 1024), mG = smem_desc(sa + L::g, kRowTile, 1024);
      const uint64_t kRingD = smem_desc(sa + L::ring, 16, 1024);             // Q, Q0, dO half tiles as K-major B
      const uint64_t mRingD = smem_desc(sa + L::ring, kRowTile, 1024);       // the same tiles as "K rows" operands
      auto ring_off = [](int hn) { return (uint32_t)((hn % kRing) * 3 * kHalfTile); };
      auto issue_l0 = [&](int hn) {                                          // L0^T -> Z (both operands in shared memory)
        const uint32_t st = ring_off(hn);
        mbar_wait(&bar_ld[hn % kRing], (uint32_t)((hn / kRing) & 1), status, 401);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColZ, at(kK0, ks * 32), at(kRingD, st + kHalfTile + ks * 32), idesc_t, ks > 0);
        mma_commit(&bar_l0);
      };
      auto issue_s = [&](int hn) {                                           // S^T -> Y (A = K from TMEM)
        const uint32_t st = ring_off(hn);
        if (SELF) {                                                          // (otherwise issue_l0 has waited for the slot)
          mbar_wait(&bar_ld[hn % kRing], (uint32_t)((hn / kRing) & 1), status, 401);
          tc_fence_after_sync();
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColY, tmem + kColK + ks * 8, at(kRingD, st + ks * 32), idesc_t, ks > 0);
        mma_commit(&bar_s);
      };
      auto issue_dp = [&](int hn) {                                          // dP^T -> X (A = V from TMEM)
        const uint32_t st = ring_off(hn);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColX, tmem + kColV + ks * 8, at(kRingD, st + 2 * kHalfTile + ks * 32), idesc_t, ks > 0);
        mma_commit(&bar_dp);
      };
      // dV += P^T dO; dK += dz^T Q: A from TMEM, 16 queries = 8 packed columns at a stride of 16 columns
      auto issue_dv_dk = [&](int hn) {
        const uint32_t st = ring_off(hn);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDV, tmem + kColY + ks * 16, at(mRingD, st + 2 * kHalfTile + ks * 2048), idesc_acc,
                 (hn == 0 && ks == 0) ? 0u : 1u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDK, tmem + kColY + ks * 16 + 8, at(mRingD, st + ks * 2048), idesc_acc,
                 (hn == 0 && ks == 0) ? 0u : 1u);
      };
      auto issue_dk0 = [&](int hn) {                                         // dK0 += g^T Q0 (A from TMEM)
        const uint32_t st = ring_off(hn);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDK0, tmem + kColX + ks * 16, at(mRingD, st + kHalfTile + ks * 2048), idesc_acc,
                 (hn == 0 && ks == 0) ? 0u : 1u);
        mma_commit(&bar_free[hn % kRing]);                                   // every MMA reading this ring slot is issued
      };
      auto issue_dq0 = [&](int it) {                                         // dQ0 = g K0 into the shared accumulator
        mbar_wait(&bar_dqread, (uint32_t)(it & 1), status, 407);             // dQ of that tile has been read out
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(tmem + kColDQ, at(mG, ks * 2048), at(mK0, ks * 2048), idesc_dq, ks > 0);
        mma_commit(&bar_dq0);
      };

      mbar_expect_tx(&bar_kv, (SELF ? 2 : 3) * kRowTile);
      tma_load_4d(smem + L::k, &map_k, &bar_kv, 0, nj * kTile, h, b);
      tma_load_4d(smem + L::v, &map_v, &bar_kv, 0, nj * kTile, h, b);
      if (!SELF) tma_load_4d(smem + L::k0, &map_k0, &bar_kv, 0, nj * kTile, 0, b);
      for (int hn = 0; hn < kRing && hn < n_half; ++hn) load_half(hn);
      mbar_wait(&bar_setup, 0, status, 400);                   // K and V are in TMEM
      tc_fence_after_sync();
      if (!SELF) issue_l0(0);
      issue_s(0);
      issue_dp(0);

#pragma unroll 2   // the half's parity becomes a constant in each copy (-1.2 %; by six, to fix the ring slot too: +8 %)
      for (int hn = 0; hn < n_half; ++hn) {
        const int second = hn & 1, it = hn >> 1;               // second: the lower half, which completes a query tile
        const uint32_t ph = (uint32_t)(hn & 1);
        const bool more = hn + 1 < n_half;
        if (hn >= 1 && hn - 1 + kRing < n_half) {             // the slot of half hn - 1 is free once its last MMA is done
          mbar_wait(&bar_free[(hn - 1) % kRing], (uint32_t)(((hn - 1) / kRing) & 1), status, 403);
          load_half(hn - 1 + kRing);
        }
        if (!SELF) {
          mbar_wait(&bar_sel, ph, status, 402);                // L0^T read by every thread: Z takes the next half's
          tc_fence_after_sync();
          if (more) issue_l0(hn + 1);
          if (!second && it > 0) issue_dq0(it - 1);            // dQ0 of the previous tile (its dQ was read out at that tile's end)
        }
        mbar_wait(&bar_early, ph, status, 404);                // P^T (and dz^T) in place, S^T and dP^T read
        tc_fence_after_sync();
        if (SELF) {
          const uint32_t st = ring_off(hn);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)                       // dV += P^T dO; dK waits for dz + g
            mma_ts(tmem + kColDV, tmem + kColY + ks * 16, at(mRingD, st + 2 * kHalfTile + ks * 2048), idesc_acc,
                   (hn == 0 && ks == 0) ? 0u : 1u);
        } else {
          issue_dv_dk(hn);                                     // they read P^T and dz^T, which the next S^T overwrites
        }
        if (more) issue_s(hn + 1);
        if (!SELF && second) {                                 // dQ = dz K over all 128 keys
          if (it > 0) {
            mbar_wait(&bar_dq0read, (uint32_t)((it - 1) & 1), status, 405);   // dQ0 of the previous tile has been read out
            tc_fence_after_sync();
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            mma_ss(tmem + kColDQ, at(mDZ, ks * 2048), at(mK, ks * 2048), idesc_dq, ks > 0);
          mma_commit(&bar_dq);
        }
        mbar_wait(&bar_g, ph, status, 406);                    // g^T and the g half written (one head per selector: dz + g)
        tc_fence_after_sync();
        if (SELF) {
          const uint32_t st = ring_off(hn);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)                       // dK += (dz + g)^T Q, A from TMEM (this thread's X columns)
            mma_ts(tmem + kColDK, tmem + kColX + ks * 16, at(mRingD, st + ks * 2048), idesc_acc,
                   (hn == 0 && ks == 0) ? 0u : 1u);
          mma_commit(&bar_free[hn % kRing]);
        } else {
          issue_dk0(hn);                                       // it reads g^T, which the next dP^T overwrites
        }
        if (more) issue_dp(hn + 1);
        if (SELF && second) {                                  // dQ = (dz + g) K over all 128 keys
          if (it > 0) {
            mbar_wait(&bar_dqread, (uint32_t)((it - 1) & 1), status, 407);    // dQ of the previous tile has been read out
            tc_fence_after_sync();
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            mma_ss(tmem + kColDQ, at(mDZ, ks * 2048), at(mK, ks * 2048), idesc_dq, ks > 0);
          mma_commit(&bar_dq);
        }
      }
      if (!SELF) issue_dq0(n_iter - 1);
      mma_commit(&bar_fin);
    }
    __syncwarp();
  } else {
    // ======================================= arithmetic warps ============================================
    const int row = tid & 127, wg = tid >> 7;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // a warp reaches lanes 32 (warp % 4) ..
    const int j = nj * kTile + row;
    float dz_state = 0.f;            // sum of dz over the queries already visited (later queries), this key

    Ctx ctx;
    ctx.dz_tile = smem + L::dz;
    ctx.g_tile = smem + L::g;
    ctx.tmem = tmem;
    ctx.lane_base = lane_base;
    ctx.row = row;
    ctx.wg = wg;
    ctx.selectable = (j >= exempt);
    ctx.c1 = scale * kLog2e;
    ctx.lse_s = lse_s;
    ctx.dbar_s = dbar_s;
    ctx.sel_tot = sel_tot;
    ctx.dz_tot = dz_tot;
    ctx.status = status;

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
    float next_lse = fetch_lse(mi_top), next_dbar = fetch_dbar(mi_top), next_carry = fetch_carry(mi_top);

    // K and V rows from their landing tiles into TMEM as bf16 pairs (A operands of the score products); warpgroup
    // wg moves 16 of the 64 d columns = two 16-byte chunks = 8 packed columns of each matrix
    mbar_wait(&bar_kv, 0, status, 409);
    {
      const int offs[2] = {L::k, L::v};
      const uint32_t cols[2] = {kColK, kColV};
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        uint32_t w8[8];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint4 v4 = *reinterpret_cast<const uint4*>(smem + offs[m] + swz_off(row, wg * 2 + c));
          w8[4 * c] = v4.x; w8[4 * c + 1] = v4.y; w8[4 * c + 2] = v4.z; w8[4 * c + 3] = v4.w;
        }
        tmem_st8(lane_base + cols[m] + wg * 8, w8);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_setup);
    }

    // The shared accumulator (here the lane is a QUERY row, columns are d) -> scaled fp32 staging tile -> TMA reduce-add.
    auto read_out = [&](uint64_t* done_bar, const CUtensorMap* map, int i0, int row_index) {
      const int c0 = wg * kChunk;
      uint32_t r[16];
      tmem_ld16(lane_base + kColDQ + c0, r);
      tmem_ld_wait();
      uint8_t* sq = smem + L::out + (wg >> 1) * kRowTile;     // [128 queries][32 floats] tiles, 128-byte swizzle
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<float4*>(sq + swz_off(row, (wg & 1) * 4 + c)) =
            make_float4(__uint_as_float(r[4 * c]) * scale, __uint_as_float(r[4 * c + 1]) * scale,
                        __uint_as_float(r[4 * c + 2]) * scale, __uint_as_float(r[4 * c + 3]) * scale);
      fence_async_smem();
      tc_fence_before_sync();
      named_barrier(kComputeBarrier, kComputeThreads);
      if (tid == 0) {
        mbar_arrive(done_bar);                                // the accumulator may be overwritten
        tma_reduce_add_4d(map, smem + L::out, 0, i0, row_index, 0);
        tma_reduce_add_4d(map, smem + L::out + kRowTile, 32, i0, row_index, 0);
        bulk_commit();
      }
    };

    HalfState st;
    // One query tile.  The diagonal tile (the only one that needs the causal mask inside the tile) is the LAST of the
    // walk, so the loop runs the unmasked form only and the masked form follows it once.
    auto tile = [&](int it, auto diag_tag) {
      constexpr bool kDiag = decltype(diag_tag)::value;
      const int mi = mi_top - it;
      const int i0 = mi * kTile;
      const uint32_t ph = (uint32_t)(it & 1);
      if (tid < kTile) {
        lse_s[tid] = -next_lse;                                // negated: both enter packed adds directly
        dbar_s[tid] = -next_dbar;
      }
      const float cnl = next_carry * kLog2e;
      if (it + 1 < n_iter) {
        next_lse = fetch_lse(mi - 1);
        next_dbar = fetch_dbar(mi - 1);
        next_carry = fetch_carry(mi - 1);
      }
      float sel_state = 0.f;         // selection of the tile's queries already visited, this key (raw logit units)

#pragma unroll   // both halves inline: with the masked form out of the loop this is worth 4.5 % (7 % for one head per selector)
      for (int hf = 1; hf >= 0; --hf) {
        const uint32_t hp = (uint32_t)(1 - hf);               // parity of this half's barrier phases
        // the staging tile is written next at the read-out that follows this half's dz pass (dQ0 of the previous
        // tile after the upper half, dQ of this tile after the lower half): its last reduce-add must have read it
        const bool drain = SELF ? (hf == 1 && it > 0) : ((it > 0) || (hf == 0));
        half_scores<kDiag, SELF>(ctx, hf, hp, cnl, sel_state, st, &bar_l0, &bar_sel, &bar_s, &bar_dp, &bar_early, drain, true);
        if (hf == 1 && it > 0) {                               // the previous tile's last product, issued a half-tile ago:
          if (SELF) {                                          //   dQ = (dz + g) K, or dQ0 = g K0
            mbar_wait(&bar_dq, (uint32_t)((it - 1) & 1), status, 413);
            tc_fence_after_sync();
            read_out(&bar_dqread, &map_dq, i0 + kTile, n);
          } else {
            mbar_wait(&bar_dq0, (uint32_t)((it - 1) & 1), status, 412);
            tc_fence_after_sync();
            read_out(&bar_dq0read, &map_dq0, i0 + kTile, b);
          }
        }
        half_gate<SELF>(ctx, hf, dz_state, st, true);
        fence_async_smem();                                    // g half tile -> visible to the MMAs
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_g);
      }
      if (!SELF) {
        mbar_wait(&bar_dq, ph, status, 413);                   // dQ of this tile, issued before the last g pass
        tc_fence_after_sync();
        read_out(&bar_dqread, &map_dq, i0, n);
      }
    };
    for (int it = 0; it + 1 < n_iter; ++it) tile(it, std::false_type{});
    tile(n_iter - 1, std::true_type{});
    {                                                          // the first query tile's last product, visited last
      mbar_wait(SELF ? &bar_dq : &bar_dq0, (uint32_t)((n_iter - 1) & 1), status, 414);
      tc_fence_after_sync();
      if (tid == 0) bulk_wait_read();
      named_barrier(kComputeBarrier, kComputeThreads);
      if (SELF) read_out(&bar_dqread, &map_dq, nj * kTile, n);
      else read_out(&bar_dq0read, &map_dq0, nj * kTile, b);
    }

    // ---- epilogue: dV, dK (this head) and this head's share of dK0 ------------------------------------------
    mbar_wait(&bar_fin, 0, status, 415);
    tc_fence_after_sync();
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

int backward(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_bf16,
             float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  if (p.head_dim != 64) return SA_ERR_UNSUPPORTED;
  const int ntiles = (p.seq + kTile - 1) / kTile;
  const int nrows = p.batch * p.heads;
  CUtensorMap map_q, map_k, map_v, map_do, map_dq, map_dq0, map_q0, map_k0;
  int st = make_map_16bit(&map_q, p.q.ptr, 64, p.seq, p.heads, p.batch, p.q.st, p.q.sh, p.q.sb, 64);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k, p.k.ptr, 64, p.seq, p.heads, p.batch, p.k.st, p.k.sh, p.k.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_v, p.v.ptr, 64, p.seq, p.heads, p.batch, p.v.st, p.v.sh, p.v.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_do, d_out_bf16, 64, p.seq, nrows, 1, 64, (int64_t)p.seq * 64, (int64_t)nrows * p.seq * 64, 64);
  if (st != SA_OK) return st;
  st = make_map_f32_rows(&map_dq, dq_acc, p.seq, nrows);
  if (st != SA_OK) return st;
  st = make_map_f32_rows(&map_dq0, dq0, p.seq, p.batch);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_q0, p.q0.ptr, 64, p.seq, 1, p.batch, p.q0.st, 0, p.q0.sb, 64);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k0, p.k0.ptr, 64, p.seq, 1, p.batch, p.k0.st, 0, p.k0.sb, kTile);
  if (st != SA_OK) return st;
  WaitCtx status;
  st = wait_ctx(&status);
  if (st != SA_OK) return st;
  const int smem = Smem::total + 1024;
  const bool self = (p.heads == 1) && !p.external_selector;   // one head per selector: the selection logits are the head's own
  const uint8_t* alive = static_cast<const uint8_t*>(p.tile_table);
  auto launch = [&](auto kernel) -> int {
    SA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    ProfileScope prof(SA_KERNEL_TC_BACKWARD, s);
    count_launch();
    kernel<<<(unsigned)ntiles * nrows, kThreads, smem, s>>>(
        map_q, map_k, map_v, map_do, map_dq, map_dq0, map_q0, map_k0, lse2, carry, dbar, dk_acc, dk0,
        static_cast<__nv_bfloat16*>(dv), p.heads, p.seq, ntiles, p.exempt, p.scale, status, p.dv_rows, alive);
    return SA_OK;
  };
  if (alive != nullptr) st = self ? launch(backward_kernel<true, true>) : launch(backward_kernel<false, true>);
  else st = self ? launch(backward_kernel<true, false>) : launch(backward_kernel<false, false>);
  if (st != SA_OK) return st;
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
