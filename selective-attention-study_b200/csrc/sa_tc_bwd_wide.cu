// Tensor-core engine, backward at head_dim 128 (sm_100a: TMA loads, tcgen05 MMAs, fp32 accumulators in TMEM).
//
// The scheme is the one of sa_tc_bwd.cu (one CTA per 128-key tile of one head, query tiles walked last to first in
// 64-query halves, score-shaped tiles transposed with KEYS on the TMEM lanes, every product issued one arithmetic pass
// before it is needed, P^T / dz^T / g^T consumed from TMEM).  At head_dim 128 the three per-key accumulators alone
// (dV, dK, dK0: 128 fp32 columns each) and the three score tiles would need 576 of the 512 TMEM columns, so TWO CTAs
// share a (head, key tile), one per 64-wide half `dh` of the head dimension:
//   * both compute the full-depth score products (8 MMAs of K = 16 each: S^T, dP^T, L0^T) and the whole arithmetic,
//   * each accumulates only its own 64 columns of dV, dK, dK0 (B operand: the `dh` box of dO, Q, Q0),
//   * the query-side gradients are computed TRANSPOSED per half, d on the lanes: dQ^T = K^T dz^T (CTA dh = 0) and
//     dQ0^T = K0^T g^T (CTA dh = 1), M = 128 = the full head dimension, N = 64 queries, K = 128 keys, so the two CTAs
//     split that work instead of repeating it, each keeps only ONE of the dz / g tiles in shared memory, and a warp's
//     read-out of one query column is 32 consecutive floats: it leaves as coalesced fp32 reductions from registers
//     (no staging tile).  One head per selector: dQ^T = K^T (dz + g)^T, the CTAs take alternate halves.
// TMEM, 512 columns: V (64, bf16 pairs, A of dP^T) | dV | dK | dK0 | Z | X | Y | dQ^T (64 each).  K stays in shared
// memory (A of S^T, and of dQ^T through its transposed view).
// Shared memory: K 32 KB, K0 32 KB, dz-or-g 32 KB, a ring of (Q, dO) half tiles (32 KB a slot: 2 slots, freed when
// dV and dK of the half are done; 3 slots for one head per selector, where dK waits for the g pass) and a ring of
// three 16 KB Q0 half tiles (live from L0^T of a half, issued a pass early, to its dK0).  V lands in the last (Q, dO)
// slot, is moved to TMEM, and the slot then joins the ring.
//
// Reference for the arithmetic: src/selective_attention/kernels.py:196-268 (one head), :271-364 (the shared
// selection-gradient products); head_dim 128 in the reference's tests: tests/test_selective_kernels.py:159-172.
#include <type_traits>

#include "sa_tc_bwd_passes.cuh"

namespace sa {
namespace tc {
namespace {

using namespace bwd;

constexpr int kOpTile = 2 * kHalfTile;   // a [64 queries][128] bf16 operand half tile: two 64-column boxes
constexpr int kRing0 = 3;                // Q0 half tiles in flight

template <bool SELF>
struct Layout {
  static constexpr int ring_qd = SELF ? 3 : 2;              // (Q, dO) slots
  static constexpr int k = 0;                               // [128 keys][128] as two 64-column boxes, stationary
  static constexpr int k0 = k + 2 * kRowTile;
  static constexpr int t = SELF ? k0 : k0 + 2 * kRowTile;   // dz or g (one head per selector: dz + g): [128 keys][2 x 64 queries]
  static constexpr int qd = t + 2 * kRowTile;               // ring_qd x (Q, dO)
  static constexpr int q0 = qd + ring_qd * 2 * kOpTile;     // kRing0 x Q0
  static constexpr int total = SELF ? q0 : q0 + kRing0 * kOpTile;
};

// TMEM columns (Z, X, Y: sa_tc_bwd_passes.cuh)
constexpr uint32_t kColV = 0, kColDV = 64, kColDK = 128, kColDK0 = 192, kColDQT = 448;

template <bool SELF, bool LIVE>   // LIVE: a table of live tiles is given (sa_tc_skip.cu)
__global__ void __launch_bounds__(kThreads, 1) backward_wide_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const __grid_constant__ CUtensorMap map_q0, const __grid_constant__ CUtensorMap map_k0,
    const float* __restrict__ lse2, const float* __restrict__ carry, const float* __restrict__ dbar,
    float* __restrict__ dq_acc, float* __restrict__ dq0, float* __restrict__ dk_acc, float* __restrict__ dk0,
    __nv_bfloat16* __restrict__ dv, int heads, int seq, int ntiles, int exempt, float scale, WaitCtx status,
    RowLayout dv_rows, const uint8_t* __restrict__ alive) {
  using L = Layout<SELF>;
  constexpr int D = 128;
  constexpr int kRingQD = L::ring_qd;
  // Consecutive CTAs: the two halves of the head dimension of one (row, key tile), then the row's next key tile, so
  // the CTAs resident at one time walk the same query tiles and share them through L2.
  const int dh = (int)(blockIdx.x & 1);
  int n, nj;
  tile_of_block(blockIdx.x >> 1, ntiles, (gridDim.x >> 1) / ntiles, LIVE, n, nj);
  const int b = n / heads, h = n - b * heads;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // bar_l0 .. bar_g and bar_dq complete one phase per half (bar_dq, one head per selector: per half this CTA owns);
  // each side reaches its next wait on one of them only after the other side has consumed the previous phase.
  __shared__ uint64_t bar_kv, bar_setup, bar_ldqd[3], bar_freeqd[3], bar_ld0[kRing0], bar_free0[kRing0], bar_l0, bar_s,
      bar_dp, bar_sel, bar_early, bar_g, bar_dq, bar_fin;
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
    for (int u = 0; u < 3; ++u) {
      mbar_init(&bar_ldqd[u], 1);
      mbar_init(&bar_freeqd[u], 1);
    }
    for (int u = 0; u < kRing0; ++u) {
      mbar_init(&bar_ld0[u], 1);
      mbar_init(&bar_free0[u], 1);
    }
    mbar_init(&bar_setup, kComputeThreads / 32);
    mbar_init(&bar_l0, 1);
    mbar_init(&bar_s, 1);
    mbar_init(&bar_dp, 1);
    mbar_init(&bar_sel, 1);
    mbar_init(&bar_early, 1);
    mbar_init(&bar_g, kComputeThreads / 32);
    mbar_init(&bar_dq, 1);
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
  // One head per selector: this CTA computes dQ^T of the halves whose index (counted from the last) has its parity.
  auto owns = [&](int hn) { return !SELF || ((hn & 1) == dh); };

  if (warp == kComputeThreads / 32) {
    // =============================== control warp: TMA loads and MMA issue ===============================
    if (lane == 0) {
      const uint32_t idesc_t = instr_desc_bf16(128, 64, false, false);     // keys x 64 queries, K = d
      const uint32_t idesc_acc = instr_desc_bf16(128, 64, false, true);    // A K-major (keys x queries), B MN-major
      const uint32_t idesc_dq = instr_desc_bf16(128, 64, true, true);      // A MN-major (d x keys), B MN-major (keys x queries)
      // Half index hn counts from the last query half: tile it = hn / 2 (query tile mi_top - it), upper half of
      // the tile first.
      auto row_of = [&](int hn) { return (mi_top - (hn >> 1)) * kTile + (1 - (hn & 1)) * 64; };
      auto qd_off = [](int hn) { return (uint32_t)(L::qd + (hn % kRingQD) * 2 * kOpTile); };
      auto q0_off = [](int hn) { return (uint32_t)(L::q0 + (hn % kRing0) * kOpTile); };
      auto load_qd = [&](int hn) {
        const int row0 = row_of(hn), slot = hn % kRingQD;
        uint8_t* st = smem + qd_off(hn);
        mbar_expect_tx(&bar_ldqd[slot], 2 * kOpTile);
        tma_load_4d(st, &map_q, &bar_ldqd[slot], 0, row0, h, b);
        tma_load_4d(st + kHalfTile, &map_q, &bar_ldqd[slot], 64, row0, h, b);
        tma_load_4d(st + kOpTile, &map_do, &bar_ldqd[slot], 0, row0, n, 0);
        tma_load_4d(st + kOpTile + kHalfTile, &map_do, &bar_ldqd[slot], 64, row0, n, 0);
      };
      auto load_q0 = [&](int hn) {
        const int row0 = row_of(hn), slot = hn % kRing0;
        uint8_t* st = smem + q0_off(hn);
        mbar_expect_tx(&bar_ld0[slot], kOpTile);
        tma_load_4d(st, &map_q0, &bar_ld0[slot], 0, row0, 0, b);
        tma_load_4d(st + kHalfTile, &map_q0, &bar_ld0[slot], 64, row0, 0, b);
      };
      auto at = [](uint64_t desc, uint32_t byte_off) { return desc + (uint64_t)(byte_off >> 4); };
      const uint64_t kBase = smem_desc(sa, 16, 1024);                      // K-major views (rows = M or N index)
      const uint64_t mBase = smem_desc(sa, kRowTile, 1024);                // MN-major views (rows = K index)
      // byte offset of K step ks (16 of the 128 d) inside a K-major operand made of two 64-column boxes
      auto kstep = [](int ks, int box_bytes) { return (uint32_t)((ks >> 2) * box_bytes + (ks & 3) * 32); };

      auto issue_l0 = [&](int hn) {                                        // L0^T -> Z
        mbar_wait(&bar_ld0[hn % kRing0], (uint32_t)((hn / kRing0) & 1), status, 421);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(tmem + kColZ, at(kBase, L::k0 + kstep(ks, kRowTile)), at(kBase, q0_off(hn) + kstep(ks, kHalfTile)),
                 idesc_t, ks > 0);
        mma_commit(&bar_l0);
      };
      auto issue_s = [&](int hn) {                                         // S^T -> Y
        mbar_wait(&bar_ldqd[hn % kRingQD], (uint32_t)((hn / kRingQD) & 1), status, 422);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(tmem + kColY, at(kBase, L::k + kstep(ks, kRowTile)), at(kBase, qd_off(hn) + kstep(ks, kHalfTile)),
                 idesc_t, ks > 0);
        mma_commit(&bar_s);
      };
      auto issue_dp = [&](int hn) {                                        // dP^T -> X (A = V from TMEM)
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ts(tmem + kColX, tmem + kColV + ks * 8, at(kBase, qd_off(hn) + kOpTile + kstep(ks, kHalfTile)), idesc_t,
                 ks > 0);
        mma_commit(&bar_dp);
      };
      // The per-key accumulators take this CTA's 64 columns of the query-side operand: box dh of its half tile.
      auto issue_dv = [&](int hn) {                                        // dV += P^T dO
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDV, tmem + kColY + ks * 16, at(mBase, qd_off(hn) + kOpTile + dh * kHalfTile + ks * 2048),
                 idesc_acc, (hn == 0 && ks == 0) ? 0u : 1u);
      };
      auto issue_dk = [&](int hn, uint32_t a_col) {                        // dK += dz^T Q (or (dz + g)^T Q)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDK, tmem + a_col + ks * 16, at(mBase, qd_off(hn) + dh * kHalfTile + ks * 2048), idesc_acc,
                 (hn == 0 && ks == 0) ? 0u : 1u);
      };
      auto issue_dk0 = [&](int hn) {                                       // dK0 += g^T Q0
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ts(tmem + kColDK0, tmem + kColX + ks * 16, at(mBase, q0_off(hn) + dh * kHalfTile + ks * 2048), idesc_acc,
                 (hn == 0 && ks == 0) ? 0u : 1u);
        mma_commit(&bar_free0[hn % kRing0]);
      };
      // dQ^T (d x 64 queries) = K^T dz^T, or dQ0^T = K0^T g^T: A = the stationary key-side tile seen transposed,
      // B = the half tile the arithmetic warps have just written
      auto issue_dqt = [&](int hn) {
        const uint32_t a_off = (SELF || dh == 0) ? L::k : L::k0;
        const uint32_t b_off = L::t + (1 - (hn & 1)) * kRowTile;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(tmem + kColDQT, at(mBase, a_off + ks * 2048), at(mBase, b_off + ks * 2048), idesc_dq, ks > 0);
        mma_commit(&bar_dq);
      };

      // K, K0 to their places; V into the last (Q, dO) slot, from where the arithmetic warps move it to TMEM
      mbar_expect_tx(&bar_kv, (SELF ? 4 : 6) * kRowTile);
      tma_load_4d(smem + L::k, &map_k, &bar_kv, 0, nj * kTile, h, b);
      tma_load_4d(smem + L::k + kRowTile, &map_k, &bar_kv, 64, nj * kTile, h, b);
      uint8_t* v_land = smem + L::qd + (kRingQD - 1) * 2 * kOpTile;
      tma_load_4d(v_land, &map_v, &bar_kv, 0, nj * kTile, h, b);
      tma_load_4d(v_land + kRowTile, &map_v, &bar_kv, 64, nj * kTile, h, b);
      if (!SELF) {
        tma_load_4d(smem + L::k0, &map_k0, &bar_kv, 0, nj * kTile, 0, b);
        tma_load_4d(smem + L::k0 + kRowTile, &map_k0, &bar_kv, 64, nj * kTile, 0, b);
        for (int hn = 0; hn < kRing0 && hn < n_half; ++hn) load_q0(hn);
      }
      for (int hn = 0; hn < kRingQD - 1 && hn < n_half; ++hn) load_qd(hn);
      mbar_wait(&bar_setup, 0, status, 420);                   // V is in TMEM, its landing slot is free
      tc_fence_after_sync();
      if (kRingQD - 1 < n_half) load_qd(kRingQD - 1);
      if (!SELF) issue_l0(0);
      issue_s(0);
      issue_dp(0);

      for (int hn = 0; hn < n_half; ++hn) {
        const uint32_t ph = (uint32_t)(hn & 1);
        const bool more = hn + 1 < n_half;
        if (hn >= 1) {                                         // refill the slots of half hn - 1 once its last MMAs are done
          if (!SELF && hn - 1 + kRing0 < n_half) {
            mbar_wait(&bar_free0[(hn - 1) % kRing0], (uint32_t)(((hn - 1) / kRing0) & 1), status, 423);
            load_q0(hn - 1 + kRing0);
          }
          if (hn - 1 + kRingQD < n_half) {
            mbar_wait(&bar_freeqd[(hn - 1) % kRingQD], (uint32_t)(((hn - 1) / kRingQD) & 1), status, 424);
            load_qd(hn - 1 + kRingQD);
          }
        }
        if (!SELF) {
          mbar_wait(&bar_sel, ph, status, 425);                // L0^T read by every thread: Z takes the next half's
          tc_fence_after_sync();
          if (more) issue_l0(hn + 1);
        }
        mbar_wait(&bar_early, ph, status, 426);                // P^T (and dz^T) in place, S^T and dP^T read
        tc_fence_after_sync();
        issue_dv(hn);
        if (!SELF) {
          issue_dk(hn, kColY + 8);
          mma_commit(&bar_freeqd[hn % kRingQD]);
        }
        if (more) issue_s(hn + 1);
        mbar_wait(&bar_g, ph, status, 427);                    // g^T written (one head per selector: (dz + g)^T)
        tc_fence_after_sync();
        if (SELF) {
          issue_dk(hn, kColX);
          mma_commit(&bar_freeqd[hn % kRingQD]);
        } else {
          issue_dk0(hn);
        }
        if (more) issue_dp(hn + 1);
        if (owns(hn)) issue_dqt(hn);                           // its accumulator was read out before bar_g was reached
      }
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
    ctx.dz_tile = smem + L::t;
    ctx.g_tile = smem + L::t;
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

    // V rows from the landing tile into TMEM as bf16 pairs; warpgroup wg moves 32 of the 128 d columns = four
    // 16-byte chunks of box wg / 2 = 16 packed columns
    mbar_wait(&bar_kv, 0, status, 428);
    {
      const uint8_t* v_land = smem + L::qd + (kRingQD - 1) * 2 * kOpTile + (wg >> 1) * kRowTile;
      uint32_t w16[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v4 = *reinterpret_cast<const uint4*>(v_land + swz_off(row, (wg & 1) * 4 + c));
        w16[4 * c] = v4.x; w16[4 * c + 1] = v4.y; w16[4 * c + 2] = v4.z; w16[4 * c + 3] = v4.w;
      }
      tmem_st16(lane_base + kColV + wg * 16, w16);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_setup);
    }

    // dQ^T (or dQ0^T) of one half: the lane is d, this warpgroup's 16 columns are queries; one query column of a warp
    // is 32 consecutive floats of the fp32 gradient row
    float* const grad_rows = (SELF || dh == 0) ? dq_acc + (int64_t)n * seq * D : dq0 + (int64_t)b * seq * D;
    auto read_out = [&](int hn) {
      const int i_first = (mi_top - (hn >> 1)) * kTile + (1 - (hn & 1)) * 64 + wg * kChunk;
      uint32_t r[16];
      tmem_ld16(lane_base + kColDQT + wg * kChunk, r);
      tmem_ld_wait();
      float* dst = grad_rows + (int64_t)i_first * D + row;
#pragma unroll
      for (int e = 0; e < 16; ++e)
        if (i_first + e < seq) atomicAdd(dst + e * D, __uint_as_float(r[e]) * scale);
    };

    HalfState st;
    // One query tile.  The diagonal tile (the only one that needs the causal mask inside the tile) is the LAST of the
    // walk, so the loop runs the unmasked form only and the masked form follows it once.
    auto tile = [&](int it, auto diag_tag) {
      constexpr bool kDiag = decltype(diag_tag)::value;
      const int mi = mi_top - it;
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

#pragma unroll(SELF ? 2 : 1)   // both halves inline for one head per selector (-2.5 %); no gain with a shared selector
      for (int hf = 1; hf >= 0; --hf) {
        const int hn = 2 * it + (1 - hf);
        const uint32_t hp = (uint32_t)(1 - hf);               // parity of this half's barrier phases
        const bool keep_dz = !SELF && dh == 0;
        const bool keep_g = SELF ? owns(hn) : (dh == 1);
        half_scores<kDiag, SELF>(ctx, hf, hp, cnl, sel_state, st, &bar_l0, &bar_sel, &bar_s, &bar_dp, &bar_early, false, keep_dz);
        if (hn > 0 && owns(hn - 1)) {                          // the previous half's transposed gradient, issued a pass ago
          const int k = SELF ? ((hn - 1) >> 1) : (hn - 1);
          mbar_wait(&bar_dq, (uint32_t)(k & 1), status, 429);
          tc_fence_after_sync();
          read_out(hn - 1);
        }
        half_gate<SELF>(ctx, hf, dz_state, st, keep_g);
        fence_async_smem();                                    // the half tile in shared memory -> visible to the MMAs
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_g);
      }
    };
    for (int it = 0; it + 1 < n_iter; ++it) tile(it, std::false_type{});
    tile(n_iter - 1, std::true_type{});
    if (owns(n_half - 1)) {                                    // the last half's transposed gradient
      const int k = SELF ? ((n_half - 1) >> 1) : (n_half - 1);
      mbar_wait(&bar_dq, (uint32_t)(k & 1), status, 430);
      tc_fence_after_sync();
      read_out(n_half - 1);
    }

    // ---- epilogue: this CTA's 64 columns of dV, dK (this head) and of this head's share of dK0 ----------------
    mbar_wait(&bar_fin, 0, status, 431);
    tc_fence_after_sync();
    {
      const int c0 = wg * kChunk;
      __nv_bfloat16* dv_row = dv + dv_rows.at(b, h, j) + dh * 64 + c0;
      float* dk_row = dk_acc + ((int64_t)n * seq + j) * D + dh * 64 + c0;
      float* dk0_row = dk0 + ((int64_t)b * seq + j) * D + dh * 64 + c0;
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
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

int backward_wide(const Problem& p, const float* lse2, const float* carry, const float* dbar, const void* d_out_bf16,
                  float* dq_acc, float* dk_acc, float* dq0, float* dk0, void* dv, cudaStream_t s) {
  if (p.head_dim != 128) return SA_ERR_UNSUPPORTED;
  const int ntiles = (p.seq + kTile - 1) / kTile;
  const int nrows = p.batch * p.heads;
  CUtensorMap map_q, map_k, map_v, map_do, map_q0, map_k0;
  int st = make_map_16bit(&map_q, p.q.ptr, 128, p.seq, p.heads, p.batch, p.q.st, p.q.sh, p.q.sb, 64);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k, p.k.ptr, 128, p.seq, p.heads, p.batch, p.k.st, p.k.sh, p.k.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_v, p.v.ptr, 128, p.seq, p.heads, p.batch, p.v.st, p.v.sh, p.v.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_do, d_out_bf16, 128, p.seq, nrows, 1, 128, (int64_t)p.seq * 128, (int64_t)nrows * p.seq * 128, 64);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_q0, p.q0.ptr, 128, p.seq, 1, p.batch, p.q0.st, 0, p.q0.sb, 64);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k0, p.k0.ptr, 128, p.seq, 1, p.batch, p.k0.st, 0, p.k0.sb, kTile);
  if (st != SA_OK) return st;
  WaitCtx status;
  st = wait_ctx(&status);
  if (st != SA_OK) return st;
  const bool self = (p.heads == 1) && !p.external_selector;   // one head per selector: the selection logits are the head's own
  const int smem = (self ? Layout<true>::total : Layout<false>::total) + 1024;
  const uint8_t* alive = static_cast<const uint8_t*>(p.tile_table);
  const unsigned grid = 2u * (unsigned)ntiles * (unsigned)nrows;
  auto launch = [&](auto kernel) -> int {
    SA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    ProfileScope prof(SA_KERNEL_TC_BACKWARD, s);
    count_launch();
    kernel<<<grid, kThreads, smem, s>>>(map_q, map_k, map_v, map_do, map_q0, map_k0, lse2, carry, dbar, dq_acc, dq0, dk_acc,
                                        dk0, static_cast<__nv_bfloat16*>(dv), p.heads, p.seq, ntiles, p.exempt, p.scale,
                                        status, p.dv_rows, alive);
    return SA_OK;
  };
  if (alive != nullptr) st = self ? launch(backward_wide_kernel<true, true>) : launch(backward_wide_kernel<false, true>);
  else st = self ? launch(backward_wide_kernel<true, false>) : launch(backward_wide_kernel<false, false>);
  if (st != SA_OK) return st;
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
