// Tensor-core engine, backward (sm_100a: TMA loads, tcgen05 MMAs, fp32 accumulators in TMEM).
//
// One CTA owns one 128-key tile of one head and walks the 128-query tiles LAST TO FIRST.  All
// score-shaped tiles are computed transposed, KEYS on the TMEM lanes: S^T = K Q^T, dP^T = V dO^T,
// L0^T = K0 Q0^T, so one thread owns one key and sees that key's queries along its registers.  The
// two running sums down the query axis are then thread-local fp32 recurrences walked from the last
// query to the first:
//     F[i]  = carry_after_tile - sum_{r >= i} sel[r]          (history term rebuilt per key)
//     U[i]  = suffix + sum_{i' > i} dz[i']                      (logit gradient of later queries)
// with  P = exp2(z - lse),  dz = P (dP - dbar),  g = gate ? -U : 0.  P^T, dz^T and g^T go to shared
// memory as bf16 and feed five more MMAs per query tile:
//     dV += P^T dO    dK += dz^T Q    dK0 += g^T Q0    (accumulated in TMEM across query tiles)
//     dQ  = dz K      dQ0 = g K0                        (per query tile; added to global fp32 with red.v4)
// Reference for the arithmetic: src/selective_attention/kernels.py:196-268.
#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {
namespace {

constexpr int kTile = 128;
constexpr int kRowTile = 16384;     // bytes of a [128][64] bf16 operand tile

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

struct BwdSmem {
  static constexpr int k = 0;                       // [128 keys][64]
  static constexpr int v = k + kRowTile;
  static constexpr int k0 = v + kRowTile;
  static constexpr int q = k0 + kRowTile;           // [128 queries][64]
  static constexpr int q0 = q + kRowTile;
  static constexpr int dout = q0 + kRowTile;
  static constexpr int pt = dout + kRowTile;        // [128 keys][128 queries] as two query-half tiles
  static constexpr int dz = pt + 2 * kRowTile;
  static constexpr int g = dz + 2 * kRowTile;
  static constexpr int total = g + 2 * kRowTile;
};

// TMEM columns
constexpr uint32_t kColST = 0, kColDPT = 64, kColL0T = 128, kColDV = 192, kColDK = 256, kColDK0 = 320, kColDQ = 384,
                   kColDQ0 = 448;

// Writes 8 consecutive bf16 (query columns c0 .. c0 + 7 of key row `row`) of a [128][128] matrix kept
// as two 64-column tiles.
__device__ __forceinline__ void put8(uint8_t* base, int row, int c0, const float* x) {
  uint4 w = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
  *reinterpret_cast<uint4*>(base + (c0 >> 6) * kRowTile + swz_off(row, (c0 & 63) >> 3)) = w;
}

constexpr int kGroups = 4;                    // warpgroups per CTA; each owns 16 of a half's 64 query columns
constexpr int kChunk = 64 / kGroups;
constexpr int kThreads = 128 * kGroups;

struct HalfCtx {
  uint8_t* smem;
  uint32_t lane_base;
  int row;                 // key row of this thread inside the tile (its TMEM lane)
  int wg;                  // warpgroup: which 16-column chunk of the half
  int hf;                  // which half of the query tile
  bool selectable;         // key >= exempt
  float cnl;               // log2(e) * selection received through the END of this query tile
  float c1;                // scale * log2(e)
  const float* lse_s;
  const float* dbar_s;
  float (*sel_tot)[kTile];
  float (*dz_tot)[kTile];
};

// One 64-query half of a (key tile, query tile) pair; this thread handles 16 of its query columns for
// its key row.  The two running sums run from the last query to the first; a chunk computes them
// locally (two independent chains of 8) and picks up the totals of the chunks to its right, and the
// carried state, through shared memory.
template <bool DIAG>
__device__ __forceinline__ void process_half(const HalfCtx& c, float& sel_state, float& dz_state) {
  using L = BwdSmem;
  const int colw = c.wg * kChunk;
  const int col0 = c.hf * 64 + colw;
  uint32_t r[16];
  float negon[16], ls[16], p[16], lx[16];

  tmem_ld16(c.lane_base + kColL0T + colw, r);
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
  __syncthreads();
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
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const float t2 = fmaf(c.c1, ls[e], -(cb + c.lse_s[col0 + e]));
    p[e] = ex2(fmaf(__uint_as_float(r[e]), c.c1, t2));
    if (DIAG && (c.row > col0 + e)) p[e] = 0.f;       // key after the query
  }
  put8(c.smem + L::pt, c.row, col0, p);
  put8(c.smem + L::pt, c.row, col0 + 8, p + 8);

  tmem_ld16(c.lane_base + kColDPT + colw, r);
  tmem_ld_wait();
#pragma unroll
  for (int e = 0; e < 16; ++e) p[e] = p[e] * (__uint_as_float(r[e]) - c.dbar_s[col0 + e]);     // dz
  put8(c.smem + L::dz, c.row, col0, p);
  put8(c.smem + L::dz, c.row, col0 + 8, p + 8);

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
  __syncthreads();
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
#pragma unroll
  for (int e = 0; e < 16; ++e) lx[e] = negon[e] * (base + lx[e]);                                  // g
  put8(c.smem + L::g, c.row, col0, lx);
  put8(c.smem + L::g, c.row, col0 + 8, lx + 8);
}

__global__ void __launch_bounds__(kThreads, 1) backward_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const float* __restrict__ lse2, const float* __restrict__ carry, const float* __restrict__ dbar,
    float* __restrict__ dq_acc, float* __restrict__ dk_acc, float* __restrict__ dq0, float* __restrict__ dk0,
    __nv_bfloat16* __restrict__ dv, int heads, int seq, int ntiles, int exempt, float scale, unsigned int* status) {
  using L = BwdSmem;
  constexpr int D = 64;
  const int nrows = gridDim.x / ntiles;                  // batch * heads
  const int nj = (int)(blockIdx.x / nrows);              // key tiles with the most query tiles first
  const int n = blockIdx.x % nrows;
  const int b = n / heads, h = n - b * heads;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_kv, bar_ld, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(16) float lse_s[kTile];
  __shared__ __align__(16) float dbar_s[kTile];
  __shared__ float sel_tot[kGroups][kTile];
  __shared__ float dz_tot[kGroups][kTile];

  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = tid & 127, wg = tid >> 7;
  if (tid == 0) {
    mbar_init(&bar_kv, 1);
    mbar_init(&bar_ld, 1);
    mbar_init(&bar_mma, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // a warp reaches lanes 32 (warp % 4) ..
  const uint32_t sa = smem_u32(smem);

  auto load_queries = [&](int mi) {
    mbar_expect_tx(&bar_ld, 3 * kRowTile);
    tma_load_4d(smem + L::q, &map_q, &bar_ld, 0, mi * kTile, h, b);
    tma_load_4d(smem + L::q0, &map_q, &bar_ld, 0, mi * kTile, 0, b);
    tma_load_4d(smem + L::dout, &map_do, &bar_ld, 0, mi * kTile, n, 0);
  };
  if (tid == 0) {
    mbar_expect_tx(&bar_kv, 3 * kRowTile);
    tma_load_4d(smem + L::k, &map_k, &bar_kv, 0, nj * kTile, h, b);
    tma_load_4d(smem + L::v, &map_v, &bar_kv, 0, nj * kTile, h, b);
    tma_load_4d(smem + L::k0, &map_k, &bar_kv, 0, nj * kTile, 0, b);
    load_queries(ntiles - 1);
    mbar_wait(&bar_kv, 0, status, 400);
  }

  const uint32_t idesc_t = instr_desc_bf16(128, 64, false, false);     // keys x 64 queries, K = D
  const uint32_t idesc_acc = instr_desc_bf16(128, 64, false, true);    // A K-major (keys x queries), B MN-major
  const uint32_t idesc_dq = instr_desc_bf16(128, 64, true, true);      // A MN-major (queries x keys), B MN-major
  const int j = nj * kTile + row;
  float dz_state = 0.f;              // sum of dz over the queries already visited (later queries), this key
  uint32_t mma_phase = 0;
  int iter = 0;

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

  for (int mi = ntiles - 1; mi >= nj; --mi, ++iter) {
    const int i0 = mi * kTile;
    const bool diag = (mi == nj);
    if (tid < kTile) {
      const int i = i0 + tid;
      lse_s[tid] = (i < seq) ? lse2[(int64_t)n * seq + i] : INFINITY;     // +inf: P = 0 for padded queries
      dbar_s[tid] = (i < seq) ? dbar[(int64_t)n * seq + i] : 0.f;
    }
    ctx.cnl = (j < seq) ? carry[((int64_t)b * (ntiles + 1) + mi + 1) * seq + j] * kLog2e : 0.f;
    float sel_state = 0.f;           // selection of the tile's queries already visited, this key (raw logit units)
    __syncthreads();

    for (int hf = 1; hf >= 0; --hf) {
      if (tid == 0) {
        if (hf == 1) mbar_wait(&bar_ld, iter & 1, status, 401);
        tc_fence_after_sync();
        const uint32_t qoff = hf * 8192;                                    // rows 64 hf .. 64 hf + 63
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColL0T, smem_desc(sa + L::k0 + ks * 32, 16, 1024),
                 smem_desc(sa + L::q0 + qoff + ks * 32, 16, 1024), idesc_t, ks > 0);
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColST, smem_desc(sa + L::k + ks * 32, 16, 1024),
                 smem_desc(sa + L::q + qoff + ks * 32, 16, 1024), idesc_t, ks > 0);
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem + kColDPT, smem_desc(sa + L::v + ks * 32, 16, 1024),
                 smem_desc(sa + L::dout + qoff + ks * 32, 16, 1024), idesc_t, ks > 0);
        mma_commit(&bar_mma);
      }
      mbar_wait(&bar_mma, mma_phase, status, 402);
      mma_phase ^= 1;
      tc_fence_after_sync();
      ctx.hf = hf;
      if (diag) process_half<true>(ctx, sel_state, dz_state);
      else process_half<false>(ctx, sel_state, dz_state);
      fence_async_smem();
      tc_fence_before_sync();
      __syncthreads();
    }

    // ---- accumulating products and the per-query-tile dQ, dQ0 ----------------------------------------
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t first = (iter == 0) ? 0u : 1u;
      for (int ks = 0; ks < 8; ++ks)                                      // MN-major A: K = key index
        mma_ss(tmem + kColDQ, smem_desc(sa + L::dz + ks * 2048, kRowTile, 1024),
               smem_desc(sa + L::k + ks * 2048, kRowTile, 1024), idesc_dq, ks > 0);
      for (int ks = 0; ks < 8; ++ks)
        mma_ss(tmem + kColDQ0, smem_desc(sa + L::g + ks * 2048, kRowTile, 1024),
               smem_desc(sa + L::k0 + ks * 2048, kRowTile, 1024), idesc_dq, ks > 0);
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a_off = (ks >> 2) * kRowTile + (ks & 3) * 32;      // K-major A: K = query index
        mma_ss(tmem + kColDV, smem_desc(sa + L::pt + a_off, 16, 1024),
               smem_desc(sa + L::dout + ks * 2048, kRowTile, 1024), idesc_acc, (ks > 0) ? 1u : first);
      }
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a_off = (ks >> 2) * kRowTile + (ks & 3) * 32;
        mma_ss(tmem + kColDK, smem_desc(sa + L::dz + a_off, 16, 1024),
               smem_desc(sa + L::q + ks * 2048, kRowTile, 1024), idesc_acc, (ks > 0) ? 1u : first);
      }
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a_off = (ks >> 2) * kRowTile + (ks & 3) * 32;
        mma_ss(tmem + kColDK0, smem_desc(sa + L::g + a_off, 16, 1024),
               smem_desc(sa + L::q0 + ks * 2048, kRowTile, 1024), idesc_acc, (ks > 0) ? 1u : first);
      }
      mma_commit(&bar_mma);
    }
    mbar_wait(&bar_mma, mma_phase, status, 403);
    mma_phase ^= 1;
    tc_fence_after_sync();
    if (tid == 0 && mi > nj) load_queries(mi - 1);      // Q, Q0, dO tiles are free: every MMA reading them is done
    {
      const int i = i0 + row;                           // here the lane is a QUERY row
      const int c0 = wg * kChunk;
      float* dq_row = dq_acc + ((int64_t)n * seq + i) * D + c0;
      float* dq0_row = dq0 + ((int64_t)b * seq + i) * D + c0;
      uint32_t r[16], r0[16];
      tmem_ld16(lane_base + kColDQ + c0, r);
      tmem_ld16(lane_base + kColDQ0 + c0, r0);
      tmem_ld_wait();
      if (i < seq) {
#pragma unroll
        for (int e = 0; e < 16; e += 4) {
          red_add_v4(dq_row + e, __uint_as_float(r[e]) * scale, __uint_as_float(r[e + 1]) * scale,
                     __uint_as_float(r[e + 2]) * scale, __uint_as_float(r[e + 3]) * scale);
          red_add_v4(dq0_row + e, __uint_as_float(r0[e]) * scale, __uint_as_float(r0[e + 1]) * scale,
                     __uint_as_float(r0[e + 2]) * scale, __uint_as_float(r0[e + 3]) * scale);
        }
      }
    }
    tc_fence_before_sync();
    __syncthreads();
  }

  // ---- epilogue: dV, dK (this head) and this head's share of dK0 --------------------------------------------
  {
    const int c0 = wg * kChunk;
    __nv_bfloat16* dv_row = dv + ((int64_t)n * seq + j) * D + c0;
    float* dk_row = dk_acc + ((int64_t)n * seq + j) * D + c0;
    float* dk0_row = dk0 + ((int64_t)b * seq + j) * D + c0;
    uint32_t rv[16], rk[16], r0[16];
    tmem_ld16(lane_base + kColDV + c0, rv);
    tmem_ld16(lane_base + kColDK + c0, rk);
    tmem_ld16(lane_base + kColDK0 + c0, r0);
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
        red_add_v4(dk0_row + e, __uint_as_float(r0[e]) * scale, __uint_as_float(r0[e + 1]) * scale,
                   __uint_as_float(r0[e + 2]) * scale, __uint_as_float(r0[e + 3]) * scale);
      }
    }
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
  CUtensorMap map_q, map_k, map_v, map_do;
  int st = make_map_16bit(&map_q, p.q.ptr, 64, p.seq, p.heads, p.batch, p.q.st, p.q.sh, p.q.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_k, p.k.ptr, 64, p.seq, p.heads, p.batch, p.k.st, p.k.sh, p.k.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_v, p.v.ptr, 64, p.seq, p.heads, p.batch, p.v.st, p.v.sh, p.v.sb, kTile);
  if (st != SA_OK) return st;
  st = make_map_16bit(&map_do, d_out_bf16, 64, p.seq, nrows, 1, 64, (int64_t)p.seq * 64, (int64_t)nrows * p.seq * 64,
                      kTile);
  if (st != SA_OK) return st;
  unsigned int* status = nullptr;
  st = status_word(&status);
  if (st != SA_OK) return st;
  const int smem = BwdSmem::total + 1024;
  SA_CUDA_CHECK(cudaFuncSetAttribute(backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  {
    ProfileScope prof(SA_KERNEL_TC_BACKWARD, s);
    backward_kernel<<<(unsigned)ntiles * nrows, kThreads, smem, s>>>(
        map_q, map_k, map_v, map_do, lse2, carry, dbar, dq_acc, dk_acc, dq0, dk0, static_cast<__nv_bfloat16*>(dv),
        p.heads, p.seq, ntiles, p.exempt, p.scale, status);
  }
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
