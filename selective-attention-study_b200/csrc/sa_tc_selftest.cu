// Known-answer test of the tcgen05 / TMA building blocks the tensor-core engine is made of.
//
// Every operand form the forward and backward kernels use is exercised once on small integer data
// (exact in bf16 and in the fp32 accumulator) and compared with a CUDA-core evaluation of the same
// product inside the kernel:
//   0  A K-major (TMA tile) x B K-major (TMA tile)                      the Q K^T products
//   1  A K-major (thread-written, K = 128) x B MN-major N = 64 (TMA)    P V, dz^T Q, ...
//   2  accumulate of -A K-major x B MN-major N = 128 (thread-written)   the triangular running sum
//   3  A MN-major M = 128 (thread-written) x B MN-major N = 64 (TMA)    dz K
//   4  A from tensor memory (bf16 pairs) x B MN-major N = 64 (TMA)      P^T dO with P^T kept in TMEM
// result[m] = largest absolute difference of mode m (0 when the encoding of that form is right).
#include "sa_tc_host.cuh"
#include "sa_tc_ptx.cuh"

namespace sa {
namespace tc {

namespace {


__device__ __forceinline__ float pattern(int salt, int r, int c) {
  return (float)(((r * 7 + c * 13 + salt * 5 + (r * c) % 11) % 9) - 4);   // integers in [-4, 4]
}

__global__ void selftest_fill(__nv_bfloat16* x, __nv_bfloat16* y) {
  for (int idx = threadIdx.x + blockIdx.x * blockDim.x; idx < 128 * 64; idx += blockDim.x * gridDim.x) {
    int r = idx / 64, c = idx % 64;
    x[idx] = __float2bfloat16(pattern(1, r, c));
    y[idx] = __float2bfloat16(pattern(2, r, c));
  }
}

// Writes 8 consecutive bf16 (columns c0 .. c0 + 7 of a logical row) of a [rows][128]-wide matrix kept as
// two 64-column tiles of `tile_bytes` each.
__device__ __forceinline__ void put8(uint8_t* base, uint32_t tile_bytes, int row, int c0, const float* v) {
  uint8_t* tile = base + (c0 >> 6) * tile_bytes;
  uint4 w;
  w.x = pack_bf16(v[0], v[1]);
  w.y = pack_bf16(v[2], v[3]);
  w.z = pack_bf16(v[4], v[5]);
  w.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(tile + swz_off(row, (c0 & 63) >> 3)) = w;
}

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap map_x,
                                                       const __grid_constant__ CUtensorMap map_y,
                                                       const __nv_bfloat16* __restrict__ xg,
                                                       const __nv_bfloat16* __restrict__ yg, float* result,
                                                       WaitCtx status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* xs = smem;                 // [128][64] from TMA
  uint8_t* ys = smem + 16384;         // [128][64] from TMA
  uint8_t* as = smem + 32768;         // two tiles, thread-written
  uint8_t* bs = smem + 65536;         // two tiles, thread-written
  __shared__ uint64_t bar_tma, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ float red[128];

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar_tma, 1);
    mbar_init(&bar_mma, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes

  if (tid == 0) {
    mbar_expect_tx(&bar_tma, 2 * 16384);
    tma_load_4d(xs, &map_x, &bar_tma, 0, 0, 0, 0);
    tma_load_4d(ys, &map_y, &bar_tma, 0, 0, 0, 0);
  }
  // thread-written operands: A2[m][k] = pattern(3), B2[k][n] = pattern(4), both 128 x 128
  for (int c0 = 0; c0 < 128; c0 += 8) {
    float va[8], vb[8];
    for (int e = 0; e < 8; ++e) {
      va[e] = pattern(3, tid, c0 + e);
      vb[e] = pattern(4, tid, c0 + e);
    }
    put8(as, 16384, tid, c0, va);
    put8(bs, 16384, tid, c0, vb);
  }
  fence_async_smem();
  mbar_wait(&bar_tma, 0, status, 100);
  __syncthreads();

  uint32_t phase = 0;
  float worst[5];
  auto X = [&](int r, int c) { return __bfloat162float(xg[r * 64 + c]); };
  auto Y = [&](int r, int c) { return __bfloat162float(yg[r * 64 + c]); };
  auto A2 = [&](int r, int c) { return pattern(3, r, c); };
  auto B2 = [&](int r, int c) { return pattern(4, r, c); };
  const uint32_t xs_a = smem_u32(xs), ys_a = smem_u32(ys), as_a = smem_u32(as), bs_a = smem_u32(bs);
  uint32_t regs[32];

  // ---- mode 0: D[m][n] = sum_k X[m][k] Y[n][k], M = 128, N = 128, K = 64 --------------------------------
  if (tid == 0) {
    tc_fence_after_sync();
    const uint32_t idesc = instr_desc_bf16(128, 128, false, false);
    for (int ks = 0; ks < 4; ++ks)
      mma_ss(tmem, smem_desc(xs_a + ks * 32, 16, 1024), smem_desc(ys_a + ks * 32, 16, 1024), idesc, ks > 0);
    mma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, phase, status, 101);
  phase ^= 1;
  tc_fence_after_sync();
  worst[0] = 0.f;
  for (int c0 = 0; c0 < 128; c0 += 32) {
    tmem_ld32(lane_base + c0, regs);
    tmem_ld_wait();
    for (int e = 0; e < 32; ++e) {
      float want = 0.f;
      for (int k = 0; k < 64; ++k) want += X(tid, k) * Y(c0 + e, k);
      worst[0] = fmaxf(worst[0], fabsf(__uint_as_float(regs[e]) - want));
    }
  }
  tc_fence_before_sync();
  __syncthreads();

  // ---- mode 1: D[m][n] = sum_k A2[m][k] Y[k][n], M = 128, N = 64, K = 128; B is MN-major ------------------
  if (tid == 0) {
    tc_fence_after_sync();
    const uint32_t idesc = instr_desc_bf16(128, 64, false, true);
    for (int ks = 0; ks < 8; ++ks)
      mma_ss(tmem, smem_desc(as_a + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
             smem_desc(ys_a + ks * 2048, 16384, 1024), idesc, ks > 0);
    mma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, phase, status, 102);
  phase ^= 1;
  tc_fence_after_sync();
  worst[1] = 0.f;
  for (int c0 = 0; c0 < 64; c0 += 32) {
    tmem_ld32(lane_base + c0, regs);
    tmem_ld_wait();
    for (int e = 0; e < 32; ++e) {
      float want = 0.f;
      for (int k = 0; k < 128; ++k) want += A2(tid, k) * Y(k, c0 + e);
      worst[1] = fmaxf(worst[1], fabsf(__uint_as_float(regs[e]) - want));
    }
  }
  tc_fence_before_sync();
  __syncthreads();

  // ---- mode 2: D[m][n] = mode-0 result - sum_k A2[m][k] B2[k][n]; N = 128, B MN-major in two N halves -----
  if (tid == 0) {
    tc_fence_after_sync();
    const uint32_t idesc0 = instr_desc_bf16(128, 128, false, false);
    for (int ks = 0; ks < 4; ++ks)
      mma_ss(tmem + 128, smem_desc(xs_a + ks * 32, 16, 1024), smem_desc(ys_a + ks * 32, 16, 1024), idesc0, ks > 0);
    const uint32_t idesc = instr_desc_bf16(128, 128, false, true, /*negate_a=*/true);
    for (int ks = 0; ks < 8; ++ks)
      mma_ss(tmem + 128, smem_desc(as_a + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
             smem_desc(bs_a + ks * 2048, 16384, 1024), idesc, 1);
    mma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, phase, status, 103);
  phase ^= 1;
  tc_fence_after_sync();
  worst[2] = 0.f;
  for (int c0 = 0; c0 < 128; c0 += 32) {
    tmem_ld32(lane_base + 128 + c0, regs);
    tmem_ld_wait();
    for (int e = 0; e < 32; ++e) {
      float want = 0.f;
      for (int k = 0; k < 64; ++k) want += X(tid, k) * Y(c0 + e, k);
      for (int k = 0; k < 128; ++k) want -= A2(tid, k) * B2(k, c0 + e);
      worst[2] = fmaxf(worst[2], fabsf(__uint_as_float(regs[e]) - want));
    }
  }
  tc_fence_before_sync();
  __syncthreads();

  // ---- mode 3: D[m][n] = sum_k A2[k][m] Y[k][n]; A MN-major (stored [k][m]) M = 128, B MN-major N = 64 -----
  if (tid == 0) {
    tc_fence_after_sync();
    const uint32_t idesc = instr_desc_bf16(128, 64, true, true);
    for (int ks = 0; ks < 8; ++ks)
      mma_ss(tmem, smem_desc(as_a + ks * 2048, 16384, 1024), smem_desc(ys_a + ks * 2048, 16384, 1024), idesc, ks > 0);
    mma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, phase, status, 104);
  phase ^= 1;
  tc_fence_after_sync();
  worst[3] = 0.f;
  for (int c0 = 0; c0 < 64; c0 += 32) {
    tmem_ld32(lane_base + c0, regs);
    tmem_ld_wait();
    for (int e = 0; e < 32; ++e) {
      float want = 0.f;
      for (int k = 0; k < 128; ++k) want += A2(k, tid) * Y(k, c0 + e);
      worst[3] = fmaxf(worst[3], fabsf(__uint_as_float(regs[e]) - want));
    }
  }
  tc_fence_before_sync();
  __syncthreads();

  // ---- mode 4: A from tensor memory: A4[m][k] = pattern(5) as bf16 pairs in columns 128 .. 191 --------------
  for (int c0 = 0; c0 < 64; c0 += 32) {
    for (int e = 0; e < 32; ++e) regs[e] = pack_bf16(pattern(5, tid, 2 * (c0 + e)), pattern(5, tid, 2 * (c0 + e) + 1));
    tmem_st32(lane_base + 128 + c0, regs);
  }
  tmem_st_wait();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after_sync();
    const uint32_t idesc = instr_desc_bf16(128, 64, false, true);
    for (int ks = 0; ks < 8; ++ks)
      mma_ts(tmem, tmem + 128 + ks * 8, smem_desc(ys_a + ks * 2048, 16384, 1024), idesc, ks > 0);
    mma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, phase, status, 105);
  phase ^= 1;
  tc_fence_after_sync();
  worst[4] = 0.f;
  for (int c0 = 0; c0 < 64; c0 += 32) {
    tmem_ld32(lane_base + c0, regs);
    tmem_ld_wait();
    for (int e = 0; e < 32; ++e) {
      float want = 0.f;
      for (int k = 0; k < 128; ++k) want += pattern(5, tid, k) * Y(k, c0 + e);
      worst[4] = fmaxf(worst[4], fabsf(__uint_as_float(regs[e]) - want));
    }
  }
  tc_fence_before_sync();
  __syncthreads();

  for (int m = 0; m < 5; ++m) {
    red[tid] = worst[m];
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
      if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
      __syncthreads();
    }
    if (tid == 0) result[m] = red[0];
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

int selftest(void* scratch, float* result, cudaStream_t s) {
  __nv_bfloat16* x = static_cast<__nv_bfloat16*>(scratch);
  __nv_bfloat16* y = x + 128 * 64;
  selftest_fill<<<8, 256, 0, s>>>(x, y);
  SA_CUDA_CHECK(cudaGetLastError());
  CUtensorMap mx, my;
  int st = make_map_16bit(&mx, x, 64, 128, 1, 1, 64, 64 * 128, 64 * 128, 128);
  if (st != SA_OK) return st;
  st = make_map_16bit(&my, y, 64, 128, 1, 1, 64, 64 * 128, 64 * 128, 128);
  if (st != SA_OK) return st;
  const int smem = 98304 + 1024;
  SA_CUDA_CHECK(cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  WaitCtx status;
  st = wait_ctx(&status);
  if (st != SA_OK) return st;
  selftest_kernel<<<1, 128, smem, s>>>(mx, my, x, y, result, status);
  SA_CUDA_CHECK(cudaGetLastError());
  return SA_OK;
}

}  // namespace tc
}  // namespace sa
