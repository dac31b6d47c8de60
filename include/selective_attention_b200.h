/*
 * selective_attention_b200.h — C ABI of the B200 (sm_100a) Selective Attention operator.
 *
 * The reference project (Royer-Research-Labs/Selective-Attention-Study) has no FFI: its operator is a
 * Python module of Triton kernels.  This library replaces what that module launches on the device;
 * the Python host wrapper (selective_attention_b200/kernels.py) keeps the reference's Python
 * signatures and calls these entry points through ctypes.  Each declaration names the reference code
 * it replaces (paths are relative to the reference project).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host; the library never allocates
 *     device memory and never frees any: all outputs and scratch come from the caller (its only
 *     allocation is one page of pinned host memory per device for the timeout flag, see sa_device_status);
 *   - q, k, v are (batch, heads, seq, head_dim) with arbitrary batch/head/token strides (in elements)
 *     and a contiguous innermost axis; head 0 of every sequence supplies the selection (the per-head
 *     variant reshapes every head into its own one-head sequence, as the reference does);
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it;
 *   - the return value is 0 (SA_OK) or one of the SA_ERR_* codes; sa_status_string() names it.
 */
#ifndef SELECTIVE_ATTENTION_B200_H
#define SELECTIVE_ATTENTION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum sa_status {
  SA_OK = 0,
  SA_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive size, bad enum, struct size mismatch       */
  SA_ERR_UNSUPPORTED = 2,    /* shape / dtype / engine combination the selected engine cannot run     */
  SA_ERR_ALIGNMENT = 3,      /* a pointer or stride violates the engine's alignment rule              */
  SA_ERR_WORKSPACE = 4,      /* workspace smaller than sa_*_workspace_bytes() reports                 */
  SA_ERR_CUDA = 5,           /* a CUDA runtime / driver call failed; sa_last_cuda_error() has the code */
  SA_ERR_DEVICE_TIMEOUT = 6, /* a bounded device-side wait ran out (status word set by a kernel)      */
  SA_ERR_TOO_LARGE = 7       /* problem exceeds a fixed capacity (static-scratch entry point)         */
};

enum sa_dtype { SA_F32 = 0, SA_BF16 = 1, SA_F16 = 2 };

/* SA_ENGINE_SIMT   : fp32 FFMA arithmetic on CUDA cores, exact ("ieee") products; any supported dtype,
 *                    head_dim 16/32/64/128, any seq >= 1; carry checkpoints every 32 queries.
 * SA_ENGINE_TCGEN05: bf16 operands (dtype SA_BF16 only) on the tcgen05 tensor cores with fp32 TMEM
 *                    accumulators, fed by TMA; head_dim 64 or 128; carry checkpoints every 128 queries. */
enum sa_engine { SA_ENGINE_SIMT = 0, SA_ENGINE_TCGEN05 = 1 };

enum sa_damp { SA_DAMP_NONE = 0, SA_DAMP_LINEAR = 1, SA_DAMP_SQRT = 2 };

typedef struct sa_problem {
  int32_t struct_bytes; /* sizeof(sa_problem), checked                                                */
  int32_t dtype;        /* sa_dtype of q, k, v                                                        */
  int32_t engine;       /* sa_engine                                                                  */
  int32_t batch;        /* sequences (one selector, head 0, per sequence)                             */
  int32_t heads;
  int32_t seq;          /* T >= 1                                                                     */
  int32_t head_dim;     /* 16, 32, 64 or 128                                                          */
  int32_t exempt;       /* >= 1: keys [0, exempt) are never selected (1 = <BOS> only)                 */
  int32_t damp;         /* sa_damp; forward only                                                      */
  int32_t train_len;    /* used when damp != SA_DAMP_NONE                                             */
  int64_t q_stride[3];  /* batch, head, token strides of q in elements                                */
  int64_t k_stride[3];
  int64_t v_stride[3];
} sa_problem;

/* A selector kept outside q / k: the rows whose logits make the selection when the heads of one sequence
 * are split over several calls (or GPUs).  Each call then holds some heads of the sequence in q / k / v and a
 * replica of the selection head's rows here; none of its own heads is treated as the selector.  The
 * reference has no such split (its selector is always head 0 of the tensors it is given,
 * src/selective_attention/kernels.py:123-124,160-161,216-217); this is how its operator shards by head. */
typedef struct sa_selector {
  int32_t struct_bytes;  /* sizeof(sa_selector), checked                                               */
  int32_t reserved;      /* 0                                                                          */
  const void* q0;        /* (batch, seq, head_dim), element type p->dtype, contiguous innermost axis   */
  const void* k0;
  int64_t q0_stride[2];  /* batch and token strides of q0 in elements                                  */
  int64_t k0_stride[2];
} sa_selector;

/* A tensor in the caller's own layout, for the layout-fused entry points: rows of head_dim contiguous elements
 * whose starts are given by batch / head / token strides (in elements), e.g. the (batch, seq, heads, head_dim)
 * view of a model's (batch, seq, heads * head_dim) activation, or the q / k / v slots of a fused
 * (batch, seq, 3, heads, head_dim) projection gradient. */
typedef struct sa_tensor {
  void* ptr;             /* 16-byte aligned                                                            */
  int32_t dtype;         /* sa_dtype; p->dtype unless the entry point says otherwise                   */
  int32_t reserved;      /* 0                                                                          */
  int64_t stride[3];     /* batch, head, token strides in elements; each a multiple of 16 bytes        */
} sa_tensor;

/* Library / build identification. */
int sa_abi_version(void);
const char* sa_status_string(int status);
int sa_last_cuda_error(void);              /* cudaError_t of the most recent SA_ERR_CUDA on this thread */

/* 1 when the engine is compiled into this build of the library, else 0. */
int sa_engine_available(int engine);

/* 1 when the engine runs this element type and head_dim (forward only, or forward and backward). */
int sa_engine_supports(int engine, int dtype, int head_dim, int with_backward);

/* Query rows between two checkpoints of the running selection sum for an engine (32 or 128).
 * Replaces the module constant CARRY_M (src/selective_attention/kernels.py:86-87). */
int sa_carry_rows(int engine);

/* Rows of the carry buffer for a sequence length: ceil(seq / carry_rows), plus one row holding the
 * totals for the tensor-core engine (its backward sweeps query tiles last to first and starts from
 * the checkpoint AFTER the tile).  Replaces `nb` in selective_attention_forward
 * (src/selective_attention/kernels.py:573-576). */
int sa_carry_checkpoints(int engine, int seq);

/* Forward.  Replaces the two launches of selective_attention_forward
 * (src/selective_attention/kernels.py:526-605: _selective_carry :111-138 and
 * _selective_forward / _selective_forward_grouped :140-194, :366-424).
 *   out    (batch, heads, seq, head_dim) fp32, contiguous
 *   lse2   (batch, heads, seq) fp32: log2 of the softmax denominator in the log2 domain of
 *          z = (L - F) * log2(e); equals the reference's rmax + log2(rden)
 *   carry  (batch, sa_carry_checkpoints(engine, seq), seq) fp32 scratch AND saved state for the
 *          backward: row r holds, for every key, the selection received from queries < r * carry_rows
 *   total  (batch, seq) fp32: selection received from all queries ("selected_total")
 * carry needs no initialisation. */
int sa_forward(const sa_problem* p, const void* q, const void* k, const void* v,
               float* out, float* lse2, float* carry, float* total, void* stream);

/* Forward with the selector given separately (sel == NULL: identical to sa_forward).  `total` and `carry`
 * are those of the selector, so calls that share a selector produce identical copies of them. */
int sa_forward_selector(const sa_problem* p, const void* q, const void* k, const void* v,
                        const sa_selector* sel,
                        float* out, float* lse2, float* carry, float* total, void* stream);

/* The selection pass alone on the CUDA-core engine (p->engine must be SA_ENGINE_SIMT; v strides are
 * ignored): carry checkpoints every 32 queries, the layout of the reference's CARRY buffer, and the per-key
 * totals.  Replaces _selective_carry (src/selective_attention/kernels.py:111-138).  Used to hand 32-row
 * checkpoints to a consumer of the reference's aux["carry"] (scripts/investigate/history_probe.py:49-60) and
 * to the CUDA-core backward after a tensor-core forward.
 *   carry  (batch, ceil(seq / 32), seq) fp32; rows are written for keys at or before the block, the rest is
 *          left untouched (zero-fill it for the reference's layout)
 *   total  (batch, seq) fp32 */
int sa_selection_carry(const sa_problem* p, const void* q, const void* k, const sa_selector* sel,
                       float* carry, float* total, void* stream);

/* Layout-fused forward (tensor-core engine).  As sa_forward_selector, and in the same launch the output is ALSO
 * written in the operand dtype at the rows `out_lowp` names, so the caller's next GEMM reads it in place.
 * Replaces what the reference's layer does after the kernel: the `.to(v.dtype)` pass over the fp32 output
 * (src/selective_attention/mixers.py:94) and the transpose-and-copy of _merge_heads
 * (src/selective_attention/model.py:69-71).  out_lowp == NULL: identical to sa_forward_selector. */
int sa_forward_fused(const sa_problem* p, const void* q, const void* k, const void* v,
                     const sa_selector* sel,
                     float* out, const sa_tensor* out_lowp, float* lse2, float* carry, float* total,
                     void* stream);

/* Prefill continuation (tensor-core engine): the forward for a chunk of NEW tokens appended to a cache.  p->seq is
 * the total length (cached + new); q_new holds only the new queries, (batch, heads, seq - cached, head_dim) at the
 * strides of p->q_stride; k_cache / v_cache hold all p->seq keys and values at p->k_stride / p->v_stride (the new
 * tokens' rows already written); selected[b * selected_stride + j] is the selection key j has received from the
 * `cached` queries before (zero for the new keys).  Computes exactly what sa_forward computes for the last
 * seq - cached queries of the whole sequence, without the earlier queries:
 *   out, lse2  (batch, heads, seq - cached, ...) for the new queries
 *   total      (batch, seq): selection received from ALL queries so far (the cache's new `selected`)
 *   carry      (batch, sa_carry_checkpoints(engine, seq), seq) scratch
 * The reference has no such entry: its begin_cache prefills from position 0 only
 * (src/selective_attention/mixers.py:105-113) and continues token by token with step_cache (:115-130). */
int sa_prefill_extend(const sa_problem* p, int cached, const void* q_new, const void* k_cache, const void* v_cache,
                      const float* selected, int64_t selected_stride,
                      float* out, float* lse2, float* carry, float* total, void* stream);

/* Forward for callers that must not allocate.  It has no counterpart in the reference (whose forward
 * allocates its CARRY scratch with torch on every call, src/selective_attention/kernels.py:573-580).
 *
 * Who needs it: a serving process that hands its whole HBM budget to a KV-cache pool at start-up and
 * forbids allocation afterwards (an allocation can synchronise the device, fragment the pool or simply
 * fail under load), and host runtimes without an allocator binding at all (a plain C caller holding
 * only the q/k/v/out buffers it was given).  Such a caller cannot produce the `carry` buffer sa_forward
 * asks for, so this variant keeps it inside the library: a file-scope device array of
 * SA_STATIC_SCRATCH_FLOATS floats (8 MiB), which every GPU that loads the library holds until the
 * process exits.  Same kernels and same results as sa_forward; the checkpoints are not returned, so the
 * call serves inference / prefill (out, lse2 and the per-key totals), not a later sa_backward.
 *
 *   - limit: batch * sa_carry_checkpoints(engine, seq) * seq <= SA_STATIC_SCRATCH_FLOATS, else
 *     SA_ERR_TOO_LARGE and nothing is launched (e.g. one sequence up to T = 16,000 on the tensor-core
 *     engine, or batch 8 at T = 4,096);
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and caches it; make that first call during set-up, before any stream
 *     capture begins;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine (it does not create the
 *     timeout flag of sa_device_status either; it uses the flag if an earlier call made it);
 *   - all calls on a device share the one array and it keeps the previous call's contents.  Nothing in
 *     it has to start at zero (every checkpoint that is read is written first by the same call), but
 *     two calls whose kernels overlap on the GPU (different streams, or different host threads) race
 *     on it: serialise them. */
#define SA_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
size_t sa_static_scratch_floats(void);
int sa_forward_static_scratch(const sa_problem* p, const void* q, const void* k, const void* v,
                              float* out, float* lse2, float* total, void* stream);

/* Bytes of scratch sa_backward needs for this problem (0 on a bad problem). */
size_t sa_backward_workspace_bytes(const sa_problem* p);

/* Backward.  Replaces _SelectiveAttentionFn.backward (src/selective_attention/kernels.py:621-666):
 * the dbar reduction (:636), the zero fills (:638-642), _selective_backward / _selective_backward_pair
 * (:196-364) and the fold of dq0 / dk0 into head 0 with the casts (:662-666).
 *   out, lse2, carry      as produced by sa_forward for the same problem
 *   d_out                 (batch, heads, seq, head_dim) contiguous, element type d_out_dtype
 *   dq, dk, dv            (batch, heads, seq, head_dim) contiguous, element type p->dtype
 *   workspace             sa_backward_workspace_bytes(p) bytes, 256-byte aligned; contents undefined
 *                         on entry and exit */
int sa_backward(const sa_problem* p, const void* q, const void* k, const void* v,
                const float* out, const float* lse2, const float* carry,
                const void* d_out, int d_out_dtype,
                void* dq, void* dk, void* dv,
                void* workspace, size_t workspace_bytes, void* stream);

/* Backward with the selector given separately (sel == NULL: identical to sa_backward).  With a selector,
 * dq / dk hold only the heads' own gradients (nothing is folded into head 0) and the gradient that reaches
 * the selector through the history term comes back UNFOLDED and in fp32:
 *   dq0, dk0   (batch, seq, head_dim) fp32 contiguous, 16-byte aligned; zero-filled by the call, then
 *              accumulated.  They are this call's partial sums: the caller adds the dq0 / dk0 of all calls
 *              that share the selector (an all-reduce across GPUs) and adds the result to the gradient
 *              of the selection head's q / k rows.  Replaces the fold of kernels.py:662-665 for a split. */
int sa_backward_selector(const sa_problem* p, const void* q, const void* k, const void* v,
                         const sa_selector* sel,
                         const float* out, const float* lse2, const float* carry,
                         const void* d_out, int d_out_dtype,
                         void* dq, void* dk, void* dv, float* dq0, float* dk0,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Layout-fused backward (tensor-core engine).  As sa_backward_selector, with the cotangent read from, and the
 * three gradients written to, tensors in the caller's layout (gradients: element type p->dtype; the cotangent:
 * any supported element type): d_out is typically the
 * (batch, seq, heads, head_dim) view of the gradient of the merged activation, dq / dk / dv the three slots of
 * the fused projection's gradient.  Replaces the `.contiguous()` copy of the cotangent
 * (src/selective_attention/kernels.py:632-635) and the copies autograd makes to scatter dq / dk / dv back through
 * _split_heads (src/selective_attention/model.py:59-67). */
int sa_backward_fused(const sa_problem* p, const void* q, const void* k, const void* v,
                      const sa_selector* sel,
                      const float* out, const float* lse2, const float* carry,
                      const sa_tensor* d_out,
                      const sa_tensor* dq, const sa_tensor* dk, const sa_tensor* dv, float* dq0, float* dk0,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Leaving out dead tiles (tensor-core engine, bf16, head_dim 64 / 128, seq <= 131072; optional).  The history term of
 * a (query, key) pair never decreases with the query index, so for keys that many later queries have selected
 * against, whole 128 x 128 tiles of far queries have probabilities that the exponential flushes to exactly zero:
 * they add nothing to the output or to any gradient.  The reference computes every causal tile
 * (src/selective_attention/kernels.py:100-160, :196-268); with a tile table the forward decides after its selection
 * pass, from a rigorous bound (largest row norms of the q / k tiles, smallest running selection sum of the key tile,
 * a margin of 24 binades beyond the flush threshold), which tiles are dead, records the live ones in the table and
 * leaves the dead ones out; the backward of the same call is given the same table and starts each key tile's walk at
 * its last live query tile.  Results are those of the plain calls (bit-identical forward; gradients equal up to the
 * order of the fp32 reductions).  What is saved depends on the data: nothing when the selection is weak, most of the
 * tiles at long context when it is strong.
 *   sa_tile_table_bytes     size of the table for a problem; 0 when leaving out tiles is not offered for it.
 *   sa_forward_live_tiles   sa_forward_fused plus the table (256-byte aligned device memory; contents undefined on
 *                           entry; NULL: identical to sa_forward_fused).
 *   sa_backward_live_tiles  sa_backward_fused plus the table the forward filled (NULL: identical to it).
 *   sa_prefill_extend_live_tiles  sa_prefill_extend plus a table sized for the problem it is given (seq = cached + new
 *                           tokens): a long prompt prefilled in chunks skips the dead part of the cache. */
size_t sa_tile_table_bytes(const sa_problem* p);
int sa_forward_live_tiles(const sa_problem* p, const void* q, const void* k, const void* v,
                          const sa_selector* sel,
                          float* out, const sa_tensor* out_lowp, float* lse2, float* carry, float* total,
                          void* tile_table, size_t tile_table_bytes, void* stream);
int sa_prefill_extend_live_tiles(const sa_problem* p, int cached, const void* q_new, const void* k_cache,
                                 const void* v_cache, const float* selected, int64_t selected_stride,
                                 float* out, float* lse2, float* carry, float* total,
                                 void* tile_table, size_t tile_table_bytes, void* stream);
int sa_backward_live_tiles(const sa_problem* p, const void* q, const void* k, const void* v,
                           const sa_selector* sel,
                           const float* out, const float* lse2, const float* carry,
                           const sa_tensor* d_out,
                           const sa_tensor* dq, const sa_tensor* dk, const sa_tensor* dv, float* dq0, float* dk0,
                           void* workspace, size_t workspace_bytes, const void* tile_table, void* stream);

/* Bytes of scratch sa_decode_step needs: per-split partial sums, the step's new selection values and the
 * tickets with which the last CTA of a row / key range is found.  Contents undefined on entry and exit; two
 * steps in flight at once (different streams) need separate workspaces. */
size_t sa_decode_workspace_bytes(int batch, int heads, int groups, int length, int head_dim);

/* One cached decode step.  Replaces the PyTorch ops of SelectiveAttention.step_cache
 * (src/selective_attention/mixers.py:115-130) and _append_kv (src/selective_attention/model.py:86-93).
 *   k_cache, v_cache (batch, heads, capacity, head_dim) contiguous, element type dtype
 *   selected         (batch, groups, capacity) fp32: selection each cached key has received so far;
 *                    updated in place AFTER y is formed
 *   q1, k1, v1       (batch, heads, head_dim) contiguous, element type dtype: the new token
 *   length           number of cached tokens BEFORE this step; k1/v1 are written at index `length`
 *   y                (batch, heads, head_dim) fp32
 *   k_cache, v_cache 16-byte aligned (they are streamed with bulk copies)
 * Heads are split in `groups` contiguous runs; the first head of a run is its selector.  The bounded waits of
 * the copy pipeline report into the word sa_device_status reads. */
int sa_decode_step(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim,
                   int exempt, const void* q1, const void* k1, const void* v1,
                   void* k_cache, void* v_cache, float* selected, float* y,
                   void* workspace, size_t workspace_bytes, void* stream);

/* The same step, leaving out the dead part of the cache (optional).  The history term of a key only grows, so in a
 * long context most keys end up with a weight below 2^-150 for every new query: they add nothing to sums of order
 * one.  With per-key norms the step first marks, from 8 bytes per key, the 64-key stages that hold a key whose bound
 *   scale log2e |q| |k_j| - log2e selected[j]  >=  (logit of the newest key) - 150
 * and streams K and V of those stages only; the heads that select stay dense (their new selection is needed for
 * every key).  The reference reads the whole cache (mixers.py:119-129).
 *   key_norms        (batch, heads, capacity) fp32: |k_j| of every cached key; the step stores the new key's.
 *                    NULL: identical to sa_decode_step. */
int sa_decode_step_live_keys(int dtype, int batch, int heads, int groups, int length, int capacity, int head_dim,
                             int exempt, const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                             float* selected, float* key_norms, float* y, void* workspace, size_t workspace_bytes,
                             void* stream);

/* Per-kernel device timing for benchmarks.  sa_profile_enable(id) makes every later launch of that
 * kernel record a CUDA event pair on its stream (id 0 disables); sa_profile_collect waits for the
 * recorded pairs, writes their durations in milliseconds (launch order) to ms_host, forgets them and
 * returns how many it wrote (-1 on error).  At most 512 launches are kept between two collects.  Not
 * thread-safe; meant for one benchmarking thread.  No counterpart in the reference (it times whole
 * steps with the host clock, scripts/bench_kernels.py:36-55). */
enum sa_kernel {
  SA_KERNEL_NONE = 0,
  SA_KERNEL_TC_COLSUM = 1,
  SA_KERNEL_TC_SCAN = 2,
  SA_KERNEL_TC_FORWARD = 3,
  SA_KERNEL_TC_BACKWARD = 4,
  SA_KERNEL_DBAR = 5,
  SA_KERNEL_DECODE = 6
};
int sa_profile_enable(int kernel_id);
int sa_profile_collect(float* ms_host, int capacity);

/* Kernels of this library launched by this process so far (all devices, all threads).  Benchmarks report the
 * difference across their timed region.  No counterpart in the reference. */
unsigned long long sa_launch_count(void);

/* Bounded device-side waits.  Every wait inside the tensor-core engine and the decode step gives up after a
 * fixed number of clock ticks (~0.2 s), records (site << 8) | 1 in a per-device word, and its kernel returns;
 * only the launch sequence that gave up is cut short.  The word is also mirrored into mapped host memory (one
 * pinned page per device, created by the first entry-point call on the device), so from then on every
 * sa_forward* / sa_backward* / sa_decode_step call on that device returns SA_ERR_DEVICE_TIMEOUT without
 * launching anything until the word is cleared.
 *   sa_device_status  reads the word (0 = no wait ever ran out on the current device); clear != 0 resets it.
 *                     It copies with cudaMemcpy on the legacy default stream: synchronise streams created
 *                     with cudaStreamNonBlocking before calling it.
 * No counterpart in the reference (Triton kernels have no such waits). */
int sa_device_status(unsigned int* value_host, int clear);

/* Makes one bounded wait run out on purpose: a single CTA waits on an mbarrier nobody arrives on, with a
 * limit of limit_kcycles * 1024 clock ticks (1 .. 100000), reports site 900 and returns.  The kernel
 * terminates by itself; nothing faults.  For testing the path above.  No counterpart in the reference. */
int sa_selftest_wait_timeout(unsigned int limit_kcycles, void* stream);

/* Known-answer test of the tcgen05 / TMA operand encodings the tensor-core engine uses.
 *   scratch  32 KiB of device memory, 1024-byte aligned
 *   result   8 floats: result[m] = largest absolute error of operand form m (0 when correct)
 * No counterpart in the reference. */
int sa_selftest_tcgen05(void* scratch, float* result, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SELECTIVE_ATTENTION_B200_H */
