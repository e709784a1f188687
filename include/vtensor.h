/*
 * libvtensor — C ABI of the B200 vTensor decode path.
 *
 * Three groups of entry points, each replacing one piece of GLakeServe:
 *   1. the VMM allocator (vmm_allocator/vmm_allocator.{h,cpp}): a pool of 2 MiB
 *      physical chunks and, per sequence slot, one contiguous virtual K range
 *      and one V range per layer that grow by mapping chunks, never by copying;
 *   2. the KV append (csrc/cache_kernels.cu reshape_and_cache);
 *   3. single-query decode attention over those ranges
 *      (csrc/attention/attention_kernels.cu paged_attention_v1 and the external
 *      flash_attn_2_cuda.fwd_kvcache call in vllm/attention/backends/xformers.py).
 *
 * Conventions: every function returns an int status (VT_OK == 0), nothing
 * throws across the boundary, handles are opaque, the caller owns q/k/v/out
 * and passes the CUDA stream explicitly (a cudaStream_t cast to void*; NULL is
 * the legacy default stream).  Kernel entry points only enqueue work; they
 * never synchronise and never allocate.  All functions are thread-safe.
 * File:line citations name the reference interface each entry point stands in
 * for (paths inside the reference project, under GLakeServe/).
 */
#ifndef VTENSOR_H_
#define VTENSOR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ------------------------------------------------------------ */
enum {
  VT_OK = 0,
  VT_ERR_INVALID = 1,      /* bad argument (null, negative, misaligned, out of range) */
  VT_ERR_DRIVER = 2,       /* a CUDA driver call failed; see vt_last_driver_error */
  VT_ERR_POOL_EMPTY = 3,   /* not enough free physical chunks */
  VT_ERR_RESERVE = 4,      /* growth would exceed the slot's reserved virtual range */
  VT_ERR_TIMEOUT = 5,      /* bounded wait for a pending growth ran out */
  VT_ERR_UNSUPPORTED = 6,  /* shape / dtype outside what the kernels implement */
  VT_ERR_CUDA = 7,         /* kernel launch or runtime call failed */
  VT_ERR_STATE = 8,        /* call not valid in the object's current state */
  VT_ERR_NO_DRIVER = 9,    /* libcuda could not be loaded (no GPU on this machine) */
  VT_ERR_KERNEL = 10,      /* a kernel reported a bounded wait that ran out */
  VT_ERR_TOO_LARGE = 11    /* problem exceeds a fixed built-in limit (scratch of vt_decode_attn_static, max_bytes of a vt_ar) */
};

/* Human-readable text for a status code (static storage). */
const char *vt_strerror(int status);
/* CUresult of the last failing driver call on the calling thread, 0 if none.
 * Replaces the reference's print-and-assert(0) (vmm_allocator.h:19-42). */
int vt_last_driver_error(void);
/* Library version string, e.g. "vtensor-b200 0.1 sm_100a". */
const char *vt_version(void);

/* ---- KV element types -------------------------------------------------- */
enum {
  VT_KV_BF16 = 0,     /* 2-byte cache elements, bit-exact copy of the inputs      */
  VT_KV_FP8_E4M3 = 1  /* 1-byte e4m3 (max 448), stored = sat(x / scale[kv_head]) */
};

/* ---- allocator --------------------------------------------------------- */
typedef struct vt_pool vt_pool;
typedef struct vt_seg vt_seg;
typedef struct vt_table vt_table;

typedef struct vt_stats {
  uint64_t chunks_total, chunks_free;
  uint64_t chunk_bytes;
  uint64_t map_calls, unmap_calls, set_access_calls; /* driver calls issued   */
  uint64_t map_ns;                                   /* wall time spent in growth (map + set-access) */
  uint64_t access_ns;                                /* of which cuMemSetAccess */
  uint64_t async_requests, async_completed, async_failed;
  uint64_t segments;
} vt_stats;

/* Routes every driver call of pools created AFTERWARDS to an in-process fake
 * (no GPU needed; addresses are synthetic).  For host-side tests only. */
int vt_use_mock_driver(int enable);
/* Mock only: make the n-th next call (1-based; 0 disables) of the named driver
 * entry point ("cuMemCreate", "cuMemAddressReserve", "cuMemMap",
 * "cuMemSetAccess", "cuMemUnmap", "cuMemAlloc", "cuMemcpyHtoD") fail once. */
int vt_mock_fail_nth(const char *call, int nth);
/* Mock only: delay every cuMemMap by this many microseconds (tests the bounded wait). */
int vt_mock_map_delay_us(int us);

/* Creates n_chunks physical chunks of chunk_bytes (0 = 2 MiB; must be a multiple
 * of the device's allocation granularity) on `device` and starts the background
 * growth worker.  Replaces init_physical_handle (vmm_allocator.cpp:113-151) and
 * PhyBlock (vmm_allocator.cpp:154-174).  The driver charges per chunk, not per byte
 * (B200: cuMemCreate 0.07 ms, cuMemSetAccess 0.15 ms per chunk of 2 to 32 MiB), so a
 * larger chunk makes pool creation and every growth cheaper per byte at the price of
 * up to one chunk of unused memory per range. */
int vt_pool_create(int device, size_t n_chunks, size_t chunk_bytes, vt_pool **out);
/* Stops the worker, releases every chunk.  All segments and tables of the pool
 * must have been destroyed first (VT_ERR_STATE otherwise). */
int vt_pool_destroy(vt_pool *pool);
/* Free chunk count; replaces showFreeBlocks (vmm_allocator.cpp:472-474). */
int vt_pool_free_chunks(vt_pool *pool, size_t *out);
int vt_pool_stats(vt_pool *pool, vt_stats *out);

/* One sequence slot: reserves 2 * n_layers virtual ranges of reserve_bytes each
 * (rounded up to the chunk size) in ONE address reservation, K of layer l at
 * base + (2l) * reserve, V at base + (2l + 1) * reserve, and maps premap_bytes
 * of every range right away.  Replaces the KVcacheSegment constructor
 * (vmm_allocator.cpp:177-211). */
int vt_seg_create(vt_pool *pool, int n_layers, size_t reserve_bytes, size_t premap_bytes, vt_seg **out);
/* Unmaps everything, returns the chunks, frees the address reservation. */
int vt_seg_destroy(vt_seg *seg);
/* Base device address of layer's K / V range; replaces getKeyDevicePtr /
 * getValueDevicePtr (vmm_allocator.cpp:299-305). */
int vt_seg_k_ptr(vt_seg *seg, int layer, uint64_t *dptr);
int vt_seg_v_ptr(vt_seg *seg, int layer, uint64_t *dptr);
/* Logical fill in bytes per range; replaces get_used_slot / set_used_size
 * (vmm_allocator.cpp:339-346). */
int vt_seg_used(vt_seg *seg, size_t *bytes);
int vt_seg_set_used(vt_seg *seg, size_t bytes);
/* Mapped bytes per range (the reference's actual_size) and the reservation. */
int vt_seg_mapped(vt_seg *seg, size_t *bytes);
int vt_seg_reserved(vt_seg *seg, size_t *bytes);
/* Synchronously map chunks until every range has >= bytes_needed mapped.
 * Replaces expandMultiSegment / the prefill-side copy_kv_cache
 * (vmm_allocator.cpp:214-297, :322-337) without the fixed 100-token headroom. */
int vt_seg_grow(vt_seg *seg, size_t bytes_needed);
/* Queue a growth of n_chunks per range on the pool's worker thread and return
 * at once.  Replaces eagerExtend + the eagerly_extend thread
 * (vmm_allocator.cpp:307-320, :40-72). */
int vt_seg_grow_async(vt_seg *seg, int n_chunks);
/* 1 if no growth is pending for the segment; replaces query_shm
 * (vmm_allocator.cpp:85-92). */
int vt_seg_ready(vt_seg *seg, int *ready);
/* Blocks until no growth is pending or timeout_us elapsed (VT_ERR_TIMEOUT).
 * Returns the status of the last finished background growth.  Replaces the
 * unbounded spin in vllm/model_executor/models/llama.py:322-326. */
int vt_seg_wait(vt_seg *seg, uint64_t timeout_us);
/* Unmap everything beyond keep_bytes (rounded up to a chunk) in every range,
 * return those chunks, reset used to 0.  Replaces release_seq
 * (vmm_allocator.cpp:383-421); keep_bytes = 0 is preempt_seq (:348-381). */
int vt_seg_release(vt_seg *seg, size_t keep_bytes);

/* The decode-step bookkeeping of extend_kv_cache_batch (vmm_allocator.h:138-168)
 * for n segments in one call: for entry i, if set_used_tokens[i] > 0 then
 * used = set_used_tokens[i] * kv_size; out_offsets[i] = used; then
 *   gen != 0 (decode):  used += token_bytes[i]; if the rows would not fit into
 *                       mapped memory the call first waits up to wait_us for the
 *                       slot's pending background growth (VT_ERR_TIMEOUT) and, if
 *                       that does not cover them, maps synchronously;
 *   gen == 0 (prefill): grow synchronously to used + token_bytes[i], used += token_bytes[i].
 * Nothing is committed when any entry fails.
 * set_used_tokens may be NULL. */
int vt_extend_batch(vt_seg *const *segs, int n, const int64_t *set_used_tokens,
                    const uint64_t *token_bytes, uint64_t kv_size, int gen,
                    uint64_t wait_us, int64_t *out_offsets);

/* Device array of n_slots 8-byte base addresses indexed by slot id; replaces
 * KVCache (vmm_allocator.cpp:458-470). */
int vt_table_create(vt_pool *pool, int n_slots, vt_table **out);
int vt_table_destroy(vt_table *tbl);
int vt_table_set(vt_table *tbl, int slot, uint64_t dptr);
/* Fills slots [0, n) of k_tbl / v_tbl with the layer's K / V base of segs[i];
 * replaces the per-layer loop of copy_kv_cache (vmm_allocator.h:170-182). */
int vt_table_fill(vt_table *k_tbl, vt_table *v_tbl, vt_seg *const *segs, int n, int layer);
int vt_table_dptr(vt_table *tbl, uint64_t *dptr);

/* Debug helpers: synchronous copies between host memory and an address inside a
 * mapped range (or a table).  Replace write_string / read_string
 * (vmm_allocator.cpp:423-446).  They synchronise the device. */
int vt_pool_read(vt_pool *pool, void *dst_host, uint64_t src_dptr, size_t bytes);
int vt_pool_write(vt_pool *pool, uint64_t dst_dptr, const void *src_host, size_t bytes);

/* ---- KV append --------------------------------------------------------- */
/* Writes new K/V rows into the slots' ranges.  Replaces reshape_and_cache
 * (csrc/cache_kernels.cu:153-200, :257-297; declared csrc/cache.h:18-29).
 *   key/value     bf16 [tokens, kvh, d], dim-0 stride in ELEMENTS (fused-qkv views allowed)
 *   k_table/v_table  device arrays of base addresses indexed by slot id
 *   byte_off[i]   device int64: destination byte offset of entry i's first row
 *                 (what extend_kv_cache_batch returned); negative = skip entry
 *   slot_ids[i]   device int64: slot of entry i
 *   max_seq_len   1 = decode (one row per entry, source row i); otherwise
 *                 prefill: entry i writes seq_lens[i] rows read from source rows
 *                 cache_seq_lens[i] + t (both device int32, required then)
 *   kv_dtype      VT_KV_BF16: bit-exact copy, row = kvh*d*2 bytes;
 *                 VT_KV_FP8_E4M3: byte = sat_e4m3(x / scale[kv_head]),
 *                 row = kvh*d bytes, k_scale/v_scale device float[kvh]
 *                 (fp8 storage has no counterpart on the reference's vTensor
 *                 path; arithmetic follows csrc/quantization/fp8/nvidia/quant_utils.cuh:467-479)
 * d must be 128. */
int vt_append(const void *key, const void *value, int64_t key_stride, int64_t value_stride,
              const uint64_t *k_table, const uint64_t *v_table, const int64_t *byte_off,
              const int64_t *slot_ids, const int32_t *seq_lens, const int32_t *cache_seq_lens,
              int max_seq_len, int batch, int kvh, int d, int kv_dtype, const float *k_scale,
              const float *v_scale, void *stream);

/* Per-kv-head scale = amax / 448 over n_tokens rows of x (bf16 [n_tokens, kvh, d],
 * dim-0 stride in elements), 1.0 for an all-zero head.  scale: device float[kvh].
 * No counterpart in the reference (its scales come from a checkpoint file,
 * vllm/model_executor/model_loader/weight_utils.py:296-333). */
int vt_kv_scales(const void *x, int64_t stride, int n_tokens, int kvh, int d, float *scale,
                 void *stream);

/* Widens fp8 e4m3 ranges into dense bf16 rows, x = bf16(e4m3 * scale[kv_head]): the
 * dequantising direction of the reference's scaled_convert
 * (GLakeServe/csrc/quantization/fp8/nvidia/quant_utils.cuh:347-359).  Entry i's first
 * seq_lens[i] rows of K (and V) go to the device address k_out[i] (v_out[i]),
 * 16-byte aligned, row = kvh * 128 bf16, token-major like the ranges themselves.
 * This is how prompt / prefix-extend attention runs over an fp8 cache: the rows are
 * widened into scratch ranges once and the bf16 tensor-core prefill kernels
 * (vt_prefill_attn / vt_prefill_attn_tma) run on those; the extra traffic, 3 bytes
 * per cache byte, is small next to the attention's flops. */
int vt_kv_widen(const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                int batch, int kvh, int d, int max_seq_len, const float *k_scale, const float *v_scale,
                const uint64_t *k_out, const uint64_t *v_out, void *stream);

/* ---- decode attention -------------------------------------------------- */
/* Scratch bytes vt_decode_attn needs for this problem size (max_seq_len is an
 * upper bound of every seq_lens entry).  The scratch holds the split-K partial
 * results; the caller allocates it once and may reuse it for every layer. */
int vt_decode_attn_workspace_bytes(int batch, int h, int d, int max_seq_len, size_t *bytes);

/* out[i, hq, :] = softmax_t(scale * q[i, hq] . K[t, hq / (h / kvh)]) . V[t, hq / (h / kvh)]
 * over tokens t < seq_lens[i] of slot slot_ids[i]; element (t, kv_head, x) of a
 * range sits at ((t * kvh + kv_head) * d + x) elements from its base.
 * Replaces paged_attention_v1 as modified for vTensor
 * (csrc/attention/attention_kernels.cu:93-420, :721-737; csrc/ops.h:6-19) and
 * the decode call of fwd_kvcache (vllm/attention/backends/xformers.py:407-430).
 *   out, q        bf16 [batch, h, d]; strides of dim 0 in elements
 *   seq_lens      device int32 [batch] (context INCLUDING the appended token)
 *   max_seq_len   host upper bound of seq_lens, sizes the split-K grid
 *   scale         softmax scale (1/sqrt(d) in the reference)
 *   kv_dtype, k_scale, v_scale   as for vt_append
 *   lse           optional device float [batch, h]: log-sum-exp of the scaled
 *                 logits (second return value of fwd_kvcache); may be NULL
 *   workspace     >= vt_decode_attn_workspace_bytes(...) bytes, 256-byte aligned
 *   num_splits    0 = choose; otherwise the number of token partitions per sequence
 * Long contexts are split over tokens; a second kernel merges the partial
 * results.  d must be 128; h / kvh in {1,2,4,8,16}; no ALiBi, no sliding window. */
int vt_decode_attn(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                   const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                   const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len,
                   float scale, int kv_dtype, const float *k_scale, const float *v_scale,
                   float *lse, void *workspace, size_t workspace_bytes, int num_splits,
                   void *stream);

/* Process-wide override of the planner, for benchmarks and tests (no counterpart
 * in the reference).  variant: -1 = the planner's choice, 0 = SIMT split-K,
 * 1 = tensor-core split-K, 2 = tensor-core persistent schedule (ignored where the
 * variant does not take the shape); part_tokens: 0 = the planner's choice, else
 * tokens per split-K partition (>= 32, rounded down to a multiple of 32).  The
 * environment variables VT_ATTN_VARIANT (simt | mma | flat) and
 * VT_ATTN_PART_TOKENS give the initial values and are read once. */
int vt_attn_set_tuning(int variant, int part_tokens);

/* What vt_decode_attn will do for this problem: tokens per split-K partition,
 * partitions per sequence the scratch is laid out for (> 1 means the merge
 * kernel runs too), and the kernel variant (0 = SIMT, 1 = tensor-core GQA).
 * Introspection for benchmarks and tests; no counterpart in the reference. */
int vt_decode_attn_plan(int batch, int h, int kvh, int max_seq_len, int kv_dtype, int num_splits,
                        int *part_tokens, int *max_parts, int *variant);

/* One decode step of a layer in a single call: append this step's K/V rows
 * (vt_append with max_seq_len == 1) and attend (vt_decode_attn).  Results are
 * identical to the two calls in sequence; seq_lens INCLUDES the appended token and
 * byte_off[i] is its destination offset, as extend_kv_cache_batch returned it.
 * On the persistent schedule (every supported head shape of both cache types) the
 * two are ONE kernel launch: the attention kernel takes the newest row from key /
 * value (copied for a bf16 cache, quantised for an fp8 cache) and stores it into the
 * range itself, so the step has no append launch and no dependency between the two.
 * Otherwise the call enqueues the append kernel followed by the attention kernels.
 * Replaces the pair of calls in XFormersImpl.forward
 * (vllm/attention/backends/xformers.py:310-312 and :407-430).
 * key / value must be 16-byte aligned with strides that are multiples of 8 elements.
 *
 * flags: 0, or VT_STEP_OVERLAP to let this launch overlap the tail of the previous
 * kernel on the stream when that kernel was a vt_decode_step too (programmatic
 * dependent launch): this call's CTAs take SM slots as the previous call's CTAs
 * exit and stream their K/V early.  Only set it when (1) nothing this call reads
 * — q, key, value, seq_lens, slot_ids, byte_off, the slots' ranges — is written by
 * the previous kernel on the stream (consecutive LAYERS of one step qualify; two
 * steps on the same layer do not), and (2) the workspace was zero-filled once
 * after allocation and is used by nothing but these calls.
 * VT_STEP_EARLY_KV is the form for a step whose q / key / value ARE produced by the
 * kernel in front of it (the usual case inside a model): the launch is again a
 * programmatic dependent, reads its metadata (seq_lens, slot_ids, byte_off, the
 * tables — none of them written by that kernel) and starts streaming the cache
 * rows of earlier tokens at once, but waits for the preceding kernel to complete
 * before it touches q, key, value or the scratch.  It hides the launch ramp and the
 * fill of the copy ring behind the tail of the preceding kernel when that kernel
 * releases its dependents early (vt_all_reduce and vt_decode_step do); behind any
 * other kernel it behaves like an ordinary launch.  Condition (2) applies.
 * VT_STEP_CLEAN_SCRATCH (may be combined with the others, which imply it): the caller
 * guarantees condition (2), so the call does not clear the scratch's ticket counters first
 * (an ordinary launch otherwise enqueues a small memset in front of the kernel: about 2 us
 * per call).  The kernels leave the counters at zero; after a call that reported
 * VT_ERR_KERNEL through the status word, zero the scratch again before reusing it. */
#define VT_STEP_OVERLAP 1u
#define VT_STEP_EARLY_KV 2u
#define VT_STEP_CLEAN_SCRATCH 4u
int vt_decode_step(void *out, int64_t out_stride, const void *q, int64_t q_stride, const void *key,
                   const void *value, int64_t key_stride, int64_t value_stride, const int64_t *byte_off,
                   const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                   const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len, float scale,
                   int kv_dtype, const float *k_scale, const float *v_scale, float *lse, void *workspace,
                   size_t workspace_bytes, unsigned flags, void *stream);

/* vt_decode_step for an fp8 cache with the K/V tiles fetched by TMA tensor copies and
 * the two products on tcgen05.mma.kind::f8f6f4 (the cache bytes reach the tensor core
 * unconverted; Q is carried as two and P as three e4m3 terms).  Same arguments and
 * results within the fp8 tolerance of vt_decode_step, plus
 *   maps   device copy of the table vt_decode_maps_encode filled: for every slot id a
 *          K and a V tensor map of this layer's ranges (2 x 128 bytes per slot,
 *          64-byte aligned).
 * key / value may both be NULL (plain attention over rows already appended; of the
 * flags only VT_STEP_CLEAN_SCRATCH applies then).  Shapes the tcgen05 kernel does not take (kv heads not a power of
 * two >= 8, more than 4 q heads per kv head, bf16 ranges) run exactly as vt_decode_step.
 * vt_decode_maps_encode writes the table into HOST memory (n_slots x 256 bytes, 64-byte
 * aligned; the caller copies it to the device once): k_bases / v_bases are the slots'
 * range bases of one layer, max_tokens the rows a range is reserved for.  Bases never
 * move, so the table stays valid while the slots live.  kv_dtype must be
 * VT_KV_FP8_E4M3 and kvh a power of two <= 256 (VT_ERR_UNSUPPORTED otherwise).
 * No counterpart in the reference (its fp8 decode is paged_attention_v1/v2 with
 * per-element conversion, csrc/attention/attention_kernels.cu:93-420). */
int vt_decode_maps_encode(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, int d,
                          int kv_dtype, uint64_t max_tokens, void *host_maps);
int vt_decode_step_tma(void *out, int64_t out_stride, const void *q, int64_t q_stride, const void *key,
                       const void *value, int64_t key_stride, int64_t value_stride, const int64_t *byte_off,
                       const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                       const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len, float scale,
                       int kv_dtype, const float *k_scale, const float *v_scale, float *lse, void *workspace,
                       size_t workspace_bytes, unsigned flags, const void *maps, void *stream);

/* Causal attention of the NEW tokens of each sequence over its whole range
 * (prefix + new tokens; the new rows must have been appended with vt_append):
 * query row j of entry i sits at position seq_lens[i] - q_lens[i] + j and attends
 * tokens [0, position].  Replaces the prefix-prefill call of fwd_kvcache with
 * seqlen_q > 1 (vllm/attention/backends/xformers.py:362-385).
 *   out, q      bf16 [tokens, h, d]; stride of a token row in elements
 *   seq_lens    device int32 [batch]: context INCLUDING the new tokens
 *   q_lens      device int32 [batch]: new tokens per entry (<= seq_lens)
 *   q_start     device int32 [batch]: first row of entry i in q / out
 *   max_q_len   host upper bound of q_lens (sizes the grid)
 *   status      optional device word set to a non-zero magic if a bounded wait ran out; may be NULL
 * bf16 KV only; d must be 128; q 16-byte aligned with a row stride that is a multiple of 8 elements. */
int vt_prefill_attn(void *out, int64_t out_stride, const void *q, int64_t q_stride, const uint64_t *k_table,
                    const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                    const int32_t *q_lens, const int32_t *q_start, int batch, int h, int kvh, int d,
                    int max_q_len, float scale, int kv_dtype, uint32_t *status, void *stream);

/* vt_prefill_attn with the K/V tiles fetched by TMA tensor copies (one request
 * per 32 tokens x 64 dims instead of one per token row) and, when the shapes allow
 * (kvh <= 128, out rows 16-byte aligned, scale > 0), the math on tcgen05.mma with
 * the accumulators in tensor memory; otherwise on mma.sync.  Same results within
 * the tolerance of vt_prefill_attn.  Same arguments plus
 *   maps   device copy of the table vt_prefill_maps_encode filled: for every slot
 *          id a K and a V tensor map (2 x 128 bytes per slot, 64-byte aligned).
 * vt_prefill_maps_encode writes that table into HOST memory (n_slots x 256 bytes,
 * 64-byte aligned; the caller copies it to the device once): k_bases / v_bases are
 * the slots' range bases of one layer (vt_seg_k_ptr / vt_seg_v_ptr), max_tokens
 * the rows a range is reserved for.  Bases never move, so the table stays valid
 * while the slots live.  kvh must be a power of two <= 256 (a 32-token box may not
 * straddle a 2 MiB chunk); VT_ERR_UNSUPPORTED otherwise — use vt_prefill_attn.
 * No counterpart in the reference (its prefill runs in the external flash-attn fork). */
#define VT_TMA_MAP_BYTES 128
int vt_prefill_maps_encode(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, int d,
                           uint64_t max_tokens, void *host_maps);
int vt_prefill_attn_tma(void *out, int64_t out_stride, const void *q, int64_t q_stride, const uint64_t *k_table,
                        const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                        const int32_t *q_lens, const int32_t *q_start, int batch, int h, int kvh, int d,
                        int max_q_len, float scale, int kv_dtype, uint32_t *status, const void *maps,
                        void *stream);

/* ---- element-wise steps either side of the attention --------------------- */
/* Rotary embedding of q and k followed by the KV append, in one launch.
 * Replaces the pair rotary_embedding (csrc/pos_encoding_kernels.cu:77-130,
 * declared csrc/ops.h:52-58; called at vllm/model_executor/models/llama.py:172-181)
 * + reshape_and_cache (csrc/cache_kernels.cu:153-200): the rotated key goes
 * straight into the slot's range instead of making a round trip through memory.
 *   positions      device int64 [tokens]: position of each token row
 *   query          bf16 [tokens, num_heads, d], rotated IN PLACE; stride of dim 0 in elements
 *   key, value     bf16 [tokens, kvh, d]; key is left untouched unless
 *                  VT_ROPE_WRITE_KEY is given (the reference's rotary_embedding
 *                  rotates it in place; only callers that read key again need that)
 *   cos_sin_cache  bf16 [max_position, rot_dim]: cos of the rot_dim/2 frequencies,
 *                  then their sin (vllm/model_executor/layers/rotary_embedding.py:83-93)
 *   rot_dim        multiple of 16, <= d; elements beyond it pass through unrotated
 *   is_neox        non-zero: pairs (j, j + rot_dim/2); zero: GPT-J pairs (2j, 2j+1)
 *   the remaining arguments are vt_append's, with the same meaning; token row
 *   numbering (decode: row i; prefill: cache_seq_lens[i] + t) also indexes positions.
 * Arithmetic as the reference's CPU kernel (csrc/cpu/pos_encoding.cpp:23-89,
 * :109-166): fp32 products, one rounding to bf16; with an fp8 cache the rounded
 * bf16 key is what gets quantised, as in the two-kernel sequence.  Pointers must
 * be 16-byte aligned and strides multiples of 8 elements (VT_ERR_UNSUPPORTED). */
#define VT_ROPE_WRITE_KEY 1u
int vt_rope_append(const int64_t *positions, void *query, int64_t query_stride, int num_heads, void *key,
                   const void *value, int64_t key_stride, int64_t value_stride, const void *cos_sin_cache,
                   int rot_dim, int is_neox, const uint64_t *k_table, const uint64_t *v_table,
                   const int64_t *byte_off, const int64_t *slot_ids, const int32_t *seq_lens,
                   const int32_t *cache_seq_lens, int max_seq_len, int batch, int kvh, int d, int kv_dtype,
                   const float *k_scale, const float *v_scale, unsigned flags, void *stream);

/* out = input * rsqrt(mean(input^2) + epsilon) * weight per token row.
 * Replaces rms_norm (csrc/layernorm_kernels.cu:21-47, :277-297; csrc/ops.h:40-44).
 *   out, input   bf16 [num_tokens, hidden]; row strides in elements (out may alias input)
 *   weight       bf16 [hidden]
 * hidden must be a multiple of 8 and at most 16384; 16-byte aligned pointers. */
int vt_rms_norm(void *out, const void *input, const void *weight, float epsilon, int num_tokens, int hidden,
                int64_t input_stride, int64_t out_stride, void *stream);

/* residual += input (stored back to residual), then input = rms_norm(residual) * weight,
 * both contiguous bf16 [num_tokens, hidden].  Replaces fused_add_rms_norm
 * (csrc/layernorm_kernels.cu:187-274, :318-352; csrc/ops.h:46-50), the op on either
 * side of the attention block (vllm/model_executor/models/llama.py:245-259).
 * Arithmetic as csrc/cpu/layernorm.cpp:44-88: the variance is taken from the
 * fp32 sums, the scaling from the sums after their rounding to bf16. */
int vt_fused_add_rms_norm(void *input, void *residual, const void *weight, float epsilon, int num_tokens,
                          int hidden, void *stream);

/* ---- low-latency all-reduce over NVLink peer memory ----------------------- */
/* Sum all-reduce of small bf16 messages for the model-level reduction of a
 * tensor-parallel layer (vllm/distributed/communication_op.py:57-84).  Replaces the
 * reference's custom all-reduce (csrc/custom_all_reduce.cuh:182-247, :249-330;
 * csrc/custom_all_reduce.cu:58-68, :116-135;
 * vllm/distributed/device_communicators/custom_all_reduce.py:85, :155-165).
 * One process per GPU; every rank owns one shared buffer that all ranks map:
 *   vt_ar_buffer_bytes   size of that buffer for messages up to max_bytes
 *                        (a multiple of 256)
 *   vt_ar_alloc / free   allocate it zero-filled on the current device (cudaMalloc,
 *                        so that it can be exported); any other zero-filled,
 *                        256-byte aligned, peer-mappable memory works too
 *   vt_ar_ipc_export / open / close   the CUDA IPC route to map it into the other
 *                        processes; the 64-byte handles travel by any host channel
 *   vt_ar_create         peer_bufs[r] = rank r's buffer as mapped in THIS process
 *                        (own buffer at [rank]); n_ctas CTAs per call (0 = 32,
 *                        at most 64), the same on every rank.  All ranks must
 *                        have zero-filled their buffers before anybody's first call
 *                        (a host barrier after creation).
 *   vt_all_reduce        out = sum over ranks of in, n_elems bf16 (a multiple of 8,
 *                        at most max_bytes / 2; VT_ERR_TOO_LARGE beyond), fp32
 *                        accumulation in rank order, bit-identical on every rank;
 *                        in may equal out.  Every rank must make the same sequence
 *                        of calls.  One kernel launch, no host state per call:
 *                        it may be captured into a CUDA graph.
 *   vt_ar_status         0, or non-zero once a wait for a peer ran out of time
 *                        (default 1 s; the results of that call are invalid and the
 *                        communicator should be dropped); synchronises.
 *   vt_ar_configure      wait limit in ns (<= 0 keeps it); the message size up
 *                        to which every rank reads everything itself (one-shot)
 *                        instead of reduce-scatter + all-gather (< 0 keeps it;
 *                        default 6 MiB / (world - 1); two ranks are always one-shot);
 *                        the message size up to which the flag-free push path is
 *                        used (< 0 keeps it, 0 disables it; default and maximum
 *                        256 KiB); the message size up to which larger messages
 *                        take the two-phase push path (scatter-reduce, then
 *                        broadcast, both by stores into sentinel-filled receive
 *                        buffers; < 0 keeps it, 0 disables it; default and maximum
 *                        2 MiB).  On the push paths an input word (or a sum) holding
 *                        two negative zeros travels as two positive zeros.
 *   vt_all_reduce_emulated   runs all `world` ranks of one call as ONE cooperative
 *                        launch on a single GPU (every vt_ar created on that GPU
 *                        with the same peer_bufs): the way to exercise the protocol
 *                        where fewer GPUs than ranks are available.
 * Only plain peer loads and stores are used (no multimem, no TMA). */
typedef struct vt_ar vt_ar;
int vt_ar_buffer_bytes(size_t max_bytes, size_t *bytes);
int vt_ar_alloc(size_t bytes, void **buf);
int vt_ar_free(void *buf);
int vt_ar_ipc_export(void *buf, unsigned char handle[64]);
int vt_ar_ipc_open(const unsigned char handle[64], void **buf);
int vt_ar_ipc_close(void *buf);
int vt_ar_create(int rank, int world, void *const *peer_bufs, size_t max_bytes, int n_ctas, vt_ar **out);
int vt_ar_destroy(vt_ar *ar);
int vt_ar_configure(vt_ar *ar, long long wait_ns, long long one_shot_bytes, long long push_bytes,
                    long long push2_bytes);
int vt_ar_status(vt_ar *ar, uint32_t *status);
int vt_all_reduce(vt_ar *ar, const void *in, void *out, size_t n_elems, void *stream);
int vt_all_reduce_emulated(vt_ar *const *ars, const void *const *ins, void *const *outs, int world,
                           size_t n_elems, void *stream);

/* vt_decode_attn for callers that cannot allocate device memory at all.
 * (No counterpart in the reference: its attention ops get their scratch from
 * torch's allocator.)
 *
 * Some hosts of this library have no way to obtain the scratch buffer that
 * vt_decode_attn asks for: a plugin running inside another runtime's callback
 * where cudaMalloc is forbidden (it may synchronise the device or deadlock on the
 * host runtime's allocator lock), a process whose memory budget is fixed at start
 * and policed, or code that must stay free of allocator calls on its hot path.
 * For them the split-K / piece scratch lives inside the library, in one
 * file-scope __device__ array of VT_STATIC_SCRATCH_BYTES bytes that every GPU
 * holds from the moment it loads the library until the process exits.
 *
 * Same arguments and results as vt_decode_attn minus workspace / workspace_bytes.
 * Differences:
 *   - scratch need is checked against VT_STATIC_SCRATCH_BYTES.  The default
 *     (persistent) schedule fits for every bf16 shape and for an fp8 cache with
 *     query groups up to 8.  When it does not fit (fp8 with a query group of 16)
 *     and num_splits is 0, the call falls back to the split-K schedule with 4, 2
 *     or 1 partitions per sequence, whichever fits first: same result within the
 *     library's parity tolerance, slower kernel.  If nothing fits (or the split
 *     count the caller forced does not), it returns VT_ERR_TOO_LARGE and launches
 *     nothing;
 *   - when the default schedule fits, outputs are bit-identical to
 *     vt_decode_attn's for the same inputs;
 *   - the call itself never allocates or frees: no cudaMalloc / cudaFree and no
 *     allocating library routine;
 *   - the FIRST call on each device resolves the array's device address
 *     (cudaGetSymbolAddress with that device current) and remembers it; make that
 *     first call before any stream capture begins;
 *   - all calls on a device share the one array and it keeps the previous call's
 *     contents (the ticket counters are cleared on every call).  Two calls that
 *     overlap on the GPU (different streams) race on it: serialise them;
 *   - the kernel status word of this buffer cannot be read back. */
#define VT_STATIC_SCRATCH_BYTES (24u << 20)
int vt_decode_attn_static(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                          const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                          const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len,
                          float scale, int kv_dtype, const float *k_scale, const float *v_scale,
                          float *lse, int num_splits, void *stream);

/* Reads (synchronously, on `stream`) the error word the attention kernels set
 * when one of their bounded waits ran out: *code = 0 or VT_ERR_KERNEL. */
int vt_decode_attn_status(void *workspace, void *stream, int *code);

#ifdef __cplusplus
}
#endif
#endif /* VTENSOR_H_ */
