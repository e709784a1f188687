// Host-visible launch interface of the CUDA kernels (internal to the library).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

namespace vt {

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is per device: remembers, per
// kernel instantiation (one static instance each) and device, the size already set.
struct SmemOptIn {
  std::atomic<int> set[64];
  SmemOptIn() { for (auto &x : set) x.store(0); }
  template <typename K>
  bool ensure(K kernel, int bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (set[dev].load(std::memory_order_relaxed) >= bytes) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    // Without a stated preference the driver may pick a shared-memory carve-out that fits one CTA only.
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) !=
        cudaSuccess)
      return false;
    set[dev].store(bytes, std::memory_order_relaxed);
    return true;
  }
};

struct AppendParams {
  const void *key, *value;
  int64_t key_stride, value_stride;  // elements
  const uint64_t *k_table, *v_table;
  const int64_t *byte_off, *slot_ids;
  const int32_t *seq_lens, *cache_seq_lens;
  int max_seq_len, batch, kvh;
  const float *k_scale, *v_scale;
};
int launch_append(const AppendParams &p, int kv_dtype, cudaStream_t stream);
int launch_kv_scales(const void *x, int64_t stride, int n_tokens, int kvh, float *scale, cudaStream_t stream);

struct KvWidenParams {
  const uint64_t *k_table, *v_table;  // fp8 ranges
  const int64_t *slot_ids;
  const int32_t *seq_lens;            // rows to widen per entry
  const uint64_t *k_out, *v_out;      // per entry: destination of its dense bf16 rows (16-byte aligned)
  int batch, kvh;
  const float *k_scale, *v_scale;
};
int launch_kv_widen(const KvWidenParams &p, int max_seq_len, cudaStream_t stream);

struct AttnParams {
  void *out;  int64_t out_stride;     // bf16, elements per batch row
  const void *q; int64_t q_stride;
  const uint64_t *k_table, *v_table;
  const int64_t *slot_ids;
  const int32_t *seq_lens;
  int batch, h, kvh;
  float scale;                        // softmax scale (natural-log domain)
  const float *k_scale, *v_scale;     // fp8 only
  float *lse;                         // optional [batch, h]
  int part_tokens;                    // tokens per split-K partition (multiple of 32)
  int max_parts;                      // partitions per sequence the scratch is laid out for
  uint32_t *status;                   // scratch status word
  float *ws_ml;                       // [batch, h, max_parts, 2]  (max in log2 domain, sum)
  float *ws_o;                        // [batch, h, max_parts, 128] unnormalised partial outputs
  // flat (persistent) schedule only
  int n_ctas;                         // grid size
  unsigned *fl_count;                 // [batch * kv-head slabs] piece tickets, zero between launches
  float *fl_part;                     // [n_ctas, 2 slots, 4 warps, 8 or 16 heads, 132] piece states
  // fused step (flat schedule only): this step's K/V rows, appended by the attention kernel itself
  const void *new_key, *new_value;    // bf16 [batch, kvh, 128]; nullptr = plain attention
  int64_t new_key_stride, new_value_stride;   // elements per batch row
  const int64_t *byte_off;            // destination byte offset per entry (negative = nothing to append)
  const void *maps;                   // tcgen05 engine only: device table [slot][K, V] of 128-byte TMA tensor maps
  int overlap;                        // launched as a programmatic dependent of the previous kernel on the stream:
                                      // 1 = its inputs are ready already, 2 = wait for that kernel before reading q / new rows
};

constexpr int kFlatMaxBatch = 1024;   // prefix table of the flat schedule lives in shared memory
constexpr int kFlatPartRow = 132;     // floats per published piece state row (16-byte aligned)
constexpr int kFlatSms = 148;         // SMs of a B200; a part with more just runs the same grid on fewer CTAs per SM
constexpr int kFlatMaxCtas = 3 * kFlatSms;   // upper bound of any engine's grid (3 resident CTAs per SM)

struct PrefillParams {
  void *out; int64_t out_stride;      // bf16 [tokens, h, 128]; stride of a token row in elements
  const void *q; int64_t q_stride;
  const uint64_t *k_table, *v_table;
  const int64_t *slot_ids;
  const int32_t *seq_lens;            // context INCLUDING the new tokens
  const int32_t *q_lens;              // new tokens per entry
  const int32_t *q_start;             // first row of the entry in q / out
  int batch, h, kvh;
  float scale;
  uint32_t *status;                   // optional status word
  const void *maps;                   // optional device table [slot][K, V] of 128-byte TMA tensor maps
};
int launch_prefill_attn(const PrefillParams &p, int max_q_len, cudaStream_t stream);
int launch_prefill_umma(const PrefillParams &p, int max_q_len, cudaStream_t stream);   // needs p.maps
constexpr int kPrefillBoxTokens = 32; // token extent of the tensor maps' box (= the kernel's K/V tile)
// Fills host_maps[slot][K, V] (128 bytes each, 64-byte aligned) for ranges of kvh heads and max_tokens rows.
int encode_prefill_maps(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, uint64_t max_tokens,
                        void *host_maps);

struct AttnPlan {
  int part_tokens, max_parts;
  int variant;       // 0 = SIMT split-K, 1 = tensor-core split-K, 2 = tensor-core flat schedule
  size_t ws_bytes;
};
// Picks the partition size and kernel variant for a problem; num_splits 0 = auto.
int plan_attn(int batch, int h, int kvh, int max_seq_len, int kv_dtype, int num_splits, AttnPlan *plan);
size_t attn_workspace_bytes(int batch, int h, int max_parts);
size_t attn_workspace_bound(int batch, int h, int max_seq_len);
void carve_workspace(void *ws, int batch, int h, int max_parts, AttnParams *p);

int launch_attn_simt(const AttnParams &p, int kv_dtype, cudaStream_t stream);
int launch_attn_mma(const AttnParams &p, int kv_dtype, cudaStream_t stream);
bool attn_mma_supports(int h, int kvh, int kv_dtype);
int launch_attn_flat(const AttnParams &p, int kv_dtype, cudaStream_t stream);
bool attn_flat_supports(int batch, int h, int kvh, int kv_dtype);
int flat_consumer_warps(int kv_dtype);
int flat_max_ctas(int h, int kvh, int kv_dtype);
int launch_attn_reduce(const AttnParams &p, int kv_dtype, cudaStream_t stream);
// fp8 cache on tcgen05 (same schedule and scratch as the flat kernel); needs p.maps from encode_decode_maps_f8
int launch_attn_flat_umma(const AttnParams &p, cudaStream_t stream);
bool attn_flat_umma_supports(int batch, int h, int kvh, int kv_dtype);
int encode_decode_maps_f8(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, uint64_t max_tokens,
                          void *host_maps);

}  // namespace vt
