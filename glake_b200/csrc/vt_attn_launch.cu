// Split-K planning, the partial-result merge kernel, and the C entry points of
// the device-side path.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"

namespace vt {
namespace {

constexpr int kMinPartTokens = 256;
constexpr size_t kStatusBytes = 256;

// Merges the per-partition partials of one (sequence, q head):
//   out = sum_p 2^(m_p - M) * o_p / sum_p 2^(m_p - M) * l_p,  M = max_p m_p.
// Sequences that fit one partition were finalised by the attention kernel.
template <bool FP8>
__global__ void __launch_bounds__(kHeadDim) attn_reduce_kernel(AttnParams p) {
  const int hq = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int seq_len = p.seq_lens[b];
  const int n_parts = (seq_len + p.part_tokens - 1) / p.part_tokens;
  if (n_parts <= 1) return;
  const size_t base = (static_cast<size_t>(b) * p.h + hq) * p.max_parts;
  float M = -INFINITY;
  for (int i = 0; i < n_parts; ++i) M = fmaxf(M, p.ws_ml[(base + i) * 2]);
  float L = 0.f, O = 0.f;
  for (int i = 0; i < n_parts; ++i) {
    const float f = exp2f(p.ws_ml[(base + i) * 2] - M);
    L = fmaf(f, p.ws_ml[(base + i) * 2 + 1], L);
    O = fmaf(f, p.ws_o[(base + i) * kHeadDim + d], O);
  }
  const float vs = FP8 ? p.v_scale[hq / (p.h / p.kvh)] : 1.0f;
  static_cast<__nv_bfloat16 *>(p.out)[b * p.out_stride + hq * kHeadDim + d] = __float2bfloat16(O / L * vs);
  if (p.lse && d == 0) p.lse[b * p.h + hq] = (M + log2f(L)) * 0.6931471805599453f;
}

}  // namespace

namespace {
// Process-wide tuning override: variant -1 = the planner's choice, part_tokens 0 = likewise.
struct Tuning { int variant, part_tokens; };
std::atomic<int> g_tune_variant{-1}, g_tune_part{0};
std::once_flag g_tune_env;
Tuning tuning() {
  std::call_once(g_tune_env, [] {
    if (const char *v = getenv("VT_ATTN_VARIANT")) {
      if (!strcmp(v, "simt")) g_tune_variant.store(0);
      if (!strcmp(v, "mma")) g_tune_variant.store(1);
      if (!strcmp(v, "flat")) g_tune_variant.store(2);
    }
    if (const char *v = getenv("VT_ATTN_PART_TOKENS")) g_tune_part.store(atoi(v));
  });
  return Tuning{g_tune_variant.load(std::memory_order_relaxed), g_tune_part.load(std::memory_order_relaxed)};
}
}  // namespace

size_t attn_workspace_bytes(int batch, int h, int max_parts) {
  const size_t rows = static_cast<size_t>(batch) * h * max_parts;
  size_t ml = (rows * 2 * sizeof(float) + 255) / 256 * 256;
  return kStatusBytes + ml + rows * kHeadDim * sizeof(float);
}

static size_t flat_counter_bytes(int batch, int kvh) {
  return (static_cast<size_t>(batch) * kvh * sizeof(unsigned) + 255) / 256 * 256;
}
static size_t flat_workspace_bytes(int batch, int h, int kvh, int kv_dtype, bool worst_case = false) {
  const int heads = (!worst_case && (h / kvh) <= 8) ? 8 : 16;
  const int warps = worst_case ? 8 : flat_consumer_warps(kv_dtype);
  const int ctas = worst_case ? kFlatMaxCtas : flat_max_ctas(h, kvh, kv_dtype);
  return kStatusBytes + flat_counter_bytes(batch, kvh) +
         static_cast<size_t>(ctas) * 2 * warps * heads * kFlatPartRow * sizeof(float);
}

size_t attn_workspace_bound(int batch, int h, int max_seq_len) {
  const int parts = std::max(1, (max_seq_len + kMinPartTokens - 1) / kMinPartTokens);
  // the flat schedule's scratch does not depend on the context length; h stands in
  // for the kv-head count (its upper bound) when sizing the ticket counters
  return std::max(attn_workspace_bytes(batch, h, parts), flat_workspace_bytes(batch, h, h, VT_KV_BF16, true));
}

void carve_workspace(void *ws, int batch, int h, int max_parts, AttnParams *p) {
  char *c = static_cast<char *>(ws);
  const size_t rows = static_cast<size_t>(batch) * h * max_parts;
  p->status = reinterpret_cast<uint32_t *>(c);
  p->ws_ml = reinterpret_cast<float *>(c + kStatusBytes);
  p->ws_o = reinterpret_cast<float *>(c + kStatusBytes + (rows * 2 * sizeof(float) + 255) / 256 * 256);
}

static void carve_flat(void *ws, int batch, int kvh, AttnParams *p) {
  char *c = static_cast<char *>(ws);
  p->status = reinterpret_cast<uint32_t *>(c);
  p->fl_count = reinterpret_cast<unsigned *>(c + kStatusBytes);
  p->fl_part = reinterpret_cast<float *>(c + kStatusBytes + flat_counter_bytes(batch, kvh));
}

int plan_attn(int batch, int h, int kvh, int max_seq_len, int kv_dtype, int num_splits, AttnPlan *plan) {
  const int g = h / kvh;
  // Tensor-core engine wherever it applies (bf16 KV) — on the flat persistent
  // schedule unless the caller asks for explicit splits — SIMT otherwise (fp8 KV).
  (void)g;
  plan->variant = attn_mma_supports(h, kvh, kv_dtype) ? 1 : 0;
  if (num_splits == 0 && attn_flat_supports(batch, h, kvh, kv_dtype)) plan->variant = 2;
  // Tuning override (vt_attn_set_tuning, or the VT_ATTN_VARIANT / VT_ATTN_PART_TOKENS
  // environment variables read once when the library first plans a call).
  const Tuning tn = tuning();
  if (tn.variant == 0) plan->variant = 0;
  if (tn.variant == 1 && attn_mma_supports(h, kvh, kv_dtype)) plan->variant = 1;
  if (tn.variant == 2 && attn_flat_supports(batch, h, kvh, kv_dtype)) plan->variant = 2;
  int part;
  if (num_splits > 0) {
    part = (max_seq_len + num_splits - 1) / num_splits;
    part = std::max(32, (part + 31) / 32 * 32);
  } else {
    // Enough CTAs to keep 148 SMs x 3 resident CTAs busy for several waves and to
    // even out ragged context lengths, without partitions so small that the
    // pipeline fill and the partial write-back show up.
    const long units = static_cast<long>(batch) * kvh;
    const long target = 148L * 3 * 8;
    long want_parts = (target + units - 1) / std::max(1L, units);
    part = static_cast<int>((max_seq_len + want_parts - 1) / want_parts);
    part = std::max(kMinPartTokens, std::min(1024, (part + 31) / 32 * 32));
  }
  if (tn.part_tokens >= 32) part = tn.part_tokens / 32 * 32;
  plan->part_tokens = part;
  plan->max_parts = std::max(1, (max_seq_len + part - 1) / part);
  plan->ws_bytes = attn_workspace_bytes(batch, h, plan->max_parts);
  if (plan->variant == 2) {
    plan->max_parts = 1;   // no merge kernel: the last CTA of a stream merges it
    plan->ws_bytes = flat_workspace_bytes(batch, h, kvh, kv_dtype);
  }
  return VT_OK;
}

int launch_attn_reduce(const AttnParams &p, int kv_dtype, cudaStream_t stream) {
  dim3 grid(p.h, p.batch);
  if (kv_dtype == VT_KV_FP8_E4M3)
    attn_reduce_kernel<true><<<grid, kHeadDim, 0, stream>>>(p);
  else
    attn_reduce_kernel<false><<<grid, kHeadDim, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

}  // namespace vt

extern "C" {

int vt_append(const void *key, const void *value, int64_t key_stride, int64_t value_stride,
              const uint64_t *k_table, const uint64_t *v_table, const int64_t *byte_off,
              const int64_t *slot_ids, const int32_t *seq_lens, const int32_t *cache_seq_lens,
              int max_seq_len, int batch, int kvh, int d, int kv_dtype, const float *k_scale,
              const float *v_scale, void *stream) {
  if (batch < 0 || kvh <= 0 || max_seq_len < 1) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (!key || !value || !k_table || !v_table || !byte_off || !slot_ids) return VT_ERR_INVALID;
  if (d != vt::kHeadDim) return VT_ERR_UNSUPPORTED;
  if (kv_dtype != VT_KV_BF16 && kv_dtype != VT_KV_FP8_E4M3) return VT_ERR_UNSUPPORTED;
  if (kv_dtype == VT_KV_FP8_E4M3 && (!k_scale || !v_scale)) return VT_ERR_INVALID;
  if (max_seq_len > 1 && (!seq_lens || !cache_seq_lens)) return VT_ERR_INVALID;
  if (key_stride < static_cast<int64_t>(kvh) * d || value_stride < static_cast<int64_t>(kvh) * d) return VT_ERR_INVALID;
  vt::AppendParams p{key, value, key_stride, value_stride, k_table, v_table, byte_off, slot_ids,
                     seq_lens, cache_seq_lens, max_seq_len, batch, kvh, k_scale, v_scale};
  return vt::launch_append(p, kv_dtype, static_cast<cudaStream_t>(stream));
}

int vt_kv_scales(const void *x, int64_t stride, int n_tokens, int kvh, int d, float *scale, void *stream) {
  if (!x || !scale || n_tokens < 0 || kvh <= 0) return VT_ERR_INVALID;
  if (d != vt::kHeadDim) return VT_ERR_UNSUPPORTED;
  return vt::launch_kv_scales(x, stride, n_tokens, kvh, scale, static_cast<cudaStream_t>(stream));
}

int vt_kv_widen(const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                int batch, int kvh, int d, int max_seq_len, const float *k_scale, const float *v_scale,
                const uint64_t *k_out, const uint64_t *v_out, void *stream) {
  if (batch < 0 || kvh <= 0 || max_seq_len < 0) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (!k_table || !v_table || !slot_ids || !seq_lens || !k_scale || !v_scale || !k_out || !v_out) return VT_ERR_INVALID;
  if (d != vt::kHeadDim) return VT_ERR_UNSUPPORTED;
  vt::KvWidenParams p{k_table, v_table, slot_ids, seq_lens, k_out, v_out, batch, kvh, k_scale, v_scale};
  return vt::launch_kv_widen(p, max_seq_len, static_cast<cudaStream_t>(stream));
}

int vt_decode_attn_workspace_bytes(int batch, int h, int d, int max_seq_len, size_t *bytes) {
  if (!bytes || batch < 0 || h <= 0 || max_seq_len < 0) return VT_ERR_INVALID;
  if (d != vt::kHeadDim) return VT_ERR_UNSUPPORTED;
  *bytes = vt::attn_workspace_bound(std::max(batch, 1), h, std::max(max_seq_len, 1));
  return VT_OK;
}

static int decode_attn_impl(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                   const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                   const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len,
                   float scale, int kv_dtype, const float *k_scale, const float *v_scale,
                   float *lse, void *workspace, size_t workspace_bytes, int num_splits,
                   void *stream, const void *new_key, const void *new_value, int64_t new_key_stride,
                   int64_t new_value_stride, const int64_t *byte_off, unsigned flags, const void *maps = nullptr) {
  if (batch < 0 || h <= 0 || kvh <= 0 || max_seq_len < 0 || num_splits < 0) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (!out || !q || !k_table || !v_table || !slot_ids || !seq_lens || !workspace) return VT_ERR_INVALID;
  if (d != vt::kHeadDim || h % kvh != 0) return VT_ERR_UNSUPPORTED;
  const int g = h / kvh;
  if (g != 1 && g != 2 && g != 4 && g != 8 && g != 16) return VT_ERR_UNSUPPORTED;
  if (kv_dtype != VT_KV_BF16 && kv_dtype != VT_KV_FP8_E4M3) return VT_ERR_UNSUPPORTED;
  if (kv_dtype == VT_KV_FP8_E4M3 && (!k_scale || !v_scale)) return VT_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride % 8) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return VT_ERR_INVALID;
  if (q_stride < static_cast<int64_t>(h) * d || out_stride < static_cast<int64_t>(h) * d) return VT_ERR_INVALID;
  vt::AttnPlan plan;
  vt::plan_attn(batch, h, kvh, std::max(max_seq_len, 1), kv_dtype, num_splits, &plan);
  if (plan.ws_bytes > workspace_bytes) return VT_ERR_INVALID;
  vt::AttnParams p{};
  p.out = out; p.out_stride = out_stride; p.q = q; p.q_stride = q_stride;
  p.k_table = k_table; p.v_table = v_table; p.slot_ids = slot_ids; p.seq_lens = seq_lens;
  p.batch = batch; p.h = h; p.kvh = kvh; p.scale = scale; p.k_scale = k_scale; p.v_scale = v_scale;
  p.lse = lse; p.part_tokens = plan.part_tokens; p.max_parts = plan.max_parts;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool fused = new_key && plan.variant == 2;   // the persistent kernel appends the step's rows itself
  if (new_key && !fused) {
    // no fused kernel for this shape / dtype: append first, then attend
    int st = vt_append(new_key, new_value, new_key_stride, new_value_stride, k_table, v_table, byte_off, slot_ids,
                       nullptr, nullptr, 1, batch, kvh, d, kv_dtype, k_scale, v_scale, stream);
    if (st != VT_OK) return st;
  }
  if (plan.variant == 2) {
    if (fused) {
      p.new_key = new_key; p.new_value = new_value;
      p.new_key_stride = new_key_stride; p.new_value_stride = new_value_stride; p.byte_off = byte_off;
    }
    vt::carve_flat(workspace, batch, kvh, &p);
    // Overlap only for the fused launch: a separate append kernel in front of this one
    // writes the row this launch reads, and only ordinary stream order covers that.
    p.overlap = !fused ? 0 : (flags & VT_STEP_EARLY_KV) ? 2 : (flags & VT_STEP_OVERLAP) ? 1 : 0;
    // The ticket counters return to zero at the end of every launch.  They are
    // cleared here anyway so that a scratch buffer of unknown content works — except
    // in overlap mode, where a memset between the kernels would serialise them and
    // the caller guarantees a zero-initialised buffer instead, or when the caller
    // gives that guarantee for an ordinary launch (VT_STEP_CLEAN_SCRATCH).
    if (!p.overlap && !(flags & VT_STEP_CLEAN_SCRATCH) &&
        cudaMemsetAsync(p.fl_count, 0, static_cast<size_t>(batch) * kvh * sizeof(unsigned), s) != cudaSuccess)
      return VT_ERR_CUDA;
    // fp8 ranges with tensor maps: the tcgen05 engine where the shape allows (same schedule, same scratch)
    if (maps && kv_dtype == VT_KV_FP8_E4M3 && vt::attn_flat_umma_supports(batch, h, kvh, kv_dtype)) {
      p.maps = maps;
      return vt::launch_attn_flat_umma(p, s);
    }
    return vt::launch_attn_flat(p, kv_dtype, s);
  }
  vt::carve_workspace(workspace, batch, h, plan.max_parts, &p);
  int st = plan.variant == 0 ? vt::launch_attn_simt(p, kv_dtype, s) : vt::launch_attn_mma(p, kv_dtype, s);
  if (st != VT_OK) return st;
  if (plan.max_parts > 1) st = vt::launch_attn_reduce(p, kv_dtype, s);
  return st;
}

}  // extern "C"

// Scratch of vt_decode_attn_static.  In host code the name below is only a
// stand-in for the symbol, not a device address: the address is looked up once
// per device with cudaGetSymbolAddress and that pointer is what kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[VT_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void *g_static_ptr[64] = {nullptr};

// Device address of g_static_scratch on the current device (nullptr on failure).
void *static_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> g(g_static_mu);
  if (!g_static_ptr[dev]) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess) return nullptr;
    g_static_ptr[dev] = ptr;
  }
  return g_static_ptr[dev];
}
}  // namespace

extern "C" {

int vt_decode_attn_static(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                          const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                          const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len,
                          float scale, int kv_dtype, const float *k_scale, const float *v_scale,
                          float *lse, int num_splits, void *stream) {
  if (batch < 0 || h <= 0 || kvh <= 0 || max_seq_len < 0 || num_splits < 0) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (d != vt::kHeadDim || h % kvh != 0) return VT_ERR_UNSUPPORTED;
  vt::AttnPlan plan;
  vt::plan_attn(batch, h, kvh, std::max(max_seq_len, 1), kv_dtype, num_splits, &plan);
  if (plan.ws_bytes > VT_STATIC_SCRATCH_BYTES && num_splits == 0) {
    // The default schedule's scratch does not fit the array: see whether a split-K
    // schedule does (4, then 2, then 1 partitions per sequence) before refusing.
    for (int splits = 4; splits >= 1 && plan.ws_bytes > VT_STATIC_SCRATCH_BYTES; splits /= 2) {
      vt::plan_attn(batch, h, kvh, std::max(max_seq_len, 1), kv_dtype, splits, &plan);
      num_splits = splits;
    }
  }
  if (plan.ws_bytes > VT_STATIC_SCRATCH_BYTES) return VT_ERR_TOO_LARGE;
  void *scratch = static_scratch_for_current_device();
  if (!scratch) return VT_ERR_CUDA;
  return vt_decode_attn(out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, batch, h, kvh, d,
                        max_seq_len, scale, kv_dtype, k_scale, v_scale, lse, scratch, VT_STATIC_SCRATCH_BYTES,
                        num_splits, stream);
}

int vt_attn_set_tuning(int variant, int part_tokens) {
  if (variant < -1 || variant > 2 || part_tokens < 0 || (part_tokens != 0 && part_tokens < 32)) return VT_ERR_INVALID;
  vt::tuning();   // the environment is read first, so that it cannot overwrite this later
  vt::g_tune_variant.store(variant);
  vt::g_tune_part.store(part_tokens);
  return VT_OK;
}

int vt_decode_attn_plan(int batch, int h, int kvh, int max_seq_len, int kv_dtype, int num_splits,
                        int *part_tokens, int *max_parts, int *variant) {
  if (batch < 0 || h <= 0 || kvh <= 0 || h % kvh != 0 || max_seq_len < 0 || num_splits < 0) return VT_ERR_INVALID;
  vt::AttnPlan plan;
  vt::plan_attn(std::max(batch, 1), h, kvh, std::max(max_seq_len, 1), kv_dtype, num_splits, &plan);
  if (part_tokens) *part_tokens = plan.part_tokens;
  if (max_parts) *max_parts = plan.max_parts;
  if (variant) *variant = plan.variant;
  return VT_OK;
}

int vt_decode_attn(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                   const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                   const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len,
                   float scale, int kv_dtype, const float *k_scale, const float *v_scale,
                   float *lse, void *workspace, size_t workspace_bytes, int num_splits,
                   void *stream) {
  return decode_attn_impl(out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, batch, h, kvh, d,
                          max_seq_len, scale, kv_dtype, k_scale, v_scale, lse, workspace, workspace_bytes, num_splits,
                          stream, nullptr, nullptr, 0, 0, nullptr, 0u);
}

int vt_decode_step(void *out, int64_t out_stride, const void *q, int64_t q_stride, const void *key,
                   const void *value, int64_t key_stride, int64_t value_stride, const int64_t *byte_off,
                   const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                   const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len, float scale,
                   int kv_dtype, const float *k_scale, const float *v_scale, float *lse, void *workspace,
                   size_t workspace_bytes, unsigned flags, void *stream) {
  if (batch < 0 || kvh <= 0 || (flags & ~static_cast<unsigned>(VT_STEP_OVERLAP | VT_STEP_EARLY_KV | VT_STEP_CLEAN_SCRATCH))) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (!key || !value || !byte_off) return VT_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15) return VT_ERR_INVALID;
  if ((key_stride % 8) || (value_stride % 8) || key_stride < static_cast<int64_t>(kvh) * d ||
      value_stride < static_cast<int64_t>(kvh) * d)
    return VT_ERR_INVALID;
  return decode_attn_impl(out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, batch, h, kvh, d,
                          max_seq_len, scale, kv_dtype, k_scale, v_scale, lse, workspace, workspace_bytes, 0, stream,
                          key, value, key_stride, value_stride, byte_off, flags);
}

int vt_decode_step_tma(void *out, int64_t out_stride, const void *q, int64_t q_stride, const void *key,
                       const void *value, int64_t key_stride, int64_t value_stride, const int64_t *byte_off,
                       const uint64_t *k_table, const uint64_t *v_table, const int64_t *slot_ids,
                       const int32_t *seq_lens, int batch, int h, int kvh, int d, int max_seq_len, float scale,
                       int kv_dtype, const float *k_scale, const float *v_scale, float *lse, void *workspace,
                       size_t workspace_bytes, unsigned flags, const void *maps, void *stream) {
  if (batch < 0 || kvh <= 0 || (flags & ~static_cast<unsigned>(VT_STEP_OVERLAP | VT_STEP_EARLY_KV | VT_STEP_CLEAN_SCRATCH))) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (!maps || (reinterpret_cast<uintptr_t>(maps) & 63) != 0) return VT_ERR_INVALID;
  if (key || value) {
    if (!key || !value || !byte_off) return VT_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15) return VT_ERR_INVALID;
    if ((key_stride % 8) || (value_stride % 8) || key_stride < static_cast<int64_t>(kvh) * d ||
        value_stride < static_cast<int64_t>(kvh) * d)
      return VT_ERR_INVALID;
  } else if (flags & (VT_STEP_OVERLAP | VT_STEP_EARLY_KV)) {
    return VT_ERR_INVALID;   // the overlap forms are defined for the fused step only
  }
  return decode_attn_impl(out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, batch, h, kvh, d,
                          max_seq_len, scale, kv_dtype, k_scale, v_scale, lse, workspace, workspace_bytes, 0, stream,
                          key, value, key_stride, value_stride, byte_off, flags, maps);
}

int vt_decode_maps_encode(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, int d, int kv_dtype,
                          uint64_t max_tokens, void *host_maps) {
  if (!k_bases || !v_bases || !host_maps || n_slots <= 0 || kvh <= 0 || max_tokens == 0) return VT_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(host_maps) & 63) != 0) return VT_ERR_INVALID;
  if (d != vt::kHeadDim || kv_dtype != VT_KV_FP8_E4M3) return VT_ERR_UNSUPPORTED;
  // whole 32-token boxes are fetched at the ragged end of a context: a box must not straddle a 2 MiB chunk
  if ((kvh & (kvh - 1)) != 0 || kvh * 32 > 8192 || max_tokens > 0xffffffffull) return VT_ERR_UNSUPPORTED;
  return vt::encode_decode_maps_f8(k_bases, v_bases, n_slots, kvh, max_tokens, host_maps);
}

static int prefill_impl(void *out, int64_t out_stride, const void *q, int64_t q_stride, const uint64_t *k_table,
                        const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                        const int32_t *q_lens, const int32_t *q_start, int batch, int h, int kvh, int d,
                        int max_q_len, float scale, int kv_dtype, uint32_t *status, const void *maps, void *stream) {
  if (batch < 0 || h <= 0 || kvh <= 0 || max_q_len < 0) return VT_ERR_INVALID;
  if (batch == 0 || max_q_len == 0) return VT_OK;
  if (!out || !q || !k_table || !v_table || !slot_ids || !seq_lens || !q_lens || !q_start) return VT_ERR_INVALID;
  if (d != vt::kHeadDim || h % kvh != 0 || kv_dtype != VT_KV_BF16) return VT_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(out) & 3) || (out_stride % 2)) return VT_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride % 8)) return VT_ERR_UNSUPPORTED;   // q rows are read 16 bytes at a time
  if (q_stride < static_cast<int64_t>(h) * d || out_stride < static_cast<int64_t>(h) * d) return VT_ERR_INVALID;
  if (maps) {
    // Whole 32-token boxes are fetched even at the ragged end of a context, so a box must never
    // straddle a 2 MiB chunk: rows per chunk (8192 / kvh) has to be a multiple of the box.
    if ((reinterpret_cast<uintptr_t>(maps) & 63) != 0) return VT_ERR_INVALID;
    if ((kvh & (kvh - 1)) != 0 || kvh * vt::kPrefillBoxTokens > 8192) return VT_ERR_UNSUPPORTED;
  }
  vt::PrefillParams p{out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, q_lens, q_start,
                      batch, h, kvh, scale, status, maps};
  return vt::launch_prefill_attn(p, max_q_len, static_cast<cudaStream_t>(stream));
}

int vt_prefill_attn(void *out, int64_t out_stride, const void *q, int64_t q_stride, const uint64_t *k_table,
                    const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                    const int32_t *q_lens, const int32_t *q_start, int batch, int h, int kvh, int d,
                    int max_q_len, float scale, int kv_dtype, uint32_t *status, void *stream) {
  return prefill_impl(out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, q_lens, q_start, batch, h,
                      kvh, d, max_q_len, scale, kv_dtype, status, nullptr, stream);
}

int vt_prefill_attn_tma(void *out, int64_t out_stride, const void *q, int64_t q_stride, const uint64_t *k_table,
                        const uint64_t *v_table, const int64_t *slot_ids, const int32_t *seq_lens,
                        const int32_t *q_lens, const int32_t *q_start, int batch, int h, int kvh, int d,
                        int max_q_len, float scale, int kv_dtype, uint32_t *status, const void *maps, void *stream) {
  if (!maps) return VT_ERR_INVALID;
  return prefill_impl(out, out_stride, q, q_stride, k_table, v_table, slot_ids, seq_lens, q_lens, q_start, batch, h,
                      kvh, d, max_q_len, scale, kv_dtype, status, maps, stream);
}

int vt_prefill_maps_encode(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, int d,
                           uint64_t max_tokens, void *host_maps) {
  if (!k_bases || !v_bases || !host_maps || n_slots <= 0 || kvh <= 0 || max_tokens == 0) return VT_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(host_maps) & 63) != 0) return VT_ERR_INVALID;
  if (d != vt::kHeadDim) return VT_ERR_UNSUPPORTED;
  if ((kvh & (kvh - 1)) != 0 || kvh * vt::kPrefillBoxTokens > 8192 || max_tokens > 0xffffffffull) return VT_ERR_UNSUPPORTED;
  return vt::encode_prefill_maps(k_bases, v_bases, n_slots, kvh, max_tokens, host_maps);
}

int vt_decode_attn_status(void *workspace, void *stream, int *code) {
  if (!workspace || !code) return VT_ERR_INVALID;
  uint32_t word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&word, workspace, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) return VT_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return VT_ERR_CUDA;
  *code = word == vt::kKernelErrMagic ? VT_ERR_KERNEL : VT_OK;
  return VT_OK;
}

const char *vt_version(void) { return "vtensor-b200 0.1 sm_100a"; }

const char *vt_strerror(int status) {
  switch (status) {
    case VT_OK: return "ok";
    case VT_ERR_INVALID: return "invalid argument";
    case VT_ERR_DRIVER: return "CUDA driver call failed";
    case VT_ERR_POOL_EMPTY: return "chunk pool exhausted";
    case VT_ERR_RESERVE: return "growth exceeds the reserved virtual range";
    case VT_ERR_TIMEOUT: return "timed out waiting for a pending growth";
    case VT_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case VT_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
    case VT_ERR_STATE: return "call not valid in the current state";
    case VT_ERR_NO_DRIVER: return "libcuda.so.1 could not be loaded";
    case VT_ERR_KERNEL: return "a kernel's bounded wait ran out";
    case VT_ERR_TOO_LARGE: return "problem needs more scratch than the built-in static buffer holds";
    default: return "unknown status";
  }
}

}  // extern "C"
