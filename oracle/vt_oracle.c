/*
 * TEST INFRASTRUCTURE — CPU restatement of the vTensor decode path.
 *
 * This file is the checker for the CUDA kernels; it is never linked into, nor
 * called from, the shipped library.  Only tests, the smoke check and the
 * CPU-baseline leg of the bench may load it.
 *
 * What it restates (paths are inside the reference project):
 *   - KV append:        GLakeServe/csrc/cache_kernels.cu:153-200
 *                       (reshape_and_cache_kernel: row copy to
 *                        table[slot] + byte_offset + t * KVH * D * 2)
 *   - decode attention: GLakeServe/csrc/attention/attention_kernels.cu:93-420
 *                       with BLOCK_SIZE = 1 (token-major layout, strides at
 *                       :631-632) for the addressing, and
 *                       GLakeServe/csrc/cpu/attention.cpp:44-66, :216-340
 *                       for the arithmetic (fp32 logits, exp(x - max),
 *                       division by the plain sum, fp32 P.V, one rounding
 *                       to bf16 at the end).
 *   - fp8 e4m3:         GLakeServe/csrc/quantization/fp8/nvidia/quant_utils.cuh
 *                       :467-479 (quantise: sat(float(x) / scale)) and
 *                       :347-359 (dequantise: fp8 -> half -> float, * scale,
 *                       round to bf16).
 *   - prefill:          GLakeServe/csrc/cache_kernels.cu:168-190 (multi-token
 *                       append) and the causal prefix attention the backend
 *                       requests at GLakeServe/vllm/attention/backends/xformers.py:362-385.
 *   - rotary embedding: GLakeServe/csrc/cpu/pos_encoding.cpp:23-89 (NeoX pairs
 *                       (j, j + rot/2)) and :109-166 (GPT-J pairs (2j, 2j+1)):
 *                       fp32 products, one rounding to bf16, q and k in place.
 *   - rms norm:         GLakeServe/csrc/cpu/layernorm.cpp:5-41 and :44-88
 *                       (fused residual add: variance from the fp32 sums, scaling
 *                       from the sums after rounding to bf16).
 *
 * Parity pin: tests/test_oracle.py checks this file against the reference's
 * own CPU kernels compiled by oracle/build_ref.py, and against the golden
 * vectors under tests/golden/ that were generated from those kernels.
 *
 * "Device" pointers here are plain host pointers: the tables hold one base
 * address per slot exactly as the device tables do.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef uint16_t bf16_t;

static inline float bf16_to_f32(bf16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, NaN kept quiet */
static inline bf16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (bf16_t)(u >> 16);
}

/* float -> fp8 e4m3 (fn variant: no inf, max 448), round-to-nearest-even,
 * saturating to +-448 (the __NV_SATFINITE behaviour). */
uint8_t vto_f32_to_e4m3(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu); /* NaN */
  float af;
  memcpy(&af, &a, 4);
  if (af >= 448.0f) return (uint8_t)(sign | 0x7eu);
  int e = (int)(a >> 23) - 127;
  if (e < -6) { /* subnormal target: step 2^-9 */
    float q = nearbyintf(af * 512.0f);
    return (uint8_t)(sign | (uint8_t)q); /* q == 8 is the smallest normal */
  }
  uint32_t mant = a & 0x7fffffu;
  uint32_t lsb = (mant >> 20) & 1u;
  mant += 0x7ffffu + lsb;
  uint32_t q = mant >> 20;
  if (q == 8u) { q = 0u; e += 1; }
  uint32_t enc = ((uint32_t)(e + 7) << 3) | q;
  if (enc > 0x7eu) enc = 0x7eu;
  return (uint8_t)(sign | enc);
}

float vto_e4m3_to_f32(uint8_t v) {
  uint32_t e = (v >> 3) & 0xfu, m = v & 7u;
  float r;
  if (e == 0xfu && m == 7u) r = NAN;
  else if (e == 0u) r = ldexpf((float)m, -9);
  else r = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
  return (v & 0x80u) ? -r : r;
}

/* Dequantise the way the reference's scaled_convert does: the product with the
 * scale is rounded to bf16 before it is used. */
static inline float e4m3_dequant_bf16(uint8_t v, float scale) {
  return bf16_to_f32(f32_to_bf16(vto_e4m3_to_f32(v) * scale));
}

/* ------------------------------------------------------------------------- */
/* KV append                                                                  */
/* ------------------------------------------------------------------------- */

/* One call appends, for every batch entry i, rows t in [0, n_i) where
 * n_i = 1 when max_seq_len == 1 (decode) and seq_lens[i] otherwise (prefill).
 * Destination of row t: table[slot_ids[i]] + byte_off[i] + t * KVH * D * 2.
 * Source row: decode -> key + i * key_stride; prefill ->
 * key + (cache_seq_lens[i] + t) * key_stride (strides in elements).
 * A negative byte offset skips the entry (padding), as the reference does. */
void vto_append_bf16(const bf16_t *key, const bf16_t *value, int64_t key_stride,
                     int64_t value_stride, const uint64_t *k_table,
                     const uint64_t *v_table, const int64_t *byte_off,
                     const int64_t *slot_ids, const int32_t *seq_lens,
                     const int32_t *cache_seq_lens, int max_seq_len, int batch,
                     int kvh, int d) {
  const size_t row = (size_t)kvh * d;
  for (int i = 0; i < batch; ++i) {
    if (byte_off[i] < 0) continue;
    int n = (max_seq_len == 1) ? 1 : seq_lens[i];
    char *kb = (char *)(uintptr_t)k_table[slot_ids[i]] + byte_off[i];
    char *vb = (char *)(uintptr_t)v_table[slot_ids[i]] + byte_off[i];
    for (int t = 0; t < n; ++t) {
      int64_t src = (max_seq_len == 1) ? (int64_t)i : (int64_t)cache_seq_lens[i] + t;
      memcpy(kb + (size_t)t * row * 2, key + src * key_stride, row * 2);
      memcpy(vb + (size_t)t * row * 2, value + src * value_stride, row * 2);
    }
  }
}

/* fp8 e4m3 append: element (h, d) of a row is stored as
 * sat_e4m3(float(x) / scale[h]); one byte per element, row = KVH * D bytes. */
void vto_append_fp8(const bf16_t *key, const bf16_t *value, int64_t key_stride,
                    int64_t value_stride, const uint64_t *k_table,
                    const uint64_t *v_table, const int64_t *byte_off,
                    const int64_t *slot_ids, const int32_t *seq_lens,
                    const int32_t *cache_seq_lens, int max_seq_len, int batch,
                    int kvh, int d, const float *k_scale, const float *v_scale) {
  const size_t row = (size_t)kvh * d;
  for (int i = 0; i < batch; ++i) {
    if (byte_off[i] < 0) continue;
    int n = (max_seq_len == 1) ? 1 : seq_lens[i];
    uint8_t *kb = (uint8_t *)(uintptr_t)k_table[slot_ids[i]] + byte_off[i];
    uint8_t *vb = (uint8_t *)(uintptr_t)v_table[slot_ids[i]] + byte_off[i];
    for (int t = 0; t < n; ++t) {
      int64_t src = (max_seq_len == 1) ? (int64_t)i : (int64_t)cache_seq_lens[i] + t;
      const bf16_t *ks = key + src * key_stride, *vs = value + src * value_stride;
      for (int h = 0; h < kvh; ++h)
        for (int x = 0; x < d; ++x) {
          kb[(size_t)t * row + h * d + x] = vto_f32_to_e4m3(bf16_to_f32(ks[h * d + x]) / k_scale[h]);
          vb[(size_t)t * row + h * d + x] = vto_f32_to_e4m3(bf16_to_f32(vs[h * d + x]) / v_scale[h]);
        }
    }
  }
}

/* Per-kv-head scale = amax / 448 over n_tokens rows (1.0 when the head is all
 * zero, so that the division at append time is defined). */
void vto_kv_scales(const bf16_t *x, int64_t stride, int n_tokens, int kvh, int d,
                   float *scale) {
  for (int h = 0; h < kvh; ++h) {
    float amax = 0.f;
    for (int t = 0; t < n_tokens; ++t)
      for (int i = 0; i < d; ++i) {
        float v = fabsf(bf16_to_f32(x[t * stride + h * d + i]));
        if (v > amax) amax = v;
      }
    scale[h] = amax > 0.f ? amax / 448.0f : 1.0f;
  }
}

/* ------------------------------------------------------------------------- */
/* Attention                                                                  */
/* ------------------------------------------------------------------------- */

static inline float kv_elem(const void *base, size_t idx, int kv_fp8, float scale) {
  if (kv_fp8) return e4m3_dequant_bf16(((const uint8_t *)base)[idx], scale);
  return bf16_to_f32(((const bf16_t *)base)[idx]);
}

/* One query row against tokens [0, n_ctx) of one kv head. */
static void attend_row(bf16_t *out, const bf16_t *q, const void *kbase,
                       const void *vbase, int n_ctx, int kvh, int kv_head, int d,
                       float scale, int kv_fp8, float ks, float vs, float *logits,
                       float *lse_out) {
  float qf[512];
  for (int i = 0; i < d; ++i) qf[i] = bf16_to_f32(q[i]);
  float mx = -INFINITY;
  for (int t = 0; t < n_ctx; ++t) {
    size_t off = ((size_t)t * kvh + kv_head) * d;
    float acc = 0.f;
    for (int i = 0; i < d; ++i) acc += qf[i] * kv_elem(kbase, off + i, kv_fp8, ks);
    logits[t] = acc * scale;
    if (logits[t] > mx) mx = logits[t];
  }
  float sum = 0.f;
  for (int t = 0; t < n_ctx; ++t) {
    logits[t] = expf(logits[t] - mx);
    sum += logits[t];
  }
  float of[512];
  for (int i = 0; i < d; ++i) of[i] = 0.f;
  for (int t = 0; t < n_ctx; ++t) {
    float p = logits[t] / sum;
    size_t off = ((size_t)t * kvh + kv_head) * d;
    for (int i = 0; i < d; ++i) of[i] += p * kv_elem(vbase, off + i, kv_fp8, vs);
  }
  for (int i = 0; i < d; ++i) out[i] = f32_to_bf16(n_ctx > 0 ? of[i] : 0.f);
  if (lse_out) *lse_out = n_ctx > 0 ? mx + logf(sum) : -INFINITY;
}

/* Single-query decode attention.
 *   out[i, h, :] = softmax_t(scale * q[i, h] . K[t, h / g]) . V[t, h / g],
 *   t < seq_lens[i], K/V base = table[slot_ids[i]], element (t, kvh, x) at
 *   ((t * KVH + kvh) * D + x).  q_stride / out_stride in elements per batch row.
 * kv_fp8 != 0: cache bytes are e4m3 with per-kv-head scales. lse may be NULL. */
void vto_decode_attn(bf16_t *out, int64_t out_stride, const bf16_t *q,
                     int64_t q_stride, const uint64_t *k_table,
                     const uint64_t *v_table, const int64_t *slot_ids,
                     const int32_t *seq_lens, int batch, int h, int kvh, int d,
                     float scale, int kv_fp8, const float *k_scale,
                     const float *v_scale, float *lse) {
  const int g = h / kvh;
  int max_len = 1;
  for (int i = 0; i < batch; ++i)
    if (seq_lens[i] > max_len) max_len = seq_lens[i];
#pragma omp parallel
  {
    float *logits = (float *)malloc(sizeof(float) * (size_t)max_len);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int i = 0; i < batch; ++i)
      for (int hh = 0; hh < h; ++hh) {
        const void *kb = (const void *)(uintptr_t)k_table[slot_ids[i]];
        const void *vb = (const void *)(uintptr_t)v_table[slot_ids[i]];
        int kh = hh / g;
        attend_row(out + i * out_stride + (int64_t)hh * d,
                   q + i * q_stride + (int64_t)hh * d, kb, vb, seq_lens[i], kvh, kh,
                   d, scale, kv_fp8, kv_fp8 ? k_scale[kh] : 1.f,
                   kv_fp8 ? v_scale[kh] : 1.f, logits,
                   lse ? lse + (size_t)i * h + hh : NULL);
      }
    free(logits);
  }
}

/* Causal prefix attention for prefill into the contiguous range.  Batch entry
 * i contributes q_lens[i] query rows, stored from row q_start[i] of q/out
 * (row stride q_stride / out_stride elements).  Query row j of entry i sits at
 * position seq_lens[i] - q_lens[i] + j and attends tokens [0, position]. */
void vto_prefill_attn(bf16_t *out, int64_t out_stride, const bf16_t *q,
                      int64_t q_stride, const uint64_t *k_table,
                      const uint64_t *v_table, const int64_t *slot_ids,
                      const int32_t *seq_lens, const int32_t *q_lens,
                      const int32_t *q_start, int batch, int h, int kvh, int d,
                      float scale, int kv_fp8, const float *k_scale,
                      const float *v_scale) {
  const int g = h / kvh;
  int max_len = 1;
  for (int i = 0; i < batch; ++i)
    if (seq_lens[i] > max_len) max_len = seq_lens[i];
#pragma omp parallel
  {
    float *logits = (float *)malloc(sizeof(float) * (size_t)max_len);
#pragma omp for schedule(dynamic, 1)
    for (int i = 0; i < batch; ++i) {
      const void *kb = (const void *)(uintptr_t)k_table[slot_ids[i]];
      const void *vb = (const void *)(uintptr_t)v_table[slot_ids[i]];
      for (int j = 0; j < q_lens[i]; ++j) {
        int n_ctx = seq_lens[i] - q_lens[i] + j + 1;
        int64_t r = (int64_t)q_start[i] + j;
        for (int hh = 0; hh < h; ++hh) {
          int kh = hh / g;
          attend_row(out + r * out_stride + (int64_t)hh * d,
                     q + r * q_stride + (int64_t)hh * d, kb, vb, n_ctx, kvh, kh, d,
                     scale, kv_fp8, kv_fp8 ? k_scale[kh] : 1.f,
                     kv_fp8 ? v_scale[kh] : 1.f, logits, NULL);
        }
      }
    }
    free(logits);
  }
}

/* Rotary embedding of q and k in place (pos_encoding.cpp:23-89, :109-166).
 * cos_sin: bf16 [max_position, rot_dim], cos of the rot_dim/2 frequencies then sin. */
void vto_rotary_embedding(const int64_t *positions, bf16_t *query, bf16_t *key,
                          const bf16_t *cos_sin, int rot_dim, int64_t query_stride,
                          int64_t key_stride, int num_heads, int num_kv_heads,
                          int head_size, int num_tokens, int is_neox) {
  const int half = rot_dim / 2;
#pragma omp parallel for
  for (int t = 0; t < num_tokens; ++t) {
    const bf16_t *cs = cos_sin + positions[t] * rot_dim;
    for (int pass = 0; pass < 2; ++pass) {
      bf16_t *base = pass == 0 ? query + t * query_stride : key + t * key_stride;
      const int heads = pass == 0 ? num_heads : num_kv_heads;
      for (int h = 0; h < heads; ++h) {
        bf16_t *v = base + (int64_t)h * head_size;
        for (int j = 0; j < half; ++j) {
          const int xi = is_neox ? j : 2 * j, yi = is_neox ? half + j : 2 * j + 1;
          const float c = bf16_to_f32(cs[j]), s = bf16_to_f32(cs[half + j]);
          const float x = bf16_to_f32(v[xi]), y = bf16_to_f32(v[yi]);
          v[xi] = f32_to_bf16(fmaf(x, c, -(y * s)));
          v[yi] = f32_to_bf16(fmaf(y, c, x * s));
        }
      }
    }
  }
}

/* out = x * (1 / sqrt(mean(x^2) + eps)) * w; with residual != NULL first
 * x = input + residual (fp32), residual = bf16(x), and the scaling uses the
 * rounded value while the variance uses the fp32 one (layernorm.cpp:5-41, :44-88). */
void vto_rms_norm(bf16_t *out, const bf16_t *input, bf16_t *residual, const bf16_t *weight,
                  float eps, int num_tokens, int hidden) {
#pragma omp parallel for
  for (int t = 0; t < num_tokens; ++t) {
    const bf16_t *in = input + (int64_t)t * hidden;
    bf16_t *res = residual ? residual + (int64_t)t * hidden : NULL;
    bf16_t *o = out + (int64_t)t * hidden;
    float lanes[8] = {0};
    for (int j = 0; j < hidden; ++j) {
      float x = bf16_to_f32(in[j]);
      if (res) {
        x += bf16_to_f32(res[j]);
        res[j] = f32_to_bf16(x);
      }
      lanes[j & 7] = fmaf(x, x, lanes[j & 7]);
    }
    float ss = 0.f;
    for (int l = 0; l < 8; ++l) ss += lanes[l];
    const float s = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int j = 0; j < hidden; ++j) {
      const float x = bf16_to_f32(res ? res[j] : in[j]);
      o[j] = f32_to_bf16(x * s * bf16_to_f32(weight[j]));
    }
  }
}
