// The element-wise steps either side of the attention of a decoder layer, written
// so that each makes one pass over its bytes:
//
//   rope_append_kernel   rotary embedding of q (in place) and k, then the KV append
//                        of the rotated k and of v into the slots' ranges — bf16, or
//                        fp8 e4m3 quantised with the per-head scales — in ONE launch.
//                        The rotated k goes from registers to the range; it is written
//                        back to the key tensor only on request.
//   rms_norm_kernel      out = x * rsqrt(mean(x^2) + eps) * w, optionally preceded by
//                        x = input + residual with the sum stored to residual
//                        (fused_add_rms_norm).  One CTA per token row; the row stays in
//                        registers between the variance pass and the scaling pass, so a
//                        row is read once and written once.
//
// Arithmetic follows the reference's CPU kernels (fp32 products and sums, one
// rounding to bf16 per stored element): GLakeServe/csrc/cpu/pos_encoding.cpp:23-89
// (NeoX pairs (j, j + rot/2)), :109-166 (GPT-J pairs (2j, 2j+1)), and
// GLakeServe/csrc/cpu/layernorm.cpp:5-41, :44-88.  The rotation is evaluated as
// fma(x, cos, -(y * sin)) and fma(y, cos, x * sin).
// Algorithmic bytes: rope+append per token = (H + KVH) * 256 read, H * 256 written
// (q), KVH * 128 * e written twice (k, v rows), KVH * 256 read (v) + 2 * rot bytes of
// cos/sin; rms norm per token = hidden * 2 * (1 read + 1 write), doubled by the
// residual stream when fused.
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"

namespace vt {
namespace {

constexpr int kRopeThreads = 256;
constexpr int kRopeRowsPerCta = 4;

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint4 pack_bf16x8(const float *f) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ uint2 pack_e4m3x8(const float *f, float sc) {
  uint2 o;
  o.x = float2_to_e4m3x2(f[0] / sc, f[1] / sc) | (float2_to_e4m3x2(f[2] / sc, f[3] / sc) << 16);
  o.y = float2_to_e4m3x2(f[4] / sc, f[5] / sc) | (float2_to_e4m3x2(f[6] / sc, f[7] / sc) << 16);
  return o;
}
// values of a bf16x8 vector after the rounding a store to bf16 would apply
__device__ __forceinline__ void round_bf16x8(float *f) {
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(__float2bfloat16_rn(f[e]));
}

// Rotates the 8 x-elements / 8 y-elements of one work item.
//   NeoX : x = dims [c*8, c*8+8), y = the same dims + rot/2; cos/sin = 8 values each at c*8.
//   GPT-J: the 16 consecutive dims [c*16, c*16+16) hold 8 (x, y) pairs; cos/sin at c*8.
template <bool NEOX>
__device__ __forceinline__ void rotate16(float *a, float *b, const float *cs, const float *sn) {
  if constexpr (NEOX) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = a[e], y = b[e];
      a[e] = __fmaf_rn(x, cs[e], -(y * sn[e]));
      b[e] = __fmaf_rn(y, cs[e], x * sn[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float x = a[2 * e], y = a[2 * e + 1];
      a[2 * e] = __fmaf_rn(x, cs[e], -(y * sn[e]));
      a[2 * e + 1] = __fmaf_rn(y, cs[e], x * sn[e]);
      x = b[2 * e], y = b[2 * e + 1];
      b[2 * e] = __fmaf_rn(x, cs[4 + e], -(y * sn[4 + e]));
      b[2 * e + 1] = __fmaf_rn(y, cs[4 + e], x * sn[4 + e]);
    }
  }
}

struct RopeParams {
  const int64_t *positions;
  __nv_bfloat16 *query; int64_t query_stride; int num_heads;
  __nv_bfloat16 *key;
  const __nv_bfloat16 *cos_sin; int rot_dim;
  AppendParams a;
  int write_key;
};

// grid: (batch, ceil(rows / kRopeRowsPerCta)).  A work item is 16 elements of one
// head (two 16-byte vectors); items of q heads, k heads (rotate + append) and v
// heads (append only) of a row are spread over the CTA's threads.
template <bool FP8, bool NEOX>
__global__ void __launch_bounds__(kRopeThreads) rope_append_kernel(RopeParams p) {
  const int i = blockIdx.x;
  const bool decode = p.a.max_seq_len == 1;
  const int n_rows = decode ? 1 : p.a.seq_lens[i];
  const int t0 = blockIdx.y * kRopeRowsPerCta;
  if (t0 >= n_rows) return;
  const int64_t off = p.a.byte_off[i];
  const int64_t slot = p.a.slot_ids[i];
  const int kvh = p.a.kvh;
  const int64_t row_bytes = static_cast<int64_t>(kvh) * kHeadDim * (FP8 ? 1 : 2);
  char *kb = off < 0 ? nullptr : reinterpret_cast<char *>(p.a.k_table[slot]) + off;
  char *vb = off < 0 ? nullptr : reinterpret_cast<char *>(p.a.v_table[slot]) + off;
  const int half = p.rot_dim / 2;
  const int items_per_head = half / 8;                  // rotated items of a head
  const int pass_items = (kHeadDim - p.rot_dim) / 8;    // 16-byte vectors of a head beyond rot_dim (copied for k)
  const int n_q = p.num_heads * items_per_head;
  const int n_k = kvh * items_per_head;
  const int n_kpass = kvh * pass_items;
  const int n_v = kvh * (kHeadDim / 8);
  const int total = n_q + n_k + n_kpass + n_v;
  const int t1 = min(t0 + kRopeRowsPerCta, n_rows);
  for (int t = t0; t < t1; ++t) {
    const int64_t src_row = decode ? i : static_cast<int64_t>(p.a.cache_seq_lens[i]) + t;
    const int64_t pos = p.positions[src_row];
    const __nv_bfloat16 *cs_row = p.cos_sin + pos * p.rot_dim;
    __nv_bfloat16 *qrow = p.query + src_row * p.query_stride;
    __nv_bfloat16 *krow = p.key + src_row * p.a.key_stride;
    const __nv_bfloat16 *vrow = static_cast<const __nv_bfloat16 *>(p.a.value) + src_row * p.a.value_stride;
    char *kdst = kb ? kb + t * row_bytes : nullptr;
    char *vdst = vb ? vb + t * row_bytes : nullptr;
    for (int w = threadIdx.x; w < total; w += kRopeThreads) {
      if (w < n_q + n_k) {
        const bool is_k = w >= n_q;
        const int u = is_k ? w - n_q : w;
        const int head = u / items_per_head, c = u % items_per_head;
        __nv_bfloat16 *hp = (is_k ? krow : qrow) + head * kHeadDim;
        const int xa = NEOX ? c * 8 : c * 16;           // first element of vector a
        const int xb = NEOX ? half + c * 8 : c * 16 + 8;
        float a[8], b[8], cs[8], sn[8];
        Unpack<false>::run(*reinterpret_cast<const uint4 *>(hp + xa), a);
        Unpack<false>::run(*reinterpret_cast<const uint4 *>(hp + xb), b);
        Unpack<false>::run(__ldg(reinterpret_cast<const uint4 *>(cs_row + c * 8)), cs);
        Unpack<false>::run(__ldg(reinterpret_cast<const uint4 *>(cs_row + half + c * 8)), sn);
        rotate16<NEOX>(a, b, cs, sn);
        if (!is_k) {
          *reinterpret_cast<uint4 *>(hp + xa) = pack_bf16x8(a);
          *reinterpret_cast<uint4 *>(hp + xb) = pack_bf16x8(b);
        } else {
          const uint4 ra = pack_bf16x8(a), rb = pack_bf16x8(b);
          if (p.write_key) {
            *reinterpret_cast<uint4 *>(hp + xa) = ra;
            *reinterpret_cast<uint4 *>(hp + xb) = rb;
          }
          if (kdst) {
            if constexpr (!FP8) {
              *reinterpret_cast<uint4 *>(kdst + (head * kHeadDim + xa) * 2) = ra;
              *reinterpret_cast<uint4 *>(kdst + (head * kHeadDim + xb) * 2) = rb;
            } else {  // quantise the bf16-rounded rotated key, as a separate append would
              round_bf16x8(a); round_bf16x8(b);
              const float sc = p.a.k_scale[head];
              *reinterpret_cast<uint2 *>(kdst + head * kHeadDim + xa) = pack_e4m3x8(a, sc);
              *reinterpret_cast<uint2 *>(kdst + head * kHeadDim + xb) = pack_e4m3x8(b, sc);
            }
          }
        }
      } else {
        // plain row copies: k beyond rot_dim, and all of v
        int u = w - n_q - n_k;
        const bool is_v = u >= n_kpass;
        int head, x;
        if (is_v) { u -= n_kpass; head = u / (kHeadDim / 8); x = (u % (kHeadDim / 8)) * 8; }
        else { head = u / pass_items; x = p.rot_dim + (u % pass_items) * 8; }
        char *dst = is_v ? vdst : kdst;
        if (!dst) continue;
        const uint4 v = *reinterpret_cast<const uint4 *>((is_v ? vrow : krow) + head * kHeadDim + x);
        if constexpr (!FP8) {
          *reinterpret_cast<uint4 *>(dst + (head * kHeadDim + x) * 2) = v;
        } else {
          float f[8];
          Unpack<false>::run(v, f);
          *reinterpret_cast<uint2 *>(dst + head * kHeadDim + x) = pack_e4m3x8(f, (is_v ? p.a.v_scale : p.a.k_scale)[head]);
        }
      }
    }
  }
}

// ---- RMS norm ------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;    // 16-byte vectors a thread keeps: rows up to 256 * 8 * 8 = 16384 elements

__device__ __forceinline__ float cta_sum(float v, float *red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) s += red[w];
  return s;
}

// ADD: x = input + residual (fp32), residual = bf16(x), out (= input) = bf16(bf16(x) * s * w);
// the variance uses the unrounded sums, the scaling the rounded ones (layernorm.cpp:56-85).
template <bool ADD>
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *input,
                                                                 __nv_bfloat16 *residual, const __nv_bfloat16 *weight,
                                                                 float eps, int hidden, int64_t in_stride,
                                                                 int64_t out_stride) {
  __shared__ float red[kNormThreads / 32];
  const int64_t row = blockIdx.x;
  const uint4 *in = reinterpret_cast<const uint4 *>(input + row * in_stride);
  uint4 *res = ADD ? reinterpret_cast<uint4 *>(residual + row * static_cast<int64_t>(hidden)) : nullptr;
  const int n_vec = hidden / 8;
  uint4 keep[kNormMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNormMaxVec; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < n_vec) {
      const uint4 raw = in[v];
      float f[8];
      Unpack<false>::run(raw, f);
      if constexpr (ADD) {
        float r[8];
        Unpack<false>::run(res[v], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += r[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = __fmaf_rn(f[e], f[e], ss);
      keep[j] = ADD ? pack_bf16x8(f) : raw;
      if constexpr (ADD) res[v] = keep[j];
    }
  }
  const float s = 1.0f / sqrtf(cta_sum(ss, red) / static_cast<float>(hidden) + eps);
  uint4 *o = reinterpret_cast<uint4 *>(out + row * out_stride);
  const uint4 *wv = reinterpret_cast<const uint4 *>(weight);
#pragma unroll
  for (int j = 0; j < kNormMaxVec; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < n_vec) {
      float f[8], w[8];
      Unpack<false>::run(keep[j], f);
      Unpack<false>::run(__ldg(wv + v), w);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = f[e] * s * w[e];
      o[v] = pack_bf16x8(f);
    }
  }
}

}  // namespace
}  // namespace vt

extern "C" {

int vt_rope_append(const int64_t *positions, void *query, int64_t query_stride, int num_heads, void *key,
                   const void *value, int64_t key_stride, int64_t value_stride, const void *cos_sin_cache,
                   int rot_dim, int is_neox, const uint64_t *k_table, const uint64_t *v_table,
                   const int64_t *byte_off, const int64_t *slot_ids, const int32_t *seq_lens,
                   const int32_t *cache_seq_lens, int max_seq_len, int batch, int kvh, int d, int kv_dtype,
                   const float *k_scale, const float *v_scale, unsigned flags, void *stream) {
  if (batch < 0 || kvh <= 0 || num_heads <= 0 || max_seq_len < 1) return VT_ERR_INVALID;
  if (batch == 0) return VT_OK;
  if (!positions || !query || !key || !value || !cos_sin_cache || !k_table || !v_table || !byte_off || !slot_ids)
    return VT_ERR_INVALID;
  if (d != vt::kHeadDim) return VT_ERR_UNSUPPORTED;
  if (rot_dim <= 0 || rot_dim > d || rot_dim % 16 != 0) return VT_ERR_UNSUPPORTED;
  if (kv_dtype != VT_KV_BF16 && kv_dtype != VT_KV_FP8_E4M3) return VT_ERR_UNSUPPORTED;
  if (kv_dtype == VT_KV_FP8_E4M3 && (!k_scale || !v_scale)) return VT_ERR_INVALID;
  if (max_seq_len > 1 && (!seq_lens || !cache_seq_lens)) return VT_ERR_INVALID;
  if (flags & ~VT_ROPE_WRITE_KEY) return VT_ERR_INVALID;
  if (query_stride < static_cast<int64_t>(num_heads) * d || key_stride < static_cast<int64_t>(kvh) * d ||
      value_stride < static_cast<int64_t>(kvh) * d)
    return VT_ERR_INVALID;
  // 16-byte vector accesses throughout: rows of q, k, v and of the cos/sin table must allow them
  // (range rows always do: bases are 2 MiB aligned and rows are multiples of 128 bytes).
  if (((reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
        reinterpret_cast<uintptr_t>(cos_sin_cache)) & 15) != 0 ||
      query_stride % 8 != 0 || key_stride % 8 != 0 || value_stride % 8 != 0)
    return VT_ERR_UNSUPPORTED;
  vt::RopeParams p;
  p.positions = positions;
  p.query = static_cast<__nv_bfloat16 *>(query); p.query_stride = query_stride; p.num_heads = num_heads;
  p.key = static_cast<__nv_bfloat16 *>(key);
  p.cos_sin = static_cast<const __nv_bfloat16 *>(cos_sin_cache); p.rot_dim = rot_dim;
  p.a = vt::AppendParams{key, value, key_stride, value_stride, k_table, v_table, byte_off, slot_ids,
                         seq_lens, cache_seq_lens, max_seq_len, batch, kvh, k_scale, v_scale};
  p.write_key = (flags & VT_ROPE_WRITE_KEY) ? 1 : 0;
  const bool decode = max_seq_len == 1;
  dim3 grid(batch, decode ? 1 : (max_seq_len + vt::kRopeRowsPerCta - 1) / vt::kRopeRowsPerCta);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool fp8 = kv_dtype == VT_KV_FP8_E4M3;
  if (fp8 && is_neox) vt::rope_append_kernel<true, true><<<grid, vt::kRopeThreads, 0, s>>>(p);
  else if (fp8) vt::rope_append_kernel<true, false><<<grid, vt::kRopeThreads, 0, s>>>(p);
  else if (is_neox) vt::rope_append_kernel<false, true><<<grid, vt::kRopeThreads, 0, s>>>(p);
  else vt::rope_append_kernel<false, false><<<grid, vt::kRopeThreads, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

static int norm_checks(const void *out, const void *input, const void *weight, int num_tokens, int hidden,
                       int64_t in_stride, int64_t out_stride) {
  if (num_tokens < 0 || hidden <= 0) return VT_ERR_INVALID;
  if (num_tokens == 0) return VT_OK;
  if (!out || !input || !weight) return VT_ERR_INVALID;
  if (hidden % 8 != 0 || hidden > vt::kNormThreads * vt::kNormMaxVec * 8) return VT_ERR_UNSUPPORTED;
  if (in_stride < hidden || out_stride < hidden || in_stride % 8 != 0 || out_stride % 8 != 0) return VT_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight)) & 15) != 0)
    return VT_ERR_UNSUPPORTED;
  return -1;   // go on
}

int vt_rms_norm(void *out, const void *input, const void *weight, float epsilon, int num_tokens, int hidden,
                int64_t input_stride, int64_t out_stride, void *stream) {
  const int st = norm_checks(out, input, weight, num_tokens, hidden, input_stride, out_stride);
  if (st >= 0) return st;
  vt::rms_norm_kernel<false><<<num_tokens, vt::kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(input), nullptr,
      static_cast<const __nv_bfloat16 *>(weight), epsilon, hidden, input_stride, out_stride);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

int vt_fused_add_rms_norm(void *input, void *residual, const void *weight, float epsilon, int num_tokens, int hidden,
                          void *stream) {
  const int st = norm_checks(input, input, weight, num_tokens, hidden, hidden, hidden);
  if (st >= 0) return st;
  if (!residual || (reinterpret_cast<uintptr_t>(residual) & 15) != 0) return VT_ERR_INVALID;
  vt::rms_norm_kernel<true><<<num_tokens, vt::kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(input), static_cast<const __nv_bfloat16 *>(input),
      static_cast<__nv_bfloat16 *>(residual), static_cast<const __nv_bfloat16 *>(weight), epsilon, hidden, hidden,
      hidden);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

}  // extern "C"
