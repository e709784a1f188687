// KV append into the per-slot contiguous ranges (the reshape_and_cache of the
// vTensor path).  bf16: a bit-exact row copy with 16-byte vector accesses.
// fp8 e4m3: byte = sat(x / scale[kv_head]), 16 bytes in, 8 bytes out per thread.
// Algorithmic bytes per appended row: kvh*128*(2 + e) for K plus the same for V.
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"

namespace vt {
namespace {

constexpr int kAppendThreads = 256;
constexpr int kPrefillRowsPerCta = 8;

template <bool FP8>
__device__ __forceinline__ void copy_row(const __nv_bfloat16 *src, char *dst, int n_elems, const float *scale,
                                         bool vec_ok) {
  if (vec_ok) {
    const uint4 *s = reinterpret_cast<const uint4 *>(src);
    for (int i = threadIdx.x; i < n_elems / 8; i += blockDim.x) {
      uint4 v = __ldg(s + i);
      if constexpr (!FP8) {
        reinterpret_cast<uint4 *>(dst)[i] = v;
      } else {
        // true division (not a reciprocal multiply) so bytes equal sat(x / scale) exactly
        const float sc = scale[(i * 8) / kHeadDim];
        float f[8];
        Unpack<false>::run(v, f);
        uint2 o;
        o.x = float2_to_e4m3x2(f[0] / sc, f[1] / sc) | (float2_to_e4m3x2(f[2] / sc, f[3] / sc) << 16);
        o.y = float2_to_e4m3x2(f[4] / sc, f[5] / sc) | (float2_to_e4m3x2(f[6] / sc, f[7] / sc) << 16);
        reinterpret_cast<uint2 *>(dst)[i] = o;
      }
    }
  } else {  // unaligned source or destination: element-wise
    for (int i = threadIdx.x; i < n_elems; i += blockDim.x) {
      if constexpr (!FP8) {
        reinterpret_cast<__nv_bfloat16 *>(dst)[i] = src[i];
      } else {
        float x = __bfloat162float(src[i]) / scale[i / kHeadDim];
        reinterpret_cast<uint8_t *>(dst)[i] = static_cast<uint8_t>(float2_to_e4m3x2(x, 0.f) & 0xffu);
      }
    }
  }
}

// grid: (batch, ceil(rows / rows_per_cta)); decode has one row per entry.
template <bool FP8>
__global__ void __launch_bounds__(kAppendThreads) append_kernel(AppendParams p, int rows_per_cta, bool host_vec_ok) {
  const int i = blockIdx.x;
  const int64_t off = p.byte_off[i];
  if (off < 0) return;  // padded entry
  const bool decode = p.max_seq_len == 1;
  const int n_rows = decode ? 1 : p.seq_lens[i];
  const int t0 = blockIdx.y * rows_per_cta;
  if (t0 >= n_rows) return;
  const int64_t slot = p.slot_ids[i];
  const int n_elems = p.kvh * kHeadDim;
  const int64_t row_bytes = static_cast<int64_t>(n_elems) * (FP8 ? 1 : 2);
  char *kb = reinterpret_cast<char *>(p.k_table[slot]) + off;
  char *vb = reinterpret_cast<char *>(p.v_table[slot]) + off;
  const bool vec_ok = host_vec_ok && ((reinterpret_cast<uintptr_t>(kb) | reinterpret_cast<uintptr_t>(vb)) & 15) == 0;
  const int t1 = min(t0 + rows_per_cta, n_rows);
  for (int t = t0; t < t1; ++t) {
    const int64_t src_row = decode ? i : static_cast<int64_t>(p.cache_seq_lens[i]) + t;
    const __nv_bfloat16 *ks = static_cast<const __nv_bfloat16 *>(p.key) + src_row * p.key_stride;
    const __nv_bfloat16 *vs = static_cast<const __nv_bfloat16 *>(p.value) + src_row * p.value_stride;
    copy_row<FP8>(ks, kb + t * row_bytes, n_elems, p.k_scale, vec_ok);
    copy_row<FP8>(vs, vb + t * row_bytes, n_elems, p.v_scale, vec_ok);
  }
}

// One CTA per kv head: amax over n_tokens x 128 elements, scale = amax / 448.
__global__ void __launch_bounds__(256) kv_scales_kernel(const __nv_bfloat16 *x, int64_t stride, int n_tokens,
                                                        float *scale) {
  const int head = blockIdx.x;
  float amax = 0.f;
  for (int idx = threadIdx.x; idx < n_tokens * (kHeadDim / 8); idx += blockDim.x) {
    const int t = idx / (kHeadDim / 8), c = idx % (kHeadDim / 8);
    const __nv_bfloat16 *row = x + t * stride + head * kHeadDim + c * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(__bfloat162float(row[e])));
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    scale[head] = amax > 0.f ? amax / 448.0f : 1.0f;
  }
}

// fp8 ranges -> dense bf16 rows: x = bf16(e4m3 * scale[kv_head]), the dequantisation of the
// reference's scaled_convert (GLakeServe/csrc/quantization/fp8/nvidia/quant_utils.cuh:347-359).
// grid: (entry, row blocks); one thread widens 16 bytes to 32.
__global__ void __launch_bounds__(kAppendThreads) kv_widen_kernel(KvWidenParams p, int rows_per_cta) {
  const int i = blockIdx.x;
  const int n_rows = p.seq_lens[i];
  const int t0 = blockIdx.y * rows_per_cta;
  if (t0 >= n_rows) return;
  const int64_t slot = p.slot_ids[i];
  const int vec_per_row = p.kvh * kHeadDim / 16;
  const int t1 = min(t0 + rows_per_cta, n_rows);
#pragma unroll
  for (int kv = 0; kv < 2; ++kv) {
    const uint4 *src = reinterpret_cast<const uint4 *>(kv ? p.v_table[slot] : p.k_table[slot]);
    uint4 *dst = reinterpret_cast<uint4 *>(kv ? p.v_out[i] : p.k_out[i]);
    const float *scale = kv ? p.v_scale : p.k_scale;
    for (int idx = t0 * vec_per_row + threadIdx.x; idx < t1 * vec_per_row; idx += kAppendThreads) {
      const float sc = scale[(idx % vec_per_row) / (kHeadDim / 16)];
      float f[16];
      Unpack<true>::run(__ldg(src + idx), f);
      uint32_t w[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * e] * sc, f[2 * e + 1] * sc);
        w[e] = *reinterpret_cast<uint32_t *>(&v);
      }
      dst[2 * idx] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[2 * idx + 1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

}  // namespace

int launch_kv_widen(const KvWidenParams &p, int max_seq_len, cudaStream_t stream) {
  if (p.batch == 0 || max_seq_len <= 0) return VT_OK;
  constexpr int kRows = 32;
  dim3 grid(p.batch, (max_seq_len + kRows - 1) / kRows);
  kv_widen_kernel<<<grid, kAppendThreads, 0, stream>>>(p, kRows);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

int launch_append(const AppendParams &p, int kv_dtype, cudaStream_t stream) {
  if (p.batch == 0) return VT_OK;
  const bool decode = p.max_seq_len == 1;
  const int rows_per_cta = decode ? 1 : kPrefillRowsPerCta;
  dim3 grid(p.batch, decode ? 1 : (p.max_seq_len + rows_per_cta - 1) / rows_per_cta);
  const bool host_vec_ok = ((reinterpret_cast<uintptr_t>(p.key) | reinterpret_cast<uintptr_t>(p.value)) & 15) == 0 &&
                           (p.key_stride % 8) == 0 && (p.value_stride % 8) == 0;
  if (kv_dtype == VT_KV_BF16)
    append_kernel<false><<<grid, kAppendThreads, 0, stream>>>(p, rows_per_cta, host_vec_ok);
  else
    append_kernel<true><<<grid, kAppendThreads, 0, stream>>>(p, rows_per_cta, host_vec_ok);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

int launch_kv_scales(const void *x, int64_t stride, int n_tokens, int kvh, float *scale, cudaStream_t stream) {
  kv_scales_kernel<<<kvh, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), stride, n_tokens, scale);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

}  // namespace vt
