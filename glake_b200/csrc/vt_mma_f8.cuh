// Per-warp decode attention over an fp8 e4m3 cache with the contraction done by
// fp8 tensor-core instructions (mma.sync.m16n8k32.e4m3.e4m3.f32), so that no K or V
// byte is ever converted: the cache bytes go from shared memory straight into the
// MMA operands.  (Converting them to f16 first costs one cvt per two elements on a
// pipe that saturates long before HBM does.)
//
// What makes that possible without losing accuracy:
//  * Q (bf16) is split once per piece into two e4m3 terms, q * 2^k = q_hi + q_lo with
//    a per-head power-of-two 2^k that puts the head's largest |q| into [128, 256):
//    together they carry ~8 significant bits, as bf16 does.  Q.K^T is the sum of two
//    MMAs per 32 dims; 2^-k is folded into the logit scale.
//  * P (fp32 probabilities) is split per tile into two e4m3 terms of 256 * p.  The
//    factor never has to be removed: the running maximum is tracked as (max - 8) in
//    the log2 domain, so p' = exp2(s - m') <= 256, and both the row sums and the
//    O accumulators carry the same factor, which cancels in O / l, in the merge of
//    partial states and in lse = m' + log2(l').
//  * A 16-token tile only fills half of the instruction's k = 32; the other half
//    takes the same V bytes again, paired with the low term of P, so V . (P_hi + P_lo)
//    is ONE instruction per 16 output dims.
//  * The order of the terms of a dot product is free, so the MMA's k index is mapped
//    to whatever bytes a lane can fetch with plain 16-byte shared-memory loads:
//      Q.K^T:  k col (4 c4 + i) of step s        <->  d = 32 c4 + 8 s + i      (i = 0..3)
//              k col (16 + 4 c4 + i)             <->  d = 32 c4 + 8 s + 4 + i
//      P.V:    k col (4 c4 + i)                  <->  token {2 c4, 2 c4 + 1, 2 c4 + 8, 2 c4 + 9}[i]
//    and V's bytes of 4 tokens x 4 dims are transposed in registers with byte permutes.
#pragma once
#include "vt_mma.cuh"

namespace vt {

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Largest-magnitude-first split of two floats into e4m3 terms, exact rounding:
// hi = rn(x), lo = rn(x - hi).  Returns the two 16-bit pairs {x0 | x1 << 8}.
__device__ __forceinline__ void split_e4m3x2_rn(float x0, float x1, uint32_t *hi16, uint32_t *lo16) {
  const uint32_t h = float2_to_e4m3x2(x0, x1);
  const uint32_t hf = e4m3x2_to_f16x2(h);
  *hi16 = h;
  *lo16 = float2_to_e4m3x2(x0 - f16_lo(hf), x1 - f16_hi(hf));
}

template <int NB>
struct WarpAttnF8 {
  static constexpr int kRowBytes = 128;   // one kv head's row in the cache
  static constexpr int kWarps = 8;        // consumer warps per CTA = rows per 1 KiB group
  __device__ __forceinline__ static int dim_of(int mb, int half, int r4) { return 16 * r4 + 2 * mb + half; }
  uint32_t qh[NB][4][2], ql[NB][4][2];    // Q^T operands of the 4 k-steps, high and low e4m3 terms
  float qinv[NB][2];                      // 2^-k of the heads this lane holds accumulator columns of
  float o[NB][8][4];
  float mrun[NB][2], lrun[NB][2];         // running (max - 8) in the log2 domain; sum of 256 * p

  __device__ __forceinline__ void start(const __nv_bfloat16 *qrow, int g, int lane) {
    const int r4 = lane >> 2, c4 = lane & 3;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int head = nb * 8 + r4;
      float x[32];
      float amax = 0.f;
      if (head < g) {
        const uint4 *src = reinterpret_cast<const uint4 *>(qrow + head * kHeadDim + 32 * c4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = __ldg(src + j);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            x[8 * j + 2 * u] = bf16_lo(w[u]);
            x[8 * j + 2 * u + 1] = bf16_hi(w[u]);
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = 0.f;
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // amax = 1.m x 2^E  ->  k = 7 - E puts it into [128, 256); bf16 inputs are never
      // fp32-subnormal, an all-zero (or non-finite) head keeps k = 0
      const int E = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 127;
      const int k = (E <= -127 || E >= 128) ? 0 : max(-100, min(100, 7 - E));
      const float up = __uint_as_float(static_cast<uint32_t>(127 + k) << 23);
      const float down = __uint_as_float(static_cast<uint32_t>(127 - k) << 23);
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        uint32_t h[4], l[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) split_e4m3x2_rn(x[8 * s + 2 * u] * up, x[8 * s + 2 * u + 1] * up, &h[u], &l[u]);
        qh[nb][s][0] = h[0] | (h[1] << 16);
        qh[nb][s][1] = h[2] | (h[3] << 16);
        ql[nb][s][0] = l[0] | (l[1] << 16);
        ql[nb][s][1] = l[2] | (l[3] << 16);
      }
      // accumulator columns of this lane are heads nb*8 + 2 c4 and + 1: their 2^-k
      qinv[nb][0] = __shfl_sync(0xffffffffu, down, 8 * c4);
      qinv[nb][1] = __shfl_sync(0xffffffffu, down, 8 * c4 + 4);
      mrun[nb][0] = mrun[nb][1] = -INFINITY;
      lrun[nb][0] = lrun[nb][1] = 0.f;
#pragma unroll
      for (int mb = 0; mb < 8; ++mb) o[nb][mb][0] = o[nb][mb][1] = o[nb][mb][2] = o[nb][mb][3] = 0.f;
    }
  }

  // Arguments as WarpAttn::tile (k_off / v_off unused: offsets follow from lane and row_off).
  __device__ __forceinline__ void tile(uint32_t, unsigned char *st_generic, uint32_t, uint32_t, uint32_t row_off,
                                       int n_rows, float sl2, int lane) {
    const int r4 = lane >> 2, c4 = lane & 3;
    if (n_rows < 16) {   // ragged end: clear stale V rows (a stale NaN byte times P = 0 would poison the sums)
      for (int r = n_rows + (lane >> 3); r < 16; r += 4)
        *reinterpret_cast<uint4 *>(st_generic + kTileB + r * kPitch + row_off + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
      __syncwarp();
    }
    // ---- S^T = K . Q^T : rows = tokens r4 / r4 + 8, this lane's 32 bytes of each ----
    float sacc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
    {
      const unsigned char *ka = st_generic + r4 * kPitch + row_off + 32 * c4;
      const uint4 a_lo = *reinterpret_cast<const uint4 *>(ka), a_hi = *reinterpret_cast<const uint4 *>(ka + 16);
      const uint4 b_lo = *reinterpret_cast<const uint4 *>(ka + 8 * kPitch),
                  b_hi = *reinterpret_cast<const uint4 *>(ka + 8 * kPitch + 16);
      const uint32_t wa[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
      const uint32_t wb[8] = {b_lo.x, b_lo.y, b_lo.z, b_lo.w, b_hi.x, b_hi.y, b_hi.z, b_hi.w};
#pragma unroll
      for (int s = 0; s < 4; ++s) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mma_e4m3(sacc[nb], wa[2 * s], wb[2 * s], wa[2 * s + 1], wb[2 * s + 1], qh[nb][s][0], qh[nb][s][1]);
          mma_e4m3(sacc[nb], wa[2 * s], wb[2 * s], wa[2 * s + 1], wb[2 * s + 1], ql[nb][s][0], ql[nb][s][1]);
        }
      }
    }
    // ---- online softmax; probabilities are kept as 256 * p (see the file comment) ----
    const bool v0 = r4 < n_rows, v1 = r4 + 8 < n_rows;
    uint32_t pb[NB][2];   // P^T operand: high terms (k cols 0..15) and low terms (k cols 16..31)
    bool any_up = false;
    float fac[NB][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const float c0 = sl2 * qinv[nb][0], c1 = sl2 * qinv[nb][1];
      float s00 = v0 ? sacc[nb][0] * c0 : -INFINITY, s01 = v0 ? sacc[nb][1] * c1 : -INFINITY;
      float s10 = v1 ? sacc[nb][2] * c0 : -INFINITY, s11 = v1 ? sacc[nb][3] * c1 : -INFINITY;
      float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(mrun[nb][0], mx0 - 8.f), mn1 = fmaxf(mrun[nb][1], mx1 - 8.f);
      fac[nb][0] = exp2f(mrun[nb][0] - mn0);   // mn is finite: fragment row 0 is valid
      fac[nb][1] = exp2f(mrun[nb][1] - mn1);
      any_up |= (mn0 > mrun[nb][0]) | (mn1 > mrun[nb][1]);
      mrun[nb][0] = mn0;
      mrun[nb][1] = mn1;
      const float p00 = exp2f(s00 - mn0), p01 = exp2f(s01 - mn1), p10 = exp2f(s10 - mn0), p11 = exp2f(s11 - mn1);
      lrun[nb][0] = lrun[nb][0] * fac[nb][0] + p00 + p10;
      lrun[nb][1] = lrun[nb][1] * fac[nb][1] + p01 + p11;
      // high term = the float cut to 4 significant bits (exact in e4m3 for p' >= 2^-6; below
      // that the rounding of the conversion differs by < 2^-18 of the row's largest weight),
      // low term = the rest, rounded: ~7 significant bits together
      const float h00 = __uint_as_float(__float_as_uint(p00) & 0xfff00000u), h01 = __uint_as_float(__float_as_uint(p01) & 0xfff00000u);
      const float h10 = __uint_as_float(__float_as_uint(p10) & 0xfff00000u), h11 = __uint_as_float(__float_as_uint(p11) & 0xfff00000u);
      const uint32_t hi0 = float2_to_e4m3x2(h00, h01), lo0 = float2_to_e4m3x2(p00 - h00, p01 - h01);
      const uint32_t hi1 = float2_to_e4m3x2(h10, h11), lo1 = float2_to_e4m3x2(p10 - h10, p11 - h11);
      // 16-bit elements {high byte-term, low byte-term} per (token, head), transposed as b16
      const uint32_t m0 = movmatrix_trans(prmt(hi0, lo0, 0x5140u));   // tokens 2 c4, 2 c4 + 1 of head r4
      const uint32_t m1 = movmatrix_trans(prmt(hi1, lo1, 0x5140u));   // tokens 2 c4 + 8, 2 c4 + 9
      pb[nb][0] = prmt(m0, m1, 0x6420u);
      pb[nb][1] = prmt(m0, m1, 0x7531u);
    }
    if (__any_sync(0xffffffffu, any_up)) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int mb = 0; mb < 8; ++mb) {
          o[nb][mb][0] *= fac[nb][0]; o[nb][mb][1] *= fac[nb][1];
          o[nb][mb][2] *= fac[nb][0]; o[nb][mb][3] *= fac[nb][1];
        }
    }
    // ---- O^T += V^T . P^T : rows = dims 16 r4 + 2 mb (+ 1), k = this lane's 4 tokens ----
    {
      const unsigned char *va = st_generic + kTileB + row_off + 16 * r4;
      const uint4 t0 = *reinterpret_cast<const uint4 *>(va + (2 * c4) * kPitch);
      const uint4 t1 = *reinterpret_cast<const uint4 *>(va + (2 * c4 + 1) * kPitch);
      const uint4 t2 = *reinterpret_cast<const uint4 *>(va + (2 * c4 + 8) * kPitch);
      const uint4 t3 = *reinterpret_cast<const uint4 *>(va + (2 * c4 + 9) * kPitch);
      const uint32_t w0[4] = {t0.x, t0.y, t0.z, t0.w}, w1[4] = {t1.x, t1.y, t1.z, t1.w};
      const uint32_t w2[4] = {t2.x, t2.y, t2.z, t2.w}, w3[4] = {t3.x, t3.y, t3.z, t3.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // 4 x 4 byte transpose: x[b] = byte b of the four tokens' word j
        const uint32_t u0 = prmt(w0[j], w1[j], 0x5140u), u1 = prmt(w0[j], w1[j], 0x7362u);
        const uint32_t u2 = prmt(w2[j], w3[j], 0x5140u), u3 = prmt(w2[j], w3[j], 0x7362u);
        const uint32_t x0 = prmt(u0, u2, 0x5410u), x1 = prmt(u0, u2, 0x7632u);
        const uint32_t x2 = prmt(u1, u3, 0x5410u), x3 = prmt(u1, u3, 0x7632u);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mma_e4m3(o[nb][2 * j], x0, x1, x0, x1, pb[nb][0], pb[nb][1]);
          mma_e4m3(o[nb][2 * j + 1], x2, x3, x2, x3, pb[nb][0], pb[nb][1]);
        }
      }
    }
  }

  __device__ __forceinline__ void finish_sums() {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        lrun[nb][0] += __shfl_xor_sync(0xffffffffu, lrun[nb][0], off);
        lrun[nb][1] += __shfl_xor_sync(0xffffffffu, lrun[nb][1], off);
      }
  }

  template <int ROW>
  __device__ __forceinline__ void store(float *dst, int lane, int g) const {
    const int r4 = lane >> 2, c4 = lane & 3;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int h0 = nb * 8 + 2 * c4;
#pragma unroll
      for (int mb = 0; mb < 8; ++mb) {
        const int d0 = dim_of(mb, 0, r4), d1 = dim_of(mb, 1, r4);
        if (h0 < g) {
          dst[h0 * ROW + d0] = o[nb][mb][0];
          dst[h0 * ROW + d1] = o[nb][mb][2];
        }
        if (h0 + 1 < g) {
          dst[(h0 + 1) * ROW + d0] = o[nb][mb][1];
          dst[(h0 + 1) * ROW + d1] = o[nb][mb][3];
        }
      }
      if (r4 == 0) {
        if (h0 < g) {
          dst[h0 * ROW + 128] = mrun[nb][0];
          dst[h0 * ROW + 129] = lrun[nb][0];
        }
        if (h0 + 1 < g) {
          dst[(h0 + 1) * ROW + 128] = mrun[nb][1];
          dst[(h0 + 1) * ROW + 129] = lrun[nb][1];
        }
      }
    }
  }
};

}  // namespace vt
