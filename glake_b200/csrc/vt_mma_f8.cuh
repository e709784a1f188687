// Per-warp decode attention over an fp8 e4m3 cache (the fp8 counterpart of WarpAttn in
// vt_mma.cuh).
//
// Why the bytes are widened to f16 with cvt and multiplied by the legacy f16 MMA, although
// that costs one conversion per two elements on the XU pipe: both alternatives were built
// and measured on B200 (batch 128, 32 q / 8 kv heads, contexts 2k-8k: 268 us this way).
//  * mma.sync.m16n8k32 with e4m3 operands (Q and P carried as two e4m3 terms, so that no
//    K or V byte is converted): 338 us.  On sm_100a that legacy instruction is not a native
//    fp8 operation: ncu shows the XU pipe above 100 % of its sustained rate and the f16 MMA
//    sub-pipe busy 94 % of the time, i.e. the hardware converts and runs it at a fraction
//    of the f16 rate.  Native fp8 on this part exists only as tcgen05.mma.kind::f8f6f4.
//  * converting K with integer operations (prmt / shift / lop3 give the f16 pattern up to a
//    factor 2^-8) while V stays on cvt, to split the work between the ALU and XU pipes: 315 us;
//    the extra instructions cost more issue slots than the freed XU cycles give back.
#pragma once
#include "vt_mma.cuh"

namespace vt {

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// A kv head's row is 128 bytes, a
// 1 KiB group holds 8 rows, so a CTA runs 8 consumer warps.  e4m3 converts to f16
// exactly, so the contraction runs as f16 MMAs with Q converted bf16 -> f16 (rounded
// to nearest; saturating, which only matters beyond |q| = 65504).  Fragments are
// built from plain 16-byte shared-memory loads, not ldmatrix: the sum over d does
// not care about the order of d, so lane (r4, c4) simply owns bytes [32 c4, 32 c4 + 32)
// of its two K rows and Q is loaded with the same permutation
//   MMA k index (step s, 2 c4 + j)     <->  d = 32 c4 + 4 s + j        (j = 0, 1)
//   MMA k index (step s, 2 c4 + 8 + j) <->  d = 32 c4 + 4 s + 2 + j
// and likewise lane r4 owns output dims [16 r4, 16 r4 + 16) of V:
//   accumulator tile mb, fragment rows r4 / r4 + 8   <->  d = 16 r4 + 2 mb / + 1.
// With groups at a 1040-byte pitch both load patterns are bank-conflict free.
// The per-head scales are folded in: k_scale into the logit scale, v_scale into the
// output.
template <int NB>
struct WarpAttnF8 {
  static constexpr int kRowBytes = 128;
  static constexpr int kWarps = 8;
  __device__ __forceinline__ static int dim_of(int mb, int half, int r4) { return 16 * r4 + 2 * mb + half; }
  uint32_t qb[NB][8][2];
  float o[NB][8][4];
  float mrun[NB][2], lrun[NB][2];

  __device__ __forceinline__ void start(const __nv_bfloat16 *qrow, int g, int lane) {
    const int r4 = lane >> 2, c4 = lane & 3;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int head = nb * 8 + r4;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        if (head < g) {
          const uint2 v = __ldg(reinterpret_cast<const uint2 *>(qrow + head * kHeadDim + 32 * c4 + 4 * ks));
          qb[nb][ks][0] = pack_f16(bf16_lo(v.x), bf16_hi(v.x));
          qb[nb][ks][1] = pack_f16(bf16_lo(v.y), bf16_hi(v.y));
        } else {
          qb[nb][ks][0] = qb[nb][ks][1] = 0u;
        }
      }
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
    if (n_rows < 16) {   // ragged end: clear stale V rows (0 * NaN would poison the accumulators)
      for (int r = n_rows + (lane >> 3); r < 16; r += 4)
        *reinterpret_cast<uint4 *>(st_generic + kTileB + r * kPitch + row_off + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
      __syncwarp();
    }
    // ---- S^T = K . Q^T ----
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
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        a[0] = e4m3x2_to_f16x2(wa[ks]);
        a[1] = e4m3x2_to_f16x2(wb[ks]);
        a[2] = e4m3x2_to_f16x2(wa[ks] >> 16);
        a[3] = e4m3x2_to_f16x2(wb[ks] >> 16);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_f16(sacc[nb], a, qb[nb][ks][0], qb[nb][ks][1]);
      }
    }
    // ---- online softmax ----
    const bool v0 = r4 < n_rows, v1 = r4 + 8 < n_rows;
    uint32_t pb[NB][2];
    bool any_up = false;
    float fac[NB][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float s00 = v0 ? sacc[nb][0] * sl2 : -INFINITY, s01 = v0 ? sacc[nb][1] * sl2 : -INFINITY;
      float s10 = v1 ? sacc[nb][2] * sl2 : -INFINITY, s11 = v1 ? sacc[nb][3] * sl2 : -INFINITY;
      float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(mrun[nb][0], mx0), mn1 = fmaxf(mrun[nb][1], mx1);
      fac[nb][0] = exp2f(mrun[nb][0] - mn0);
      fac[nb][1] = exp2f(mrun[nb][1] - mn1);
      any_up |= (mn0 > mrun[nb][0]) | (mn1 > mrun[nb][1]);
      mrun[nb][0] = mn0;
      mrun[nb][1] = mn1;
      const float p00 = exp2f(s00 - mn0), p01 = exp2f(s01 - mn1), p10 = exp2f(s10 - mn0), p11 = exp2f(s11 - mn1);
      lrun[nb][0] = lrun[nb][0] * fac[nb][0] + p00 + p10;
      lrun[nb][1] = lrun[nb][1] * fac[nb][1] + p01 + p11;
      // f16 probabilities carry 11 mantissa bits: ample next to the 3-bit mantissa of
      // the e4m3 values they weigh, so no hi + lo split here.
      pb[nb][0] = movmatrix_trans(pack_f16(p00, p01));
      pb[nb][1] = movmatrix_trans(pack_f16(p10, p11));
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
    // ---- O^T += V^T . P^T ----
    {
      const unsigned char *va = st_generic + kTileB + row_off + 16 * r4;
      const uint4 t0 = *reinterpret_cast<const uint4 *>(va + (2 * c4) * kPitch);
      const uint4 t1 = *reinterpret_cast<const uint4 *>(va + (2 * c4 + 1) * kPitch);
      const uint4 t2 = *reinterpret_cast<const uint4 *>(va + (2 * c4 + 8) * kPitch);
      const uint4 t3 = *reinterpret_cast<const uint4 *>(va + (2 * c4 + 9) * kPitch);
      const uint32_t w0[4] = {t0.x, t0.y, t0.z, t0.w}, w1[4] = {t1.x, t1.y, t1.z, t1.w};
      const uint32_t w2[4] = {t2.x, t2.y, t2.z, t2.w}, w3[4] = {t3.x, t3.y, t3.z, t3.w};
#pragma unroll
      for (int mb = 0; mb < 8; ++mb) {
        const int w = mb >> 1;
        const uint32_t lo = (mb & 1) ? 0x62u : 0x40u;   // byte (2 mb) % 4 of both words
        const uint32_t hi = (mb & 1) ? 0x73u : 0x51u;   // the byte after it
        uint32_t a[4];
        a[0] = e4m3x2_to_f16x2(prmt(w0[w], w1[w], lo));
        a[1] = e4m3x2_to_f16x2(prmt(w0[w], w1[w], hi));
        a[2] = e4m3x2_to_f16x2(prmt(w2[w], w3[w], lo));
        a[3] = e4m3x2_to_f16x2(prmt(w2[w], w3[w], hi));
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_f16(o[nb][mb], a, pb[nb][0], pb[nb][1]);
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
