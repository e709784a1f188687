// Warp-level matrix helpers shared by the tensor-core attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "vt_device.cuh"

namespace vt {

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}


// ---------------------------------------------------------------------------
// Shared-memory tile geometry of the tensor-core kernels: every bulk copy moves
// one 1 KiB "group" (R consecutive tokens x HS kv heads x 256 B, R * HS = 4); a
// tile is 16 groups at a 1040-byte pitch, K tile followed by V tile per stage.
// ---------------------------------------------------------------------------
constexpr int kMmaStages = 3;
constexpr int kMmaCWarps = 4;
constexpr int kMmaThreads = (kMmaCWarps + 1) * 32;
constexpr int kGroupsPerTile = 16;
constexpr int kRowB = 256;                    // bf16 row of one kv head
constexpr int kGroupB = kMmaCWarps * kRowB;   // 1 KiB per bulk copy
constexpr int kPitch = kGroupB + 16;          // pitch between groups
constexpr int kTileB = kGroupsPerTile * kPitch;
constexpr int kStageB = 2 * kTileB;

// Per-warp attention state for one kv head: Q^T fragments of its q heads, the
// O^T accumulator and the running softmax statistics.
//   qb[nb][ks][0/1] = Q[head nb*8 + lane/4][16*ks + 2*(lane%4) (+8) .. +1]
//   o[nb][mb]       = m16n8 tile: d = 16*mb + lane/4 (+8), heads nb*8 + 2*(lane%4) + {0,1}
template <int NB>
struct WarpAttn {
  static constexpr int kRowBytes = 256;   // one kv head's row in the cache
  static constexpr int kWarps = 4;        // consumer warps per CTA = rows per 1 KiB group
  // output dim held by accumulator tile mb, fragment-row half (0: row r4, 1: row r4 + 8)
  __device__ __forceinline__ static int dim_of(int mb, int half, int r4) { return mb * 16 + r4 + 8 * half; }
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
          const uint32_t *src = reinterpret_cast<const uint32_t *>(qrow + head * kHeadDim + ks * 16 + 2 * c4);
          qb[nb][ks][0] = __ldg(src);
          qb[nb][ks][1] = __ldg(src + 4);
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

  // One tile: fragment row i of this warp is its row of group i.  n_rows (1..16)
  // fragment rows are inside the context.  st = shared address of the stage,
  // st_generic the same as a generic pointer; k_off / v_off are the per-lane
  // ldmatrix offsets, row_off the byte offset of the warp's row inside a group.
  __device__ __forceinline__ void tile(uint32_t st, unsigned char *st_generic, uint32_t k_off, uint32_t v_off,
                                       uint32_t row_off, int n_rows, float sl2, int lane) {
    const int r4 = lane >> 2;
    if (n_rows < 16) {
      // Ragged end: rows past the context hold stale bytes.  Their K only feeds
      // logits that are masked below; their V would be multiplied by P = 0, and
      // 0 * NaN is NaN, so clear them.
      for (int r = n_rows + (lane >> 4); r < 16; r += 2)
        *reinterpret_cast<uint4 *>(st_generic + kTileB + r * kPitch + row_off + (lane & 15) * 16) =
            make_uint4(0, 0, 0, 0);
      __syncwarp();
    }
    // ---- S^T = K . Q^T ----
    float sacc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(st + k_off + ks * 32, a);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) mma_bf16(sacc[nb], a, qb[nb][ks][0], qb[nb][ks][1]);
    }
    // ---- online softmax (rows = fragment rows r4, r4+8; cols = heads 2*c4, 2*c4+1) ----
    const bool v0 = r4 < n_rows, v1 = r4 + 8 < n_rows;
    uint32_t pb[NB][2], pl[NB][2];   // P^T split into bf16 high and low parts
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
      fac[nb][0] = exp2f(mrun[nb][0] - mn0);   // mn is finite: fragment row 0 is valid
      fac[nb][1] = exp2f(mrun[nb][1] - mn1);
      any_up |= (mn0 > mrun[nb][0]) | (mn1 > mrun[nb][1]);
      mrun[nb][0] = mn0;
      mrun[nb][1] = mn1;
      const float p00 = exp2f(s00 - mn0), p01 = exp2f(s01 - mn1), p10 = exp2f(s10 - mn0), p11 = exp2f(s11 - mn1);
      lrun[nb][0] = lrun[nb][0] * fac[nb][0] + p00 + p10;   // this lane's share; summed over lanes at the end
      lrun[nb][1] = lrun[nb][1] * fac[nb][1] + p01 + p11;
      // P is kept to ~16 mantissa bits as hi + lo bf16 halves (two MMAs per V
      // fragment; the tensor pipe is idle anyway), so the result tracks fp32
      // probabilities instead of bf16-rounded ones.  Then accumulator layout ->
      // B-operand layout of P^T.
      const uint32_t h0 = pack_bf16(p00, p01), h1 = pack_bf16(p10, p11);
      const uint32_t l0 = pack_bf16(p00 - bf16_lo(h0), p01 - bf16_hi(h0));
      const uint32_t l1 = pack_bf16(p10 - bf16_lo(h1), p11 - bf16_hi(h1));
      pb[nb][0] = movmatrix_trans(h0);
      pb[nb][1] = movmatrix_trans(h1);
      pl[nb][0] = movmatrix_trans(l0);
      pl[nb][1] = movmatrix_trans(l1);
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
#pragma unroll
    for (int mb = 0; mb < 8; ++mb) {
      uint32_t a[4];
      ldmatrix_x4_trans(st + v_off + mb * 32, a);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        mma_bf16(o[nb][mb], a, pb[nb][0], pb[nb][1]);
        mma_bf16(o[nb][mb], a, pl[nb][0], pl[nb][1]);
      }
    }
  }

  // lane-local row sums -> per-head sums (lanes with equal lane%4 hold the same heads)
  __device__ __forceinline__ void finish_sums() {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        lrun[nb][0] += __shfl_xor_sync(0xffffffffu, lrun[nb][0], off);
        lrun[nb][1] += __shfl_xor_sync(0xffffffffu, lrun[nb][1], off);
      }
  }

  // Spill the state as rows of (128 x O, m, l) per q head: dst[head * ROW + ...].
  // Rows of padding heads (>= g) are skipped.
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

// two e4m3 bytes (low 16 bits of w) -> f16x2, exact
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t w) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(static_cast<unsigned short>(w)));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ float f16_lo(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w))); }
__device__ __forceinline__ float f16_hi(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16))); }

// Per-lane ldmatrix offsets inside a stage for a warp whose row inside each
// group starts at row_off bytes.
__device__ __forceinline__ uint32_t k_lane_offset(int lane, uint32_t row_off) {
  const int li = lane >> 3, lr = lane & 7;
  return (lr + ((li & 1) ? 8 : 0)) * kPitch + row_off + ((li >> 1) ? 16 : 0);
}
__device__ __forceinline__ uint32_t v_lane_offset(int lane, uint32_t row_off) {
  const int li = lane >> 3, lr = lane & 7;
  return kTileB + (lr + ((li >> 1) ? 8 : 0)) * kPitch + row_off + ((li & 1) ? 16 : 0);
}

}  // namespace vt
