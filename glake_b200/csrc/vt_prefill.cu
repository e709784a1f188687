// Causal attention of the NEW tokens of a sequence over its whole contiguous
// KV range (prefix + the new tokens, already appended): the prefill /
// prefix-extend side of the vTensor path.  The reference reaches this through
// flash_attn_2_cuda.fwd_kvcache with seqlen_q > 1
// (GLakeServe/vllm/attention/backends/xformers.py:362-385).
//
// One CTA per (query tile, q head, sequence).  Query row j of a sequence with
// context L and q_len new tokens sits at position L - q_len + j and attends
// tokens [0, position].  Each consumer warp owns 16 query rows; the tile's Q rows
// sit in shared memory (A fragments re-read per tile with ldmatrix, which keeps the
// kernel at <= 128 registers so that four warps fit per scheduler).  A producer
// warp streams K/V tiles of the head's kv head into a shared-memory ring with 1-D
// bulk async copies (one 256-byte row per copy at a 272-byte pitch, which keeps
// ldmatrix conflict free; the request-rate limit of small copies does not matter
// here, the kernel is bound by issue slots and the tensor pipe, not by HBM).
// Math per tile and warp, FlashAttention-2 style:
//   S[16 q x BN tok] = Q . K^T     (mma.sync.m16n8k16 bf16, K^T via ldmatrix)
//   causal mask only on tiles that reach past the warp's first row; tiles wholly
//   beyond the warp's last row are skipped; online softmax in fp32 (log2 domain),
//   row max / sum reduced over the 4 lanes of a row with shuffles; the running
//   output is rescaled only when some row's maximum moved
//   O[16 q x 128]  += P . V        (P built 16 tokens at a time from the S
//                                    accumulators as hi + lo bf16, V via ldmatrix.trans)
// Roofline: tensor pipe (4 * q_len * L * 128 flops per head, half of that under
// the causal mask); this kernel uses the legacy mma.sync path.
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_mma.cuh"

#include <cstdlib>

namespace vt {
namespace {

constexpr int kPfPitch = 272;

template <int WARPS, int BN_, int STAGES>
struct PfCfg {
  static constexpr int kWarps = WARPS;             // consumer warps
  static constexpr int kBM = WARPS * 16;           // query rows per CTA
  static constexpr int kBN = BN_;                  // tokens per K/V tile
  static constexpr int kStages = STAGES;
  static constexpr int kThreads = (WARPS + 1) * 32;
  static constexpr int kTile = BN_ * kPfPitch;     // one K (or V) tile
  static constexpr int kStage = 2 * kTile;
  static constexpr int kQBytes = kBM * kPfPitch;
  static constexpr int kSmem = kQBytes + STAGES * kStage + 2 * STAGES * 8;
};

template <class C>
__global__ void __maxnreg__(128) prefill_attn_kernel(PrefillParams p) {
  constexpr int kBM = C::kBM, kBN = C::kBN, kStages = C::kStages, kWarps = C::kWarps;
  constexpr int kTile = C::kTile, kStage = C::kStage;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kQBytes + kStages * kStage);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t q0 = smem_u32(smem), ring0 = q0 + C::kQBytes;

  const int qt = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int q_len = p.q_lens[b], seq_len = p.seq_lens[b];
  const int j0 = qt * kBM;
  if (j0 >= q_len) return;
  const int g = p.h / p.kvh, kv_head = hq / g;
  const int pos0 = seq_len - q_len + j0;                    // position of the tile's first query row
  const int kv_end = min(seq_len, pos0 + kBM);              // keys any row of the tile may see
  const int n_tiles = (kv_end + kBN - 1) / kBN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kWarps) {
    // ---------------- producer warp ----------------
    const int64_t slot = p.slot_ids[b];
    const size_t tok_pitch = static_cast<size_t>(p.kvh) * 256;
    const char *kbase = reinterpret_cast<const char *>(p.k_table[slot]) + static_cast<size_t>(kv_head) * 256;
    const char *vbase = reinterpret_cast<const char *>(p.v_table[slot]) + static_cast<size_t>(kv_head) * 256;
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int s = tile % kStages;
      if (tile >= kStages && !mbar_wait(empty0 + 8 * s, ((tile / kStages) - 1) & 1)) {
        if (lane == 0 && p.status) atomicExch(p.status, kKernelErrMagic);
        return;
      }
      const int t0 = tile * kBN;
      const int nt = min(kBN, kv_end - t0);
      if (lane == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2u * nt * 256);
      __syncwarp();
      for (int r = lane; r < nt; r += 32) {
        const size_t goff = static_cast<size_t>(t0 + r) * tok_pitch;
        const uint32_t dst = ring0 + s * kStage + r * kPfPitch;
        bulk_g2s(dst, kbase + goff, 256, full0 + 8 * s);
        bulk_g2s(dst + kTile, vbase + goff, 256, full0 + 8 * s);
      }
    }
    return;
  }

  // ---------------- consumer warps ----------------
  const int r4 = lane >> 2, c4 = lane & 3;
  const int row_a = j0 + warp * 16 + r4, row_b = row_a + 8;          // this lane's two query rows (entry-relative)
  const bool ok_a = row_a < q_len, ok_b = row_b < q_len;
  // The warp's 16 Q rows -> shared memory (zeros beyond q_len); only this warp reads them back.
  {
    const __nv_bfloat16 *qbase = static_cast<const __nv_bfloat16 *>(p.q) + static_cast<int64_t>(p.q_start[b]) * p.q_stride +
                                 hq * kHeadDim;
    unsigned char *qs = smem + warp * 16 * kPfPitch;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = lane + 32 * i, r = idx >> 4, c = idx & 15;
      const int row = j0 + warp * 16 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < q_len) v = __ldg(reinterpret_cast<const uint4 *>(qbase + static_cast<int64_t>(row) * p.q_stride) + c);
      *reinterpret_cast<uint4 *>(qs + r * kPfPitch + c * 16) = v;
    }
    __syncwarp();
  }
  const float sl2 = p.scale * 1.4426950408889634f;
  const int lim_a = seq_len - q_len + row_a, lim_b = lim_a + 8;     // last visible token per row
  const int lim_first = pos0 + warp * 16, lim_last = lim_first + 15;  // of the warp's rows
  float o[16][4];
#pragma unroll
  for (int nb = 0; nb < 16; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  const int li = lane >> 3, lr = lane & 7;
  // Q as A operand (non-trans): matrices (rows 0-7, d lo), (rows 8-15, d lo), (rows 0-7, d hi), (rows 8-15, d hi)
  const uint32_t q_off = q0 + (warp * 16 + lr + ((li & 1) ? 8 : 0)) * kPfPitch + ((li >> 1) ? 16 : 0);
  // K^T as B operand (non-trans): matrices (tok 0-7, d lo), (tok 0-7, d hi), (tok 8-15, d lo), (tok 8-15, d hi)
  const uint32_t k_off = (lr + ((li >> 1) ? 8 : 0)) * kPfPitch + ((li & 1) ? 16 : 0);
  // V as B operand (trans): matrices (tok 0-7, d 0-7), (tok 8-15, d 0-7), (tok 0-7, d 8-15), (tok 8-15, d 8-15)
  const uint32_t v_off = kTile + (lr + ((li & 1) ? 8 : 0)) * kPfPitch + ((li >> 1) ? 16 : 0);

  bool failed = false;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kStages;
    if (!failed && !mbar_wait(full0 + 8 * s, (tile / kStages) & 1)) failed = true;
    if (failed) continue;
    const uint32_t st = ring0 + s * kStage;
    const int t0 = tile * kBN;
    if (t0 > lim_last) {                 // nothing in this tile is visible to any of the warp's rows
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
      continue;
    }
    const int nt = min(kBN, kv_end - t0);
    if (nt < kBN) {
      // Ragged last tile: stale V rows would turn 0 * NaN into NaN.  Every warp clears
      // all of them itself (same zeros from every warp: a benign overlap) so that no
      // cross-warp barrier is needed inside the loop.
      for (int r = nt + (lane >> 4); r < kBN; r += 2)
        *reinterpret_cast<uint4 *>(smem + C::kQBytes + s * kStage + kTile + r * kPfPitch + (lane & 15) * 16) =
            make_uint4(0, 0, 0, 0);
      __syncwarp();
    }
    // ---- S = Q . K^T : BN / 8 n-blocks of 8 tokens ----
    float sacc[kBN / 8][4];
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t qa[4];
      ldmatrix_x4(q_off + ks * 32, qa);
#pragma unroll
      for (int np = 0; np < kBN / 16; ++np) {   // 16 tokens per ldmatrix.x4
        uint32_t kb[4];
        ldmatrix_x4(st + k_off + np * 16 * kPfPitch + ks * 32, kb);
        mma_bf16(sacc[2 * np], qa, kb[0], kb[1]);
        mma_bf16(sacc[2 * np + 1], qa, kb[2], kb[3]);
      }
    }
    // ---- scale, mask, online softmax (row a: regs 0,1; row b: regs 2,3; cols t0 + 8 nb + 2 c4 + {0,1}) ----
    float mx_a = -INFINITY, mx_b = -INFINITY;
    if (t0 + kBN - 1 > lim_first) {      // the tile reaches past the warp's first row: mask per element
#pragma unroll
      for (int nb = 0; nb < kBN / 8; ++nb) {
        const int t = t0 + nb * 8 + 2 * c4;
        sacc[nb][0] = (t <= lim_a) ? sacc[nb][0] * sl2 : -INFINITY;
        sacc[nb][1] = (t + 1 <= lim_a) ? sacc[nb][1] * sl2 : -INFINITY;
        sacc[nb][2] = (t <= lim_b) ? sacc[nb][2] * sl2 : -INFINITY;
        sacc[nb][3] = (t + 1 <= lim_b) ? sacc[nb][3] * sl2 : -INFINITY;
      }
    } else {
#pragma unroll
      for (int nb = 0; nb < kBN / 8; ++nb) {
        sacc[nb][0] *= sl2; sacc[nb][1] *= sl2; sacc[nb][2] *= sl2; sacc[nb][3] *= sl2;
      }
    }
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb) {
      mx_a = fmaxf(mx_a, fmaxf(sacc[nb][0], sacc[nb][1]));
      mx_b = fmaxf(mx_b, fmaxf(sacc[nb][2], sacc[nb][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    // a row with nothing visible yet keeps max = -inf; use 0 as the reference point to avoid inf - inf
    const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;
    if (__any_sync(0xffffffffu, mn_a != m_a || mn_b != m_b)) {     // some row's maximum moved: rescale
      const float fa = exp2f(m_a - ref_a), fb = exp2f(m_b - ref_b);
      l_a *= fa;
      l_b *= fb;
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) {
        o[nb][0] *= fa; o[nb][1] *= fa;
        o[nb][2] *= fb; o[nb][3] *= fb;
      }
    }
    m_a = mn_a;
    m_b = mn_b;
    // ---- O += P . V : k-steps of 16 tokens x 16 n-blocks of 8 dims; P made just before its use ----
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      uint32_t ph[4], pl[4];             // P as A operand: hi and lo bf16 halves
#pragma unroll
      for (int hi8 = 0; hi8 < 2; ++hi8) {
        const int nb = 2 * kk + hi8;
        const float p0 = exp2f(sacc[nb][0] - ref_a), p1 = exp2f(sacc[nb][1] - ref_a);
        const float p2 = exp2f(sacc[nb][2] - ref_b), p3 = exp2f(sacc[nb][3] - ref_b);
        l_a += p0 + p1;
        l_b += p2 + p3;
        const uint32_t ha = pack_bf16(p0, p1), hb = pack_bf16(p2, p3);
        // C layout of n-blocks (2k, 2k+1) is the A layout of k-step k: regs (row a, row b, row a +8 cols, row b +8 cols)
        ph[0 + 2 * hi8] = ha; ph[1 + 2 * hi8] = hb;
        pl[0 + 2 * hi8] = pack_bf16(p0 - bf16_lo(ha), p1 - bf16_hi(ha));
        pl[1 + 2 * hi8] = pack_bf16(p2 - bf16_lo(hb), p3 - bf16_hi(hb));
      }
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {   // 16 dims per ldmatrix.x4.trans
        uint32_t vb[4];
        ldmatrix_x4_trans(st + v_off + kk * 16 * kPfPitch + dp * 32, vb);
        mma_bf16(o[2 * dp], ph, vb[0], vb[1]);
        mma_bf16(o[2 * dp], pl, vb[0], vb[1]);
        mma_bf16(o[2 * dp + 1], ph, vb[2], vb[3]);
        mma_bf16(o[2 * dp + 1], pl, vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
  }
  if (failed) {
    if (lane == 0 && p.status) atomicExch(p.status, kKernelErrMagic);
    return;
  }
  // ---- normalise and write ----
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
  __nv_bfloat16 *obase = static_cast<__nv_bfloat16 *>(p.out) + static_cast<int64_t>(p.q_start[b]) * p.out_stride +
                         hq * kHeadDim;
#pragma unroll
  for (int nb = 0; nb < 16; ++nb) {
    const int d = nb * 8 + 2 * c4;
    if (ok_a)
      *reinterpret_cast<uint32_t *>(obase + static_cast<int64_t>(row_a) * p.out_stride + d) =
          pack_bf16(o[nb][0] * ia, o[nb][1] * ia);
    if (ok_b)
      *reinterpret_cast<uint32_t *>(obase + static_cast<int64_t>(row_b) * p.out_stride + d) =
          pack_bf16(o[nb][2] * ib, o[nb][3] * ib);
  }
}

}  // namespace

template <class C>
int launch_cfg(const PrefillParams &p, int max_q_len, cudaStream_t stream) {
  static SmemOptIn opt_in;
  if (!opt_in.ensure(prefill_attn_kernel<C>, C::kSmem)) return VT_ERR_CUDA;
  dim3 grid((max_q_len + C::kBM - 1) / C::kBM, p.h, p.batch);
  prefill_attn_kernel<C><<<grid, C::kThreads, C::kSmem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

int launch_prefill_attn(const PrefillParams &p, int max_q_len, cudaStream_t stream) {
  // VT_PREFILL_CFG picks another tile shape (a tuning knob, like VT_ATTN_VARIANT for the decode kernels).
  static const int cfg = [] {
    const char *e = getenv("VT_PREFILL_CFG");
    return e ? atoi(e) : 0;
  }();
  if (cfg == 0 && max_q_len > 1536)      // long prompts: 112-row tiles cut the K/V copy requests per flop by 1.75
    return launch_cfg<PfCfg<7, 32, 3>>(p, max_q_len, stream);
  switch (cfg) {
    case 1: return launch_cfg<PfCfg<4, 64, 2>>(p, max_q_len, stream);   // 64 rows, 64-token tiles, 2 stages: 2 CTAs / SM
    case 2: return launch_cfg<PfCfg<6, 64, 2>>(p, max_q_len, stream);   // 96 rows, 64-token tiles, 2 stages: 2 CTAs / SM
    case 3: return launch_cfg<PfCfg<7, 32, 3>>(p, max_q_len, stream);   // 112 rows, 32-token tiles, 3 stages: 2 CTAs / SM
    case 4: return launch_cfg<PfCfg<7, 64, 2>>(p, max_q_len, stream);   // 112 rows, 64-token tiles, 2 stages: 2 CTAs / SM
    case 5: return launch_cfg<PfCfg<6, 32, 3>>(p, max_q_len, stream);   // 96 rows, 32-token tiles, 3 stages: 2 CTAs / SM
    case 6: return launch_cfg<PfCfg<4, 32, 3>>(p, max_q_len, stream);
    default: return launch_cfg<PfCfg<4, 32, 3>>(p, max_q_len, stream);  // 64 rows, 32-token tiles, 3 stages: 3 CTAs / SM
  }
}

}  // namespace vt
