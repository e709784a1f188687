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
// warp streams 32-token K/V tiles of the head's kv head into a shared-memory ring,
// either with TMA tensor copies through per-slot tensor maps (four requests per
// tile, 128-byte swizzle: conflict-free ldmatrix without padding) or, without maps,
// with one 1-D bulk copy per 256-byte row at a 272-byte pitch.  The row-copy form
// is limited by the copy-request rate (measured: the consumers wait for data a third
// of the time at 174 TFLOP/s), which is what the tensor copies remove.
// Math per tile and warp, FlashAttention-2 style:
//   S[16 q x BN tok] = Q . K^T     (mma.sync.m16n8k16 bf16, K^T via ldmatrix)
//   causal mask only on tiles that reach past the warp's first row; tiles wholly
//   beyond the warp's last row are skipped; online softmax in fp32 (log2 domain),
//   row max / sum reduced over the 4 lanes of a row with shuffles; the running
//   output is rescaled only when some row's maximum moved
//   O[16 q x 128]  += P . V        (P built 16 tokens at a time from the S
//                                    accumulators as hi + lo bf16, V via ldmatrix.trans)
// Roofline: tensor pipe (4 * q_len * L * 128 flops per head, half of that under
// the causal mask); the math runs on the legacy mma.sync path (ncu: tensor pipe
// 45 % busy at 174 TFLOP/s, so that path tops out near 390 TFLOP/s).
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_mma.cuh"

#include <cuda.h>

#include <cstdlib>

namespace vt {
namespace {

constexpr int kPfPitch = 272;

// TMA = false: K/V rows arrive by one 256-byte bulk copy each at a 272-byte pitch.
// TMA = true : a tile arrives by four tiled tensor copies (K and V, low and high 64 dims)
//              through per-slot tensor maps; each lands as [BN rows][128 bytes] in the
//              128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)),
//              which ldmatrix reads without bank conflicts and without padding.
template <int WARPS, int BN_, int STAGES, bool TMA_ = false>
struct PfCfg {
  static constexpr bool kTma = TMA_;
  static constexpr int kWarps = WARPS;             // consumer warps
  static constexpr int kBM = WARPS * 16;           // query rows per CTA
  static constexpr int kBN = BN_;                  // tokens per K/V tile
  static constexpr int kStages = STAGES;
  static constexpr int kThreads = (WARPS + 1) * 32;
  static constexpr int kHalf = BN_ * 128;          // TMA: one 64-dim half of a K (or V) tile
  static constexpr int kTile = TMA_ ? 2 * kHalf : BN_ * kPfPitch;     // one K (or V) tile
  static constexpr int kStage = 2 * kTile;
  static constexpr int kQBytes = kBM * kPfPitch;
  static constexpr int kRingPad = TMA_ ? 1024 : 0; // the swizzle pattern wants 1024-byte aligned tiles
  static constexpr int kSmem = kQBytes + kRingPad + STAGES * kStage + 2 * STAGES * 8;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

template <class C>
__global__ void __maxnreg__(128) prefill_attn_kernel(PrefillParams p) {
  constexpr int kBM = C::kBM, kBN = C::kBN, kStages = C::kStages, kWarps = C::kWarps;
  constexpr int kTile = C::kTile, kStage = C::kStage;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t q0 = smem_u32(smem);
  const uint32_t ring0 = C::kTma ? ((q0 + C::kQBytes + 1023u) & ~1023u) : q0 + C::kQBytes;
  unsigned char *ring = smem + (ring0 - q0);
  uint64_t *bars = reinterpret_cast<uint64_t *>(ring + kStages * kStage);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);

  // later query tiles see more context: they are scheduled first so that the short ones fill the tail
  const int qt = gridDim.x - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
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
      if constexpr (C::kTma) {
        // Whole boxes even on the ragged last tile: its rows past the context lie in the same
        // mapped 2 MiB chunk (the host only takes this path when tiles never straddle chunks).
        if (lane == 0) {
          const char *maps = static_cast<const char *>(p.maps) + static_cast<size_t>(slot) * 256;
          const uint32_t dst = ring0 + s * kStage, bar = full0 + 8 * s;
          mbar_arrive_expect_tx(bar, 2u * kBN * 256);
          tma_load_3d(dst, maps, 0, kv_head, t0, bar);
          tma_load_3d(dst + C::kHalf, maps, 64, kv_head, t0, bar);
          tma_load_3d(dst + kTile, maps + 128, 0, kv_head, t0, bar);
          tma_load_3d(dst + kTile + C::kHalf, maps + 128, 64, kv_head, t0, bar);
        }
        __syncwarp();
      } else {
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
  // V as B operand (trans): matrices (tok 0-7, d 0-7), (tok 8-15, d 0-7), (tok 0-7, d 8-15), (tok 8-15, d 8-15)
  // Swizzled tiles: row pitch 128; 16-byte chunk (2m + bit) of a row with (row & 7) == lr sits at
  // chunk (2m) ^ (bit ^ lr), so a lane's offset is its base XOR (m << 5), m = (16-dim step) & 3.
  const uint32_t k_off = C::kTma ? (lr + ((li >> 1) ? 8 : 0)) * 128 + ((((li & 1) ^ lr) & 7) << 4)
                                 : (lr + ((li >> 1) ? 8 : 0)) * kPfPitch + ((li & 1) ? 16 : 0);
  const uint32_t v_off = C::kTma ? kTile + (lr + ((li & 1) ? 8 : 0)) * 128 + ((((li >> 1) ^ lr) & 7) << 4)
                                 : kTile + (lr + ((li & 1) ? 8 : 0)) * kPfPitch + ((li >> 1) ? 16 : 0);
  constexpr int kRowPitch = C::kTma ? 128 : kPfPitch;

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
      if constexpr (C::kTma) {
        for (int r = nt + (lane >> 4); r < kBN; r += 2)     // 8 chunks in each 64-dim half, in any order
          *reinterpret_cast<uint4 *>(ring + s * kStage + kTile + (lane & 8 ? C::kHalf : 0) + r * 128 + (lane & 7) * 16) =
              make_uint4(0, 0, 0, 0);
      } else {
        for (int r = nt + (lane >> 4); r < kBN; r += 2)
          *reinterpret_cast<uint4 *>(ring + s * kStage + kTile + r * kPfPitch + (lane & 15) * 16) = make_uint4(0, 0, 0, 0);
      }
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
        if constexpr (C::kTma)
          ldmatrix_x4(st + (ks >> 2) * C::kHalf + np * 16 * kRowPitch + (k_off ^ ((ks & 3) << 5)), kb);
        else
          ldmatrix_x4(st + k_off + np * 16 * kRowPitch + ks * 32, kb);
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
        if constexpr (C::kTma)
          ldmatrix_x4_trans(st + (dp >> 2) * C::kHalf + kk * 16 * kRowPitch + (v_off ^ ((dp & 3) << 5)), vb);
        else
          ldmatrix_x4_trans(st + v_off + kk * 16 * kRowPitch + dp * 32, vb);
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
  if (p.maps) {
    // The tcgen05 kernel (vt_prefill_umma.cu) is the default with tensor maps; VT_PREFILL_ENGINE=mma
    // keeps the mma.sync kernel.  The tcgen05 kernel fetches 64-token tiles (no straddling of a
    // 2 MiB chunk: kvh <= 128) and stores whole 16-byte vectors of the output rows.
    static const bool legacy = [] {
      const char *e = getenv("VT_PREFILL_ENGINE");
      return e && e[0] == 'm';
    }();
    const bool umma_ok = p.kvh * 64 <= 8192 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && p.out_stride % 8 == 0 &&
                         p.scale > 0.f;
    if (!legacy && umma_ok) return launch_prefill_umma(p, max_q_len, stream);
    // mma.sync with tensor copies: 64-row query tiles, three CTAs per SM (250 TFLOP/s causal at 4k prompts, 213 at 1k).
    return launch_cfg<PfCfg<4, 32, 3, true>>(p, max_q_len, stream);
  }
  // Row copies run into the copy-request rate (one request per 256-byte row): long prompts take
  // 112-row tiles, which need 1.75 times fewer K/V requests per flop (204 vs 174 TFLOP/s at 4k);
  // short ones lose more to ragged tiles than they gain.  VT_PREFILL_ROWS=64|112 forces a shape.
  static const int forced = [] {
    const char *e = getenv("VT_PREFILL_ROWS");
    return e ? atoi(e) : 0;
  }();
  if (forced == 112 || (forced != 64 && max_q_len > 1536)) return launch_cfg<PfCfg<7, 32, 3>>(p, max_q_len, stream);
  return launch_cfg<PfCfg<4, 32, 3>>(p, max_q_len, stream);
}

int encode_prefill_maps(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, uint64_t max_tokens,
                        void *host_maps) {
  using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode) return VT_ERR_NO_DRIVER;
  // element (x, head, token) of a range: x fastest, heads 256 bytes apart, tokens kvh * 256 bytes apart
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(kvh), max_tokens};
  const cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(kvh) * 256};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kPrefillBoxTokens)};   // 128 bytes x 32 tokens of one head
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  CUtensorMap *out = static_cast<CUtensorMap *>(host_maps);
  for (int s = 0; s < n_slots; ++s)
    for (int kv = 0; kv < 2; ++kv) {
      const uint64_t base = kv ? v_bases[s] : k_bases[s];
      if (base == 0 || (base & 15) != 0) return VT_ERR_INVALID;
      if (encode(&out[2 * s + kv], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, reinterpret_cast<void *>(base), dims, strides, box,
                 elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return VT_ERR_DRIVER;
    }
  return VT_OK;
}

}  // namespace vt
