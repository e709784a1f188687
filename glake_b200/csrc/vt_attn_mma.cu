// Single-query decode attention over contiguous per-sequence KV ranges,
// tensor-core variant.  One CTA per (slab of kv heads, token partition, sequence);
// a warp serves ALL q heads of one kv head, so every K/V byte leaves HBM once.
//
// Data movement: a producer warp streams the partition's K and V rows into a
// 3-stage shared-memory ring with 1-D bulk async copies (cp.async.bulk, mbarrier
// completion).  Measured on B200, the copy engine sustains ~7.3 TB/s with
// requests of >= 1 KiB but only ~3.3 TB/s with 256-byte ones, so every request
// moves 1 KiB: a "group" of R consecutive tokens x HS kv heads x 256 B with
// R * HS = 4.  HS = 4, R = 1 when the rank holds >= 4 kv heads (a token row of a
// 4-head slab), HS = 2, R = 2 for two kv heads, HS = 1, R = 4 for one (then the
// R token rows are adjacent in memory, which only a contiguous range allows).
// A tile is 16 groups; groups sit at a 1040-byte pitch in shared memory.
//
// Math ("tokens as M"): consumer warp w owns kv head w % HS and row w / HS of
// every group, i.e. 16 tokens of the tile, one per group.  Because the 16 rows of
// a fragment come from 16 different groups, ldmatrix reads addresses 1040 B
// apart and never conflicts on banks, without padding inside a copy.
//   S^T[16 tok x 8 heads]  = K[16 x 128] . Q^T[128 x 8]        (8 x mma.m16n8k16)
//   online softmax over tokens, per head, in fp32 (log2 domain), max and sum
//   reduced across the warp with shuffles
//   O^T[128 d x 8 heads]  += V^T[128 x 16 tok] . P^T[16 x 8]   (2 x 8 x mma.m16n8k16: P as hi + lo bf16)
// K fragments come from ldmatrix, V^T fragments from ldmatrix.trans, and the
// probabilities move from the accumulator layout of S^T into the B-operand
// layout of P^T with movmatrix (an 8x8 transpose across the warp).  With 8 q
// heads per kv head no tensor-core work is wasted; groups of 1/2/4 pad N to 8 and
// a group of 16 uses two n-blocks.  The per-warp contraction is 16 x 8 x 128: far
// too small for a tcgen05/TMEM pipeline (M >= 64 per instruction) to pay, and the
// kernel is bound by HBM, not by the tensor pipe.
//
// Roofline: HBM.  Algorithmic bytes per (sequence, kv head): L * 2 * 128 * 2.
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_mma.cuh"

namespace vt {
namespace {

constexpr int kStages = kMmaStages;
constexpr int kCWarps = kMmaCWarps;
constexpr int kThreads = kMmaThreads;

template <int NB>
__host__ __device__ constexpr int smem_bytes() {
  constexpr int ring = kStages * kStageB;
  constexpr int merge = kCWarps * NB * 8 * 130 * 4;
  return (ring > merge ? ring : merge) + 2 * kStages * 8;
}

// NB = number of 8-head blocks: 1 serves groups of 1..8 q heads, 2 a group of 16.
// HS = kv heads per CTA, R = consecutive tokens per bulk copy; HS * R == 4.
template <int NB, int HS, int R>
__global__ void __launch_bounds__(kThreads) attn_mma_kernel(AttnParams p) {
  static_assert(HS * R == kCWarps, "one consumer warp per (kv head, row of a group)");
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int RING = kStages * kStageB;
  constexpr int MERGE = kCWarps * NB * 8 * 130 * 4;
  constexpr int TILE_TOK = kGroupsPerTile * R;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (RING > MERGE ? RING : MERGE));
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t ring0 = smem_u32(smem);

  const int g = p.h / p.kvh;
  const int slab = blockIdx.x, part = blockIdx.y, b = blockIdx.z;
  const int seq_len = p.seq_lens[b];
  const int t_begin = part * p.part_tokens;
  if (t_begin >= seq_len && !(part == 0 && seq_len <= 0)) return;
  const int t_end = min(seq_len, t_begin + p.part_tokens);
  const int n_tok = max(t_end - t_begin, 0);
  const int n_tiles = (n_tok + TILE_TOK - 1) / TILE_TOK;
  const int n_parts = seq_len > 0 ? (seq_len + p.part_tokens - 1) / p.part_tokens : 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kCWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kCWarps) {
    // ---------------- producer warp ----------------
    // lanes 0..15 fetch the K groups of a tile, lanes 16..31 the V groups
    const int64_t slot = p.slot_ids[b];
    const size_t tok_pitch = static_cast<size_t>(p.kvh) * kRowB;
    const char *base = reinterpret_cast<const char *>(lane < 16 ? p.k_table[slot] : p.v_table[slot]) +
                       static_cast<size_t>(slab) * HS * kRowB;
    const int grp = lane & 15;
    const uint32_t dst_lane = (lane < 16 ? 0 : kTileB) + grp * kPitch;
    const uint64_t policy = l2_policy_evict_first();
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int s = tile % kStages;
      if (tile >= kStages && !mbar_wait(empty0 + 8 * s, ((tile / kStages) - 1) & 1)) {
        if (lane == 0) atomicExch(p.status, kKernelErrMagic);
        break;
      }
      const int t0 = t_begin + tile * TILE_TOK;
      const int nt = min(TILE_TOK, t_end - t0);
      if (lane == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2u * nt * HS * kRowB);
      __syncwarp();
      const int rows = min(R, nt - grp * R);   // valid token rows of this lane's group
      if (rows > 0)
        bulk_g2s_hint(ring0 + s * kStageB + dst_lane, base + static_cast<size_t>(t0 + grp * R) * tok_pitch,
                      rows * HS * kRowB, full0 + 8 * s, policy);
    }
    return;
  }

  // ---------------- consumer warps ----------------
  const int hs = warp % HS, rr = warp / HS;      // kv head within the slab, row within each group
  const int kv_head = slab * HS + hs;
  const uint32_t row_off = (rr * HS + hs) * kRowB;
  WarpAttn<NB> st;
  st.start(static_cast<const __nv_bfloat16 *>(p.q) + b * p.q_stride + kv_head * g * kHeadDim, g, lane);
  const float sl2 = p.scale * 1.4426950408889634f;
  const uint32_t k_off = k_lane_offset(lane, row_off), v_off = v_lane_offset(lane, row_off);

  bool failed = false;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kStages;
    if (!mbar_wait(full0 + 8 * s, (tile / kStages) & 1)) { failed = true; break; }
    const int tok0 = tile * TILE_TOK + rr;      // token of fragment row 0, partition-relative
    if (tok0 < n_tok)
      st.tile(ring0 + s * kStageB, smem + s * kStageB, k_off, v_off, row_off,
              min(16, (n_tok - tok0 + R - 1) / R), sl2, lane);
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
  }

  // ---------------- merge the R warps of each kv head, write out ----------------
  st.finish_sums();
  named_bar_sync(1, kCWarps * 32);   // every consumer is done reading the ring
  constexpr int HEADS = NB * 8;
  float *mbuf = reinterpret_cast<float *>(smem);   // [kCWarps][HEADS][130]
  st.template store<130>(mbuf + warp * HEADS * 130, lane, g);
  named_bar_sync(1, kCWarps * 32);
  if (failed && threadIdx.x == 0) atomicExch(p.status, kKernelErrMagic);

  const int d = threadIdx.x;  // 0..127
  for (int hh = 0; hh < HS; ++hh) {
    for (int head = 0; head < g; ++head) {
      float M = -INFINITY;
#pragma unroll
      for (int r = 0; r < R; ++r) M = fmaxf(M, mbuf[((r * HS + hh) * HEADS + head) * 130 + 128]);
      float L = 0.f, O = 0.f;
      if (M > -INFINITY) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float *src = mbuf + ((r * HS + hh) * HEADS + head) * 130;
          const float f = exp2f(src[128] - M);
          L = fmaf(f, src[129], L);
          O = fmaf(f, src[d], O);
        }
      }
      const int hq = (slab * HS + hh) * g + head;
      if (n_parts == 1) {
        static_cast<__nv_bfloat16 *>(p.out)[b * p.out_stride + hq * kHeadDim + d] =
            __float2bfloat16(L > 0.f ? O / L : 0.f);
        if (p.lse && d == 0) p.lse[b * p.h + hq] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
      } else {
        const size_t idx = (static_cast<size_t>(b) * p.h + hq) * p.max_parts + part;
        p.ws_o[idx * kHeadDim + d] = O;
        if (d == 0) {
          p.ws_ml[idx * 2] = M;
          p.ws_ml[idx * 2 + 1] = L;
        }
      }
    }
  }
}

template <int NB, int HS, int R>
int launch(const AttnParams &p, cudaStream_t stream) {
  constexpr int SMEM = smem_bytes<NB>();
  static SmemOptIn opt_in;
  if (!opt_in.ensure(attn_mma_kernel<NB, HS, R>, SMEM)) return VT_ERR_CUDA;
  dim3 grid(p.kvh / HS, p.max_parts, p.batch);
  attn_mma_kernel<NB, HS, R><<<grid, kThreads, SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

template <int NB>
int launch_nb(const AttnParams &p, cudaStream_t stream) {
  if (p.kvh % 4 == 0) return launch<NB, 4, 1>(p, stream);
  if (p.kvh == 2) return launch<NB, 2, 2>(p, stream);
  if (p.kvh == 1) return launch<NB, 1, 4>(p, stream);
  return VT_ERR_UNSUPPORTED;
}

}  // namespace

bool attn_mma_supports(int h, int kvh, int kv_dtype) {
  const int g = h / kvh;
  return kv_dtype == VT_KV_BF16 && (kvh % 4 == 0 || kvh == 2 || kvh == 1) && (g <= 8 || g == 16);
}

int launch_attn_mma(const AttnParams &p, int kv_dtype, cudaStream_t stream) {
  if (!attn_mma_supports(p.h, p.kvh, kv_dtype)) return VT_ERR_UNSUPPORTED;
  return (p.h / p.kvh) <= 8 ? launch_nb<1>(p, stream) : launch_nb<2>(p, stream);
}

}  // namespace vt
