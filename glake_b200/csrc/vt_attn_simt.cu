// Single-query decode attention over contiguous per-sequence KV ranges, SIMT
// variant: one CTA per (kv head [x q-head pair], token partition, sequence).
//
// Data movement: a producer warp streams the partition's K and V rows of this
// kv head into a 4-stage shared-memory ring with 1-D bulk async copies
// (cp.async.bulk, one 256-byte (bf16) / 128-byte (fp8) row per copy, completion
// counted on an mbarrier).  No block table: row t of the head lives at
// base + (t * kvh + head) * 128 * e, so the copy addresses are pure arithmetic.
// Compute: four consumer warps; a group of 4 lanes owns one token of the tile,
// each lane holding 32 of the 128 dims of q (pre-scaled, fp32) and of the output
// accumulator.  q.k is reduced over the 4 lanes with two warp shuffles; every
// lane group keeps its own online-softmax state (running max / sum), so there
// is no cross-warp traffic inside the token loop.  The 32 groups are merged once
// per CTA through shared memory.  With more than one partition per sequence the
// CTA writes an unnormalised partial (max, sum, acc[128]) that the reduce kernel
// merges.
//
// Roofline: HBM.  Algorithmic bytes per (sequence, kv head): L * 2 * 128 * e.
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"

namespace vt {
namespace {

constexpr int kTile = 32;     // tokens per stage
constexpr int kStages = 4;
constexpr int kCWarps = 4;    // consumer warps; 8 tokens of a tile each
constexpr int kThreads = (kCWarps + 1) * 32;
constexpr int kGroups = kCWarps * 8;

template <bool FP8>
__host__ __device__ constexpr int row_bytes() { return kHeadDim * (FP8 ? 1 : 2); }
template <bool FP8>
__host__ __device__ constexpr int stage_bytes() { return 2 * kTile * row_bytes<FP8>(); }  // K tile then V tile

template <int G, bool FP8>
constexpr int smem_bytes() {
  // ring, then the barriers; the merge buffers alias the ring after the token loop
  constexpr int ring = kStages * stage_bytes<FP8>();
  constexpr int merge = kGroups * G * (kHeadDim + 2) * 4;
  return (ring > merge ? ring : merge) + 2 * kStages * 8;
}

template <int G, bool FP8>
__global__ void __launch_bounds__(kThreads) attn_simt_kernel(AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int ROWB = row_bytes<FP8>();
  constexpr int STAGEB = stage_bytes<FP8>();
  constexpr int EPC = Unpack<FP8>::N;      // elements per 16-byte chunk
  constexpr int CPT = 32 / EPC;            // chunks per thread per row
  constexpr int RING = kStages * STAGEB;
  constexpr int MERGE = kGroups * G * (kHeadDim + 2) * 4;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (RING > MERGE ? RING : MERGE));
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t ring0 = smem_u32(smem);

  // A query group wider than G is covered by several CTAs per kv head, each
  // re-streaming the head's rows for its own G query heads.
  const int g_total = p.h / p.kvh, subs = g_total / G;
  const int kv_head = blockIdx.x / subs, sub = blockIdx.x % subs;
  const int part = blockIdx.y, b = blockIdx.z;
  const int seq_len = p.seq_lens[b];
  const int t_begin = part * p.part_tokens;
  if (t_begin >= seq_len && !(part == 0 && seq_len <= 0)) return;
  const int t_end = min(seq_len, t_begin + p.part_tokens);
  const int n_tok = max(t_end - t_begin, 0);
  const int n_tiles = (n_tok + kTile - 1) / kTile;
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
    const int64_t slot = p.slot_ids[b];
    const size_t tok_pitch = static_cast<size_t>(p.kvh) * ROWB;
    const char *kbase = reinterpret_cast<const char *>(p.k_table[slot]) + static_cast<size_t>(kv_head) * ROWB;
    const char *vbase = reinterpret_cast<const char *>(p.v_table[slot]) + static_cast<size_t>(kv_head) * ROWB;
    const uint64_t policy = l2_policy_evict_first();
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int s = tile % kStages;
      if (tile >= kStages && !mbar_wait(empty0 + 8 * s, ((tile / kStages) - 1) & 1)) {
        if (lane == 0) atomicExch(p.status, kKernelErrMagic);
        break;
      }
      const int t0 = t_begin + tile * kTile;
      const int nt = min(kTile, t_end - t0);
      if (lane == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2u * nt * ROWB);
      __syncwarp();
      if (lane < nt) {
        const size_t goff = static_cast<size_t>(t0 + lane) * tok_pitch;
        const uint32_t dst = ring0 + s * STAGEB + lane * ROWB;
        bulk_g2s_hint(dst, kbase + goff, ROWB, full0 + 8 * s, policy);
        bulk_g2s_hint(dst + kTile * ROWB, vbase + goff, ROWB, full0 + 8 * s, policy);
      }
    }
    return;
  }

  // ---------------- consumer warps ----------------
  const int tg = lane >> 2, j = lane & 3, par = tg & 1;
  // Chunk order: lane group parity swaps neighbouring 64-byte halves so that the
  // two tokens served by one quarter-warp hit disjoint shared-memory banks.
  int chunk[CPT];
#pragma unroll
  for (int i = 0; i < CPT; ++i) chunk[i] = ((i ^ par) << 2) + j;

  float qf[G][32], acc[G][32], m[G], l[G];
  {
    const __nv_bfloat16 *qrow = static_cast<const __nv_bfloat16 *>(p.q) + b * p.q_stride + (kv_head * g_total + sub * G) * kHeadDim;
    const float qs = p.scale * 1.4426950408889634f * (FP8 ? p.k_scale[kv_head] : 1.0f);
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
#pragma unroll
        for (int e = 0; e < EPC; e += 8) {
          uint4 v = __ldg(reinterpret_cast<const uint4 *>(qrow + g * kHeadDim + chunk[i] * EPC + e));
          float f[8];
          Unpack<false>::run(v, f);
#pragma unroll
          for (int x = 0; x < 8; ++x) qf[g][i * EPC + e + x] = f[x] * qs;
        }
      }
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int x = 0; x < 32; ++x) acc[g][x] = 0.f;
    }
  }

  bool failed = false;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kStages;
    if (!mbar_wait(full0 + 8 * s, (tile / kStages) & 1)) { failed = true; break; }
    const int tok = warp * 8 + tg;
    const bool valid = tile * kTile + tok < n_tok;
    const unsigned char *krow = smem + s * STAGEB + tok * ROWB;
    const unsigned char *vrow = krow + kTile * ROWB;

    float sc[G];
    {
      float part0[G], part1[G];
#pragma unroll
      for (int g = 0; g < G; ++g) part0[g] = part1[g] = 0.f;
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        float kf[EPC];
        Unpack<FP8>::run(*reinterpret_cast<const uint4 *>(krow + chunk[i] * 16), kf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int x = 0; x < EPC; x += 2) {
            part0[g] = fmaf(qf[g][i * EPC + x], kf[x], part0[g]);
            part1[g] = fmaf(qf[g][i * EPC + x + 1], kf[x + 1], part1[g]);
          }
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float v = part0[g] + part1[g];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        sc[g] = v;
      }
    }
    if (valid) {
      float pr[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (sc[g] > m[g]) {
          const float f = exp2f(m[g] - sc[g]);
          l[g] *= f;
#pragma unroll
          for (int x = 0; x < 32; ++x) acc[g][x] *= f;
          m[g] = sc[g];
        }
        pr[g] = exp2f(sc[g] - m[g]);
        l[g] += pr[g];
      }
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        float vf[EPC];
        Unpack<FP8>::run(*reinterpret_cast<const uint4 *>(vrow + chunk[i] * 16), vf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int x = 0; x < EPC; ++x) acc[g][i * EPC + x] = fmaf(pr[g], vf[x], acc[g][i * EPC + x]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
  }

  // ---------------- merge the 32 lane groups ----------------
  named_bar_sync(1, kCWarps * 32);  // every consumer is done reading the ring
  float *macc = reinterpret_cast<float *>(smem);               // [kGroups][G][128]
  float *mml = macc + kGroups * G * kHeadDim;                  // [kGroups][G][2]
  const int grp = warp * 8 + tg;
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
#pragma unroll
      for (int x = 0; x < EPC; x += 4) {
        *reinterpret_cast<float4 *>(macc + (grp * G + g) * kHeadDim + chunk[i] * EPC + x) =
            make_float4(acc[g][i * EPC + x], acc[g][i * EPC + x + 1], acc[g][i * EPC + x + 2], acc[g][i * EPC + x + 3]);
      }
    }
    if (j == 0) {
      mml[(grp * G + g) * 2] = m[g];
      mml[(grp * G + g) * 2 + 1] = l[g];
    }
  }
  named_bar_sync(1, kCWarps * 32);
  if (failed && threadIdx.x == 0) atomicExch(p.status, kKernelErrMagic);

  const int d = threadIdx.x;  // 0..127
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int r = 0; r < kGroups; ++r) M = fmaxf(M, mml[(r * G + g) * 2]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
      for (int r = 0; r < kGroups; ++r) {
        const float f = exp2f(mml[(r * G + g) * 2] - M);
        L = fmaf(f, mml[(r * G + g) * 2 + 1], L);
        O = fmaf(f, macc[(r * G + g) * kHeadDim + d], O);
      }
    }
    const int hq = kv_head * g_total + sub * G + g;
    if (n_parts == 1) {
      const float vs = FP8 ? p.v_scale[kv_head] : 1.0f;
      const float o = L > 0.f ? O / L * vs : 0.f;
      static_cast<__nv_bfloat16 *>(p.out)[b * p.out_stride + hq * kHeadDim + d] = __float2bfloat16(o);
      if (p.lse && d == 0)
        p.lse[b * p.h + hq] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
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

template <int G, bool FP8>
int launch(const AttnParams &p, cudaStream_t stream) {
  constexpr int SMEM = smem_bytes<G, FP8>();
  static SmemOptIn opt_in;
  if (!opt_in.ensure(attn_simt_kernel<G, FP8>, SMEM)) return VT_ERR_CUDA;
  dim3 grid(p.kvh * ((p.h / p.kvh) / G), p.max_parts, p.batch);
  attn_simt_kernel<G, FP8><<<grid, kThreads, SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

}  // namespace

int launch_attn_simt(const AttnParams &p, int kv_dtype, cudaStream_t stream) {
  const int g = p.h / p.kvh;
  const bool fp8 = kv_dtype == VT_KV_FP8_E4M3;
  if (g == 1) return fp8 ? launch<1, true>(p, stream) : launch<1, false>(p, stream);
  return fp8 ? launch<2, true>(p, stream) : launch<2, false>(p, stream);
}

}  // namespace vt
