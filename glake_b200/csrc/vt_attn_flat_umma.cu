// Decode attention over an fp8 e4m3 cache on the 5th-generation tensor cores
// (tcgen05.mma.kind::f8f6f4, accumulators in tensor memory): the cache bytes go from
// HBM through shared memory into the tensor core without ever being converted by a
// thread.  Same persistent schedule, scratch format and merge as the mma.sync kernel
// of vt_attn_flat.cu (pieces, tickets, last CTA of a stream merges); the engine differs.
//
// Shapes: kv heads a multiple of 8 (one CTA streams 8 kv heads = 1 KiB token rows),
// 1, 2 or 4 q heads per kv head, head size 128.  Needs the per-slot TMA tensor maps
// of encode_decode_maps_f8: a tile is 32 tokens x 8 kv heads, fetched as sixteen
// 128-byte-swizzled boxes (32 tokens x 128 bytes of one kv head; K, then V).
//
// One CTA per SM, ten warps:
//   warp 8   producer: tensor copies into a 3-stage ring (64 KiB per stage).  The last
//            tile of a stream is patched by this warp before it is handed on: V rows past
//            the context are cleared (0 x NaN would poison the product) and, in a fused
//            step, this step's K / V row is quantised into the stage and into the range.
//   warp 9   one lane issues the MMAs.
//            S^T = K . Q^T : A = K rows of four kv heads (M = 128 = 4 heads x 32 tokens,
//            K-major), B = Q of those heads as TWO e4m3 terms per q head (hi + lo, each
//            head scaled by its own power of two: exact for bf16 inputs), N = 64.
//            Three quarters of that product pair a kv head with another head's Q and
//            are never read: the tensor core has the time, the threads do not.
//            O^T = V^T . P^T per kv head: A = V (MN-major, M = 128 dims, K = 32 tokens),
//            B = P as THREE e4m3 terms per q head (12 significant bits), N = 16, into
//            a fresh accumulator per tile.
//   warps 0-7 consumers.  Softmax: warp j owns kv head j, lane = token (the TMEM lane of
//            its row of S^T): tcgen05.ld of 16 columns, running max over the warp by
//            shuffles, P split into terms and stored as bytes.  Accumulate: the same
//            warps then add the tile's O^T (lane = output dim) into registers with the
//            usual rescale; that step runs one tile behind so that the P.V product of
//            tile i overlaps the softmax of tile i + 1.
// Every wait is bounded; a wait that runs out marks the launch as failed (status
// word) and the CTA still frees its tensor memory.
//
// Roofline: HBM.  Algorithmic bytes per (sequence, kv head): L * 2 * 128.
#include <cuda.h>

#include <algorithm>

#include "../../include/vtensor.h"
#include "vt_attn_flat_sched.cuh"
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_umma.cuh"

namespace vt {
namespace {

constexpr int kUT = 32;                       // tokens per tile
constexpr int kUHS = 8;                       // kv heads per CTA
constexpr int kUCWarps = 8;
constexpr int kUThreads = (kUCWarps + 2) * 32;
constexpr int kUStages = 3;
constexpr int kHeadTileB = kUT * 128;         // one kv head's rows of a tile: [32 tokens][128 B]
constexpr int kKVTileB = kUHS * kHeadTileB;   // K (or V) of a tile
constexpr int kUStageB = 2 * kKVTileB;        // 64 KiB
constexpr int kQSlabB = 64 * 128;             // Q operand of four kv heads: 16 rows each (2 terms x 4 heads + 8 zero rows)
constexpr int kPSlabB = 16 * 128;             // P operand of four kv heads: 16 rows (3 terms x 4 heads + 4 zero rows), 32 bytes of tokens each
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;                 // S^T buffer b, half hf: columns [128 b + 64 hf, + 64)
constexpr uint32_t kColO = 256;               // O^T of kv head j: columns [256 + 16 j, + 16)
constexpr float kPScale = 256.f;              // P is carried as 256 p: e4m3 then resolves 2^-17 of the largest term

// offsets from the 1024-byte aligned base of the dynamic shared memory
constexpr int kOffQ = kUStages * kUStageB;            // 196608
constexpr int kOffP = kOffQ + 2 * kQSlabB;            // 212992: [2 buffers][2 slabs]
constexpr int kOffBars = kOffP + 4 * kPSlabB;         // 221184: 16 mbarriers
constexpr int kOffFac = kOffBars + 16 * 8;            // ring of 4 x [8 kv heads][4 heads] rescale factors
constexpr int kOffLm = kOffFac + 4 * 32 * 4;          // [8][4] row sums of a finished stream
constexpr int kOffMisc = kOffLm + 32 * 4;             // tmem slot, failed, merge flag, pad
constexpr int kOffMeta = kOffMisc + 16;               // prefix[batch + 1], lens[batch]
__host__ __device__ constexpr int umma_smem_bytes(int batch) { return 1024 + kOffMeta + (2 * batch + 2) * 4; }

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// A warp reads 16 consecutive columns of its 32 lanes (thread i <- lane base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// Instruction descriptor for kind::f8f6f4 with e4m3 operands (format code 0) and an fp32
// accumulator; the other fields as in umma_idesc_bf16_f32.
__device__ __forceinline__ uint32_t umma_idesc_e4m3_f32(int m, int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// The four most significant bits of x as a float (truncated, so the remainder keeps x's
// sign): an e4m3 value whenever 2^-6 <= |x| < 480.  Smaller x go to the remainder whole.
__device__ __forceinline__ float top4(float x) {
  return fabsf(x) >= 0.015625f ? __uint_as_float(__float_as_uint(x) & 0xfff00000u) : 0.f;
}

__global__ void __launch_bounds__(kUThreads, 1) attn_flat_umma_f8_kernel(AttnParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t ring_s = base, q_s = base + kOffQ, p_s = base + kOffP, bars = base + kOffBars;
  const uint32_t full0 = bars, empty0 = bars + 24, s_full = bars + 48, s_free = bars + 64, p_full = bars + 80,
                 o_full = bars + 96, o_free = bars + 104, q_ready = bars + 112, aux = bars + 120;
  float *fac_g = reinterpret_cast<float *>(sm + kOffFac);
  float *lm_g = reinterpret_cast<float *>(sm + kOffLm);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + kOffMisc);
  int *failed = reinterpret_cast<int *>(sm + kOffMisc + 4);
  int *merge_flag = reinterpret_cast<int *>(sm + kOffMisc + 8);
  int *prefix = reinterpret_cast<int *>(sm + kOffMeta);   // [batch + 1]
  int *lens = prefix + p.batch + 1;                       // [batch]

  const int g = p.h / p.kvh;
  const int slabs = p.kvh / kUHS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < kUStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full + 8 * b, 1);
      mbar_init(s_free + 8 * b, kUCWarps);
      mbar_init(p_full + 8 * b, kUCWarps);
    }
    mbar_init(o_full, 1);
    mbar_init(o_free, kUCWarps);
    mbar_init(q_ready, kUCWarps);
    mbar_init(aux, 1);
    mbar_fence_init();
    *failed = 0;
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  // rows of the Q and P operands that no thread ever writes (padding terms, q heads beyond g) stay zero
  for (int i = tid; i < (2 * kQSlabB + 4 * kPSlabB) / 16; i += kUThreads)
    reinterpret_cast<uint4 *>(sm + kOffQ)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < p.batch; i += kUThreads) {
    const int len = max(p.seq_lens[i], 0);
    lens[i] = len;
    prefix[i + 1] = len > 0 ? ((len + kUT - 1) / kUT + kBoundaryCost) * slabs : 0;
  }
  fence_proxy_async();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == 0) {
    int carry = 0;
    for (int b0 = 0; b0 < p.batch; b0 += 32) {
      const int i = b0 + lane;
      int v = i < p.batch ? prefix[i + 1] : 0;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += n;
      }
      if (i < p.batch) prefix[i + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) prefix[0] = 0;
  }
  __syncthreads();
  pdl_launch_dependents();
  const uint32_t tmem = *tmem_slot;
  const long long total = prefix[p.batch];
  const int n_ctas = static_cast<int>(min(static_cast<long long>(gridDim.x), total));
  const bool active = static_cast<int>(blockIdx.x) < n_ctas;
  const long long tau0 = active ? total * blockIdx.x / n_ctas : 0;
  const long long tau1 = active ? total * (blockIdx.x + 1) / n_ctas : 0;

  if (warp == 8) {
    // ---------------- producer ----------------
    // lanes 0-7 fetch K of kv heads 0-7 of the slab, lanes 8-15 V; all 32 lanes patch a stream's last tile
    bool ok = true;
    int it = 0;
    uint32_t aux_n = 0;
    for (long long tau = tau0; ok && tau < tau1;) {
      const Piece pc = locate(prefix, p.batch, slabs, tau, tau1);
      tau += pc.advance;
      if (pc.tile_end <= pc.tile_begin) continue;
      const int seq_len = lens[pc.b];
      const int64_t slot = p.slot_ids[pc.b];
      const char *map = static_cast<const char *>(p.maps) + static_cast<size_t>(slot) * 256 + ((lane >> 3) & 1) * 128;
      const int head = pc.slab * kUHS + (lane & 7);
      const bool fresh = p.new_key != nullptr && p.byte_off[pc.b] >= 0;
      for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
        const int s = it % kUStages;
        if (it >= kUStages && !mbar_wait(empty0 + 8 * s, ((it / kUStages) - 1) & 1)) { ok = false; break; }
        const int t0 = tile * kUT;
        const int nt = min(kUT, seq_len - t0);
        const bool patch = t0 + nt == seq_len && (nt < kUT || fresh);
        const uint32_t bar = patch ? aux : full0 + 8 * s;
        const uint32_t stage = ring_s + s * kUStageB;
        if (lane == 0) mbar_arrive_expect_tx(bar, kUStageB);
        __syncwarp();
        if (lane < 16) tma_load_3d(stage + (lane >> 3) * kKVTileB + (lane & 7) * kHeadTileB, map, 0, head, t0, bar);
        if (!patch) continue;
        if (!mbar_wait(aux, aux_n & 1)) { ok = false; break; }
        ++aux_n;
        unsigned char *kst = sm + s * kUStageB, *vst = kst + kKVTileB;
        const int j = lane >> 2, part = lane & 3;          // kv head of the slab, 32-byte quarter of its row
        for (int r = nt; r < kUT; ++r) {                   // whole rows: the swizzle only permutes chunks inside a row
          uint4 *row = reinterpret_cast<uint4 *>(vst + j * kHeadTileB + r * 128 + part * 32);
          row[0] = make_uint4(0, 0, 0, 0);
          row[1] = make_uint4(0, 0, 0, 0);
        }
        if (fresh) {
          // This step's row: quantised exactly as the append kernel does (true division), into the
          // stage for this launch and into the range for good.
          if (p.overlap == 2) pdl_wait_prior_grid();       // the preceding kernel may still be writing key / value
          const int kv_head = pc.slab * kUHS + j, r = nt - 1;
          const float ks = p.k_scale[kv_head], vs = p.v_scale[kv_head];
          const size_t dst = static_cast<size_t>(p.byte_off[pc.b]) + static_cast<size_t>(kv_head) * 128 + part * 32;
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const __nv_bfloat16 *src = kv ? static_cast<const __nv_bfloat16 *>(p.new_value) + pc.b * p.new_value_stride
                                          : static_cast<const __nv_bfloat16 *>(p.new_key) + pc.b * p.new_key_stride;
            const uint4 *x = reinterpret_cast<const uint4 *>(src + kv_head * kHeadDim + part * 32);
            const float sc = kv ? vs : ks;
            uint32_t w[8];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 v = __ldg(x + c);
              w[2 * c] = float2_to_e4m3x2(bf16_lo(v.x) / sc, bf16_hi(v.x) / sc) |
                         (float2_to_e4m3x2(bf16_lo(v.y) / sc, bf16_hi(v.y) / sc) << 16);
              w[2 * c + 1] = float2_to_e4m3x2(bf16_lo(v.z) / sc, bf16_hi(v.z) / sc) |
                             (float2_to_e4m3x2(bf16_lo(v.w) / sc, bf16_hi(v.w) / sc) << 16);
            }
            const uint4 c0 = make_uint4(w[0], w[1], w[2], w[3]), c1 = make_uint4(w[4], w[5], w[6], w[7]);
            unsigned char *st = (kv ? vst : kst) + j * kHeadTileB;
            *reinterpret_cast<uint4 *>(st + sw128_offset(r, 2 * part)) = c0;
            *reinterpret_cast<uint4 *>(st + sw128_offset(r, 2 * part + 1)) = c1;
            char *range = reinterpret_cast<char *>(kv ? p.v_table[slot] : p.k_table[slot]);
            *reinterpret_cast<uint4 *>(range + dst) = c0;
            *reinterpret_cast<uint4 *>(range + dst + 16) = c1;
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * s);
      }
    }
    if (!ok && lane == 0) *failed = 1;
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_e4m3_f32(128, 64, false, false);
      const uint32_t idesc_pv = umma_idesc_e4m3_f32(128, 16, true, false);
      bool ok = true;
      int it = 0, pieces = 0;
      // O^T of tile i (all 8 kv heads) into the O columns; releases the tile's ring stage
      auto issue_pv = [&](int i) -> bool {
        const int b = i & 1, s = i % kUStages;
        if (!mbar_wait(p_full + 8 * b, (i >> 1) & 1)) return false;          // P of tile i is in shared memory
        if (i >= 1 && !mbar_wait(o_free, (i - 1) & 1)) return false;         // O^T of tile i - 1 was read
        tcgen05_fence_after();
        const uint32_t vst = ring_s + s * kUStageB + kKVTileB;
#pragma unroll
        for (int j = 0; j < kUHS; ++j) {
          const uint64_t da = umma_desc_sw128(vst + j * kHeadTileB, 0, 1024);                           // 32 tokens x 128 dims
          const uint64_t db = umma_desc_sw128(p_s + (b * 2 + (j >> 2)) * kPSlabB + (j & 3) * 32, 0, 1024);
          umma_f8(tmem + kColO + j * 16, da, db, idesc_pv, false);
        }
        umma_commit(o_full);
        umma_commit(empty0 + 8 * s);
        return true;
      };
      for (long long tau = tau0; ok && tau < tau1;) {
        const Piece pc = locate(prefix, p.batch, slabs, tau, tau1);
        tau += pc.advance;
        if (pc.tile_end <= pc.tile_begin) continue;
        // A new stream brings a new Q: the consumers write it only after the previous stream's
        // last product is done, so that product goes out first.
        if (it > 0 && !issue_pv(it - 1)) { ok = false; break; }
        if (!mbar_wait(q_ready, pieces & 1)) { ok = false; break; }
        ++pieces;
        for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
          const int b = it & 1, s = it % kUStages;
          if (!mbar_wait(full0 + 8 * s, (it / kUStages) & 1)) { ok = false; break; }
          if (it >= 2 && !mbar_wait(s_free + 8 * b, ((it >> 1) - 1) & 1)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t kst = ring_s + s * kUStageB;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint64_t da = umma_desc_sw128(kst + hf * 4 * kHeadTileB + ks * 32, 0, 1024);
              const uint64_t db = umma_desc_sw128(q_s + hf * kQSlabB + ks * 32, 0, 1024);
              umma_f8(tmem + kColS + b * 128 + hf * 64, da, db, idesc_qk, ks > 0);
            }
          umma_commit(s_full + 8 * b);
          if (tile > pc.tile_begin && !issue_pv(it - 1)) { ok = false; break; }
        }
      }
      if (ok && it > 0 && !issue_pv(it - 1)) ok = false;
      if (!ok) *failed = 1;
    }
  } else {
    // ---------------- consumer warps ----------------
    const int j = warp, hf = warp >> 2, qd = warp & 3;     // softmax: kv head j of the slab; accumulate: dims [32 qd, +32) of heads 4 hf .. 4 hf + 3
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(32 * qd) << 16);
    const float sl2_base = p.scale * 1.4426950408889634f;
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
    unsigned char *q_g = sm + kOffQ + hf * kQSlabB;

    // Sequences without context produce zeros; nobody owns a tile of theirs.
    if (blockIdx.x == 0) {
      for (int b = 0; b < p.batch; ++b)
        if (prefix[b + 1] == prefix[b]) {
          for (int i = tid; i < p.h * kHeadDim; i += kUCWarps * 32) out[b * p.out_stride + i] = __float2bfloat16(0.f);
          if (p.lse && tid < p.h) p.lse[b * p.h + tid] = -INFINITY;
        }
    }

    bool ok = true;
    int it = 0;
    bool first_piece = true;
    float acc[4][4];          // [kv head 4 hf + jj][q head]: output dim 32 qd + lane, in units of 2^-max / 256
    // Adds O^T of tile i into acc.  The factors come from the softmax warps through shared memory.
    auto accumulate = [&](int i) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(p_full + 8 * (i & 1), (i >> 1) & 1))) return false;   // all eight warps wrote their factors
      if (!__all_sync(0xffffffffu, mbar_wait(o_full, i & 1))) return false;
      tcgen05_fence_after();
      float c[4][16];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) tmem_ld_32x32b_x16(lane_addr + kColO + (4 * hf + jj) * 16, c[jj]);
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
      const float4 *f4 = reinterpret_cast<const float4 *>(fac_g + ((i & 3) * 8 + 4 * hf) * 4);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float4 f = f4[jj];
        acc[jj][0] = fmaf(acc[jj][0], f.x, c[jj][0] + c[jj][4] + c[jj][8]);
        acc[jj][1] = fmaf(acc[jj][1], f.y, c[jj][1] + c[jj][5] + c[jj][9]);
        acc[jj][2] = fmaf(acc[jj][2], f.z, c[jj][2] + c[jj][6] + c[jj][10]);
        acc[jj][3] = fmaf(acc[jj][3], f.w, c[jj][3] + c[jj][7] + c[jj][11]);
      }
      return true;
    };

    // A wait that runs out marks the warp as failed: it then skips the tile work but still walks
    // through every piece and every CTA barrier below, so that no other warp is left waiting for it.
    for (long long tau = tau0; tau < tau1;) {
      const Piece pc = locate(prefix, p.batch, slabs, tau, tau1);
      tau += pc.advance;
      if (pc.tile_end <= pc.tile_begin) continue;
      const int seq_len = lens[pc.b];
      const int kv_head = pc.slab * kUHS + j;
      // ---- Q of this kv head -> B operand: per q head a power of two brings the largest
      // element into [128, 256), then hi = top 4 bits, lo = the rest (exact for bf16) ----
      if (p.overlap == 2) pdl_wait_prior_grid();   // q may be the preceding kernel's output
      float sl2h[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        sl2h[h] = 0.f;
        if (h < g) {
          const uint2 v = __ldg(reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(p.q) + pc.b * p.q_stride +
                                                                (kv_head * g + h) * kHeadDim) + lane);
          float x[4] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y)};
          float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
          int k = 0;
          if (amax > 0.f && amax < INFINITY) k = min(max(7 - (static_cast<int>(__float_as_uint(amax) >> 23) - 127), -100), 100);
          const float mult = __uint_as_float(static_cast<uint32_t>(k + 127) << 23);
          sl2h[h] = sl2_base * p.k_scale[kv_head] * __uint_as_float(static_cast<uint32_t>(127 - k) << 23);
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            x[e] *= mult;
            hi[e] = top4(x[e]);
            lo[e] = x[e] - hi[e];
          }
          const uint32_t whi = float2_to_e4m3x2(hi[0], hi[1]) | (float2_to_e4m3x2(hi[2], hi[3]) << 16);
          const uint32_t wlo = float2_to_e4m3x2(lo[0], lo[1]) | (float2_to_e4m3x2(lo[2], lo[3]) << 16);
          *reinterpret_cast<uint32_t *>(q_g + sw128_offset(16 * qd + h, lane >> 2) + (lane & 3) * 4) = whi;
          *reinterpret_cast<uint32_t *>(q_g + sw128_offset(16 * qd + 4 + h, lane >> 2) + (lane & 3) * 4) = wlo;
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);

      float m[4], l[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[jj][h] = 0.f;
      }
      for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
        // ---- softmax of tile `it`: lane = token ----
        if (!ok) continue;
        const int b = it & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(s_full + 8 * b, (it >> 1) & 1))) { ok = false; continue; }
        tcgen05_fence_after();
        float c[16];
        tmem_ld_32x32b_x16(lane_addr + kColS + b * 128 + hf * 64 + 16 * qd, c);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free + 8 * b);
        const bool valid = tile * kUT + lane < seq_len;
        unsigned char *prow = sm + kOffP + (b * 2 + hf) * kPSlabB + (lane & 15);
        const int chunk = 2 * qd + (lane >> 4);
        float fac[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float s = valid ? (c[h] + c[4 + h]) * sl2h[h] : -INFINITY;
          float mx = s;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
          const float mn = fmaxf(m[h], mx);        // finite: the first token of a tile is always valid
          fac[h] = exp2f(m[h] - mn);
          m[h] = mn;
          const float pr = exp2f(s - mn);
          l[h] = fmaf(l[h], fac[h], pr);
          if (h < g) {
            const float pq = pr * kPScale;
            const float hi = top4(pq), r1 = pq - hi, mid = top4(r1), lo = r1 - mid;
            const uint32_t w = float2_to_e4m3x2(hi, mid);
            prow[sw128_offset(h, chunk)] = static_cast<unsigned char>(w & 0xffu);
            prow[sw128_offset(4 + h, chunk)] = static_cast<unsigned char>(w >> 8);
            prow[sw128_offset(8 + h, chunk)] = static_cast<unsigned char>(float2_to_e4m3x2(lo, 0.f) & 0xffu);
          }
        }
#pragma unroll
        for (int h = 0; h < 4; ++h)
          if (lane == h) fac_g[((it & 3) * 8 + j) * 4 + h] = fac[h];
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 8 * b);
        // ---- accumulate the previous tile of this stream (its P.V ran during the softmax above) ----
        if (tile > pc.tile_begin && !accumulate(it - 1)) ok = false;
      }
      if (ok && !accumulate(it - 1)) ok = false;
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], off);

      const bool whole = pc.tile_begin == 0 && pc.tile_end == pc.tiles_in_stream;
      if (whole) {
        // This CTA saw the whole stream: the softmax warps hand the row sums over, the
        // accumulating threads normalise and write.
#pragma unroll
        for (int h = 0; h < 4; ++h)
          if (lane == h) lm_g[j * 4 + h] = l[h];
        if (p.lse) {
#pragma unroll
          for (int h = 0; h < 4; ++h)
            if (lane == h && h < g) p.lse[pc.b * p.h + kv_head * g + h] = (m[h] + log2f(l[h])) * 0.6931471805599453f;
        }
        named_bar_sync(1, kUCWarps * 32);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int kvh_abs = pc.slab * kUHS + 4 * hf + jj;
          const float vs = p.v_scale[kvh_abs] * (1.f / kPScale);
#pragma unroll
          for (int h = 0; h < 4; ++h)
            if (h < g)
              out[pc.b * p.out_stride + (kvh_abs * g + h) * kHeadDim + 32 * qd + lane] =
                  __float2bfloat16(acc[jj][h] * vs / lm_g[(4 * hf + jj) * 4 + h]);
        }
        named_bar_sync(1, kUCWarps * 32);   // the sums are rewritten by the next stream
      } else {
        // Publish this piece in the scratch format of the merge (one row per (kv head, q head):
        // O[128], max, sum), draw a ticket, and merge the stream if it was the last one.
        if (p.overlap) pdl_wait_prior_grid();   // the scratch is shared with the previous launch
        const int slot_id = first_piece ? 0 : 1;
        float *slot_base = p.fl_part + (static_cast<size_t>(blockIdx.x) * 2 + slot_id) * kUCWarps * 8 * kPartRow;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int h = 0; h < 4; ++h)
            if (h < g) slot_base[((4 * hf + jj) * 8 + h) * kPartRow + 32 * qd + lane] = acc[jj][h] * (1.f / kPScale);
#pragma unroll
        for (int h = 0; h < 4; ++h)
          if (lane == h && h < g) {
            slot_base[(j * 8 + h) * kPartRow + 128] = m[h];
            slot_base[(j * 8 + h) * kPartRow + 129] = l[h];
          }
        __threadfence();
        named_bar_sync(1, kUCWarps * 32);
        const int c_first = owner_of(pc.stream_begin + kBoundaryCost, total, n_ctas);
        const int c_last = owner_of(pc.stream_end - 1, total, n_ctas);
        if (tid == 0) {
          unsigned *ctr = p.fl_count + pc.b * slabs + pc.slab;
          const unsigned old = atomicAdd(ctr, 1u);
          const int last = old + 1 == static_cast<unsigned>(c_last - c_first + 1);
          if (last) *ctr = 0u;   // leaves the counters clean for the next launch
          *merge_flag = last;
        }
        named_bar_sync(1, kUCWarps * 32);
        const bool merger = *merge_flag != 0;
        named_bar_sync(1, kUCWarps * 32);   // the flag may be rewritten by the next piece
        if (merger) merge_stream<kUCWarps, kUHS, 1, 8, true>(p, pc, total, n_ctas, c_first, c_last, warp, lane, g);
      }
      first_piece = false;
    }
    if (!ok && lane == 0) *failed = 1;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, kTmemCols);
  if (tid == 0 && *failed) atomicExch(p.status, kKernelErrMagic);
}

}  // namespace

bool attn_flat_umma_supports(int batch, int h, int kvh, int kv_dtype) {
  const int g = kvh > 0 ? h / kvh : 0;
  return kv_dtype == VT_KV_FP8_E4M3 && batch <= kFlatMaxBatch && kvh % kUHS == 0 && (kvh & (kvh - 1)) == 0 &&
         kvh * kUT <= 8192 && (g == 1 || g == 2 || g == 4);
}

int launch_attn_flat_umma(const AttnParams &p_in, cudaStream_t stream) {
  if (!p_in.maps || !attn_flat_umma_supports(p_in.batch, p_in.h, p_in.kvh, VT_KV_FP8_E4M3)) return VT_ERR_UNSUPPORTED;
  AttnParams p = p_in;
  int dev = 0, sms = kFlatSms;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  p.n_ctas = std::min(std::max(sms, 1), kFlatSms);
  const int smem = umma_smem_bytes(p.batch);
  static SmemOptIn opt_in;
  if (!opt_in.ensure(attn_flat_umma_f8_kernel, smem)) return VT_ERR_CUDA;
  if (p.overlap) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_ctas);
    cfg.blockDim = dim3(kUThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, attn_flat_umma_f8_kernel, p) == cudaSuccess ? VT_OK : VT_ERR_CUDA;
  }
  attn_flat_umma_f8_kernel<<<p.n_ctas, kUThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

// Fills host_maps[slot][K, V] for fp8 ranges of kvh heads: element (byte x, head, token),
// heads 128 bytes apart, tokens kvh * 128 bytes apart; box = 128 bytes x 1 head x 32 tokens.
int encode_decode_maps_f8(const uint64_t *k_bases, const uint64_t *v_bases, int n_slots, int kvh, uint64_t max_tokens,
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
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(kvh), max_tokens};
  const cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(kvh) * 128};
  const cuuint32_t box[3] = {128, 1, static_cast<cuuint32_t>(kUT)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  CUtensorMap *out = static_cast<CUtensorMap *>(host_maps);
  for (int s = 0; s < n_slots; ++s)
    for (int kv = 0; kv < 2; ++kv) {
      const uint64_t base = kv ? v_bases[s] : k_bases[s];
      if (base == 0 || (base & 15) != 0) return VT_ERR_INVALID;
      if (encode(&out[2 * s + kv], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, reinterpret_cast<void *>(base), dims, strides, box,
                 elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return VT_ERR_DRIVER;
    }
  return VT_OK;
}

}  // namespace vt
