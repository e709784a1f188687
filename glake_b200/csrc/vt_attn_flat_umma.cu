// Decode attention over an fp8 e4m3 cache on the 5th-generation tensor cores
// (tcgen05.mma.kind::f8f6f4, accumulators in tensor memory): the cache bytes go from
// HBM through shared memory into the tensor core without ever being converted by a
// thread.  Same persistent schedule, scratch format and merge as the mma.sync kernel
// of vt_attn_flat.cu (pieces, tickets, last CTA of a stream merges); the engine differs.
//
// Shapes: kv heads a power of two >= 8 (one CTA streams a slab of 8 kv heads = 1 KiB of every token row),
// 1, 2 or 4 q heads per kv head, head size 128.  Needs the per-slot TMA tensor maps
// of encode_decode_maps_f8: a tile is 32 tokens x 8 kv heads, fetched as sixteen
// 128-byte-swizzled boxes (32 tokens x 128 bytes of one kv head; K, then V).
//
// One CTA per SM, nineteen warps:
//   warps 16, 17  producers of K and of V: tensor copies into a 3-stage ring (2 x 32 KiB per stage,
//            handed over separately).  The last tile of a stream is patched by these warps before it is handed on: V rows past
//            the context are cleared (0 x NaN would poison the product) and, in a fused
//            step, this step's K / V row is quantised into the stage and into the range.
//   warp 18  one lane issues the MMAs.
//            S^T = K . Q^T : A = K rows of four kv heads (M = 128 = 4 heads x 32 tokens,
//            K-major), B = Q of those heads as TWO e4m3 terms per q head (hi + lo, each
//            head scaled by its own power of two: exact for bf16 inputs), N = 32.
//            Three quarters of that product pair a kv head with another head's Q and
//            are never read: the tensor core has the time, the threads do not.
//            O^T = V^T . P^T per kv head: A = V (MN-major, M = 128 dims, K = 32 tokens),
//            B = P as THREE e4m3 terms per q head (12 significant bits), N = 16, into
//            a fresh accumulator per tile.
//   warps 0-15 consumers, two sets of eight: set b takes the tiles of parity b and has its own
//            S^T, P and O^T buffers and its own running (max, sum, O) state, so that one set
//            computes while the other waits for a product (a set alone is latency-bound: measured
//            1.5 us per tile against 1.4 us of HBM time).  Softmax: warp j of a set owns kv head
//            j, lane = token (the TMEM lane of its row of S^T): tcgen05.ld of 8 columns, running
//            max over the warp by shuffles, P split into terms and stored as bytes.  Accumulate:
//            the same warps then add the tile's O^T (lane = output dim) into registers with the
//            usual rescale.  The two sets' states are merged with the other pieces of the stream.
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
constexpr int kUCWarps = 16;                   // two sets of eight
constexpr int kUThreads = (kUCWarps + 3) * 32;
constexpr int kUStages = 3;
constexpr int kHeadTileB = kUT * 128;         // one kv head's rows of a tile: [32 tokens][128 B]
constexpr int kKVTileB = kUHS * kHeadTileB;   // K (or V) of a tile
constexpr int kUStageB = 2 * kKVTileB;        // 64 KiB
constexpr int kQSlabB = 32 * 128;             // Q operand of four kv heads: 8 rows each (2 terms x 4 q heads); two buffers x two halves
constexpr int kPSlabB = 16 * 128;             // P operand of four kv heads: 16 rows (3 terms x 4 heads + 4 zero rows), 32 bytes of tokens each
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;                 // S^T buffer b, half hf: columns [64 b + 32 hf, + 32)
constexpr uint32_t kColO = 128;               // O^T of consumer set b, kv head j: columns [128 + 128 b + 16 j, + 16)
// Phantom positions per stream in the cost-balanced split: a stream boundary stalls the consumers
// (publish, ticket, possibly merge) for longer than the four or five tiles its own work takes: the producers wait for the stream's last tile
// to land before they patch it, and the CTA that ends a stream usually merges it.  Measured per
// boundary: 14 us against 1.25 us per 64 KiB tile; costs of 4 to 16 tiles time alike (within 1 %).
constexpr int kUCost = 8;
constexpr float kPScale = 256.f;              // P is carried as 256 p: e4m3 then resolves 2^-17 of the largest term

// offsets from the 1024-byte aligned base of the dynamic shared memory
constexpr int kOffQ = kUStages * kUStageB;            // 196608
constexpr int kOffP = kOffQ + 4 * kQSlabB;            // 212992: [2 buffers][2 slabs]
constexpr int kOffBars = kOffP + 4 * kPSlabB;         // 221184: 25 mbarriers
constexpr int kOffFac = kOffBars + 26 * 8;            // per set a ring of 2 x [8 kv heads][4 heads] rescale factors
constexpr int kOffMisc = kOffFac + 4 * 32 * 4;        // tmem slot, failed, merge flag, pad
constexpr int kOffMeta = kOffMisc + 16;               // prefix[batch + 1], lens[batch]
__host__ __device__ constexpr int umma_smem_bytes(int batch) { return 1024 + kOffMeta + (2 * batch + 2) * 4; }

// Tensor copy with an L2 eviction-priority hint (KV rows are streamed once per step).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *map, int x, int y, int z, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
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
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
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
__device__ __forceinline__ float ex2_approx(float x) {      // 2^x, one MUFU op; -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Non-blocking look at an mbarrier phase (mbar_wait's try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
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
  const uint32_t k_full = bars, v_full = bars + 24, k_empty = bars + 48, v_empty = bars + 72, s_full = bars + 96,
                 s_free = bars + 112, p_full = bars + 128, o_full = bars + 144, o_free = bars + 160, q_ready = bars + 176,
                 aux_k = bars + 184, aux_v = bars + 192;
  float *fac_g = reinterpret_cast<float *>(sm + kOffFac);
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
      mbar_init(k_full + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {                        // one of each per consumer set
      mbar_init(s_full + 8 * b, 1);
      mbar_init(s_free + 8 * b, 8);
      mbar_init(p_full + 8 * b, 8);
      mbar_init(o_full + 8 * b, 1);
      mbar_init(o_free + 8 * b, 8);
    }
    mbar_init(q_ready, 8);                                // set 0 writes Q
    mbar_init(aux_k, 1);
    mbar_init(aux_v, 1);
    mbar_fence_init();
    *failed = 0;
  }
  if (warp == kUCWarps + 2) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  // rows of the Q and P operands that no thread ever writes (padding terms, q heads beyond g) stay zero
  for (int i = tid; i < (4 * kQSlabB + 4 * kPSlabB) / 16; i += kUThreads)
    reinterpret_cast<uint4 *>(sm + kOffQ)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < p.batch; i += kUThreads) {
    const int len = max(p.seq_lens[i], 0);
    lens[i] = len;
    prefix[i + 1] = len > 0 ? ((len + kUT - 1) / kUT + kUCost) * slabs : 0;
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

  if (warp == kUCWarps || warp == kUCWarps + 1) {
    // ---------------- producers: warp 16 fetches K, warp 17 V ----------------
    // K and V of a stage are handed over separately: the K slot is free as soon as S^T of its tile is
    // done, long before the P.V product releases the V slot, so K runs further ahead of the consumers
    // (with one barrier per stage the ring was too shallow for the loaded HBM latency).
    // lanes 0-7 fetch kv heads 0-7 of the slab; all 32 lanes patch a stream's last tile.
    const int kv = warp - kUCWarps;
    const uint32_t full = kv ? v_full : k_full, empty = kv ? v_empty : k_empty, aux = kv ? aux_v : aux_k;
    const uint64_t policy = l2_policy_evict_first();
    bool ok = true;
    int it = 0;
    uint32_t aux_n = 0;
    for (long long tau = tau0; ok && tau < tau1;) {
      const Piece pc = locate<kUCost>(prefix, p.batch, slabs, tau, tau1);
      tau += pc.advance;
      if (pc.tile_end <= pc.tile_begin) continue;
      const int seq_len = lens[pc.b];
      const int64_t slot = p.slot_ids[pc.b];
      const char *map = static_cast<const char *>(p.maps) + static_cast<size_t>(slot) * 256 + kv * 128;
      const int head = pc.slab * kUHS + (lane & 7);
      const bool fresh = p.new_key != nullptr && p.byte_off[pc.b] >= 0;
      for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
        const int s = it % kUStages;
        if (it >= kUStages && !mbar_wait(empty + 8 * s, ((it / kUStages) - 1) & 1)) { ok = false; break; }
        const int t0 = tile * kUT;
        const int nt = min(kUT, seq_len - t0);
        const bool patch = t0 + nt == seq_len && (fresh || (kv && nt < kUT));
        const uint32_t bar = patch ? aux : full + 8 * s;
        const uint32_t stage = ring_s + s * kUStageB + kv * kKVTileB;
        if (lane == 0) mbar_arrive_expect_tx(bar, kKVTileB);
        __syncwarp();
        if (lane < 8) tma_load_3d(stage + lane * kHeadTileB, map, 0, head, t0, bar, policy);
        if (!patch) continue;
        if (!mbar_wait(aux, aux_n & 1)) { ok = false; break; }
        ++aux_n;
        unsigned char *st = sm + s * kUStageB + kv * kKVTileB;
        const int j = lane >> 2, part = lane & 3;          // kv head of the slab, 32-byte quarter of its row
        if (kv)
          for (int r = nt; r < kUT; ++r) {                 // whole rows: the swizzle only permutes chunks inside a row
            uint4 *row = reinterpret_cast<uint4 *>(st + j * kHeadTileB + r * 128 + part * 32);
            row[0] = make_uint4(0, 0, 0, 0);
            row[1] = make_uint4(0, 0, 0, 0);
          }
        if (fresh) {
          // This step's row: quantised exactly as the append kernel does (true division), into the
          // stage for this launch and into the range for good.
          if (p.overlap == 2) pdl_wait_prior_grid();       // the preceding kernel may still be writing key / value
          const int kv_head = pc.slab * kUHS + j, r = nt - 1;
          const float sc = kv ? p.v_scale[kv_head] : p.k_scale[kv_head];
          const size_t dst = static_cast<size_t>(p.byte_off[pc.b]) + static_cast<size_t>(kv_head) * 128 + part * 32;
          const __nv_bfloat16 *src = kv ? static_cast<const __nv_bfloat16 *>(p.new_value) + pc.b * p.new_value_stride
                                        : static_cast<const __nv_bfloat16 *>(p.new_key) + pc.b * p.new_key_stride;
          const uint4 *x = reinterpret_cast<const uint4 *>(src + kv_head * kHeadDim + part * 32);
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
          *reinterpret_cast<uint4 *>(st + j * kHeadTileB + sw128_offset(r, 2 * part)) = c0;
          *reinterpret_cast<uint4 *>(st + j * kHeadTileB + sw128_offset(r, 2 * part + 1)) = c1;
          char *range = reinterpret_cast<char *>(kv ? p.v_table[slot] : p.k_table[slot]);
          *reinterpret_cast<uint4 *>(range + dst) = c0;
          *reinterpret_cast<uint4 *>(range + dst + 16) = c1;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(full + 8 * s);
      }
    }
    if (!ok && lane == 0) *failed = 1;
  } else if (warp == kUCWarps + 2) {
    // ---------------- MMA issuer ----------------
    // One lane issues both kinds of product, whichever is ready: S^T of the next tile needs its K tile,
    // a free S^T buffer and (at a stream's first tile) the new Q; O^T of the oldest tile without one
    // needs its V tile, its P and a free O^T buffer.  Neither waits behind the other (a P.V product
    // queued behind the next tile's K would keep its V stage, and the consumers, waiting), so the
    // barriers are polled, not waited on; a second without any progress fails the launch.
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_e4m3_f32(128, 32, false, false);
      const uint32_t idesc_pv = umma_idesc_e4m3_f32(128, 16, true, false);
      bool ok = true;
      int qk_it = 0, pv_it = 0, pieces = 0;      // tiles whose S^T / O^T product has been issued; streams begun
      long long tau = tau0;
      Piece pc{};
      int tile = 0;                              // next tile of pc (tile == pc.tile_end: fetch the next piece)
      bool have_q = false;                       // the current piece's Q operand has been seen ready
      unsigned long long idle_since = 0;
      for (;;) {
        bool progress = false;
        // ---- O^T of tile pv_it ----
        if (pv_it < qk_it) {
          const int i = pv_it, b = i & 1, s = i % kUStages;
          if (mbar_test(v_full + 8 * s, (i / kUStages) & 1) && mbar_test(p_full + 8 * b, (i >> 1) & 1) &&
              (i < 2 || mbar_test(o_free + 8 * b, ((i >> 1) - 1) & 1))) {
            tcgen05_fence_after();
            const uint32_t vst = ring_s + s * kUStageB + kKVTileB;
#pragma unroll
            for (int j = 0; j < kUHS; ++j) {
              const uint64_t da = umma_desc_sw128(vst + j * kHeadTileB, 0, 1024);                           // 32 tokens x 128 dims
              const uint64_t db = umma_desc_sw128(p_s + (b * 2 + (j >> 2)) * kPSlabB + (j & 3) * 32, 0, 1024);
              umma_f8(tmem + kColO + b * 128 + j * 16, da, db, idesc_pv, false);
            }
            umma_commit(o_full + 8 * b);
            umma_commit(v_empty + 8 * s);         // releases the V half of the ring stage
            ++pv_it;
            progress = true;
          }
        }
        // ---- S^T of tile qk_it ----
        while (tile >= pc.tile_end && tau < tau1) {            // next piece with real tiles
          pc = locate<kUCost>(prefix, p.batch, slabs, tau, tau1);
          tau += pc.advance;
          tile = pc.tile_begin;
          if (pc.tile_end > pc.tile_begin) {
            have_q = false;
            ++pieces;
          }
        }
        const bool more_qk = tile < pc.tile_end;
        if (more_qk) {
          const int it = qk_it, b = it & 1, s = it % kUStages;
          const int qbuf = (pieces - 1) & 1;                   // Q operands alternate between two buffers
          if (!have_q) have_q = mbar_test(q_ready, (pieces - 1) & 1);
          if (have_q && mbar_test(k_full + 8 * s, (it / kUStages) & 1) &&
              (it < 2 || mbar_test(s_free + 8 * b, ((it >> 1) - 1) & 1))) {
            tcgen05_fence_after();
            const uint32_t kst = ring_s + s * kUStageB;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                const uint64_t da = umma_desc_sw128(kst + hf * 4 * kHeadTileB + ks * 32, 0, 1024);
                const uint64_t db = umma_desc_sw128(q_s + (qbuf * 2 + hf) * kQSlabB + ks * 32, 0, 1024);
                umma_f8(tmem + kColS + b * 64 + hf * 32, da, db, idesc_qk, ks > 0);
              }
            umma_commit(s_full + 8 * b);
            umma_commit(k_empty + 8 * s);         // releases the K half of the ring stage
            ++qk_it;
            ++tile;
            progress = true;
          }
        }
        if (!more_qk && pv_it == qk_it) break;   // every tile of the share has both products on their way
        if (progress) {
          idle_since = 0;
        } else {
          const unsigned long long now = global_timer_ns();
          if (idle_since == 0) idle_since = now;
          else if (now - idle_since > kWaitLimitNs) { ok = false; break; }
        }
      }
      if (!ok) *failed = 1;
    }
  } else {
    // ---------------- consumer warps: two sets of eight, set = parity of the tile ----------------
    const int set = warp >> 3, ws = warp & 7;
    const int j = ws, hf = ws >> 2, qd = ws & 3;           // softmax: kv head j of the slab; accumulate: dims [32 qd, +32) of heads 4 hf .. 4 hf + 3
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(32 * qd) << 16);
    const float sl2_base = p.scale * 1.4426950408889634f;
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);

    // Sequences without context produce zeros; nobody owns a tile of theirs.
    if (blockIdx.x == 0) {
      for (int b = 0; b < p.batch; ++b)
        if (prefix[b + 1] == prefix[b]) {
          for (int i = tid; i < p.h * kHeadDim; i += kUCWarps * 32) out[b * p.out_stride + i] = __float2bfloat16(0.f);
          if (p.lse && tid < p.h) p.lse[b * p.h + tid] = -INFINITY;
        }
    }

    bool ok = true;
    int it = 0, pieces = 0;
    bool first_piece = true;
    // The next piece of this CTA's share that holds real tiles (tile_end == tile_begin: none left).
    long long tau = tau0;
    auto next_piece = [&]() -> Piece {
      Piece pc{};
      while (tau < tau1) {
        pc = locate<kUCost>(prefix, p.batch, slabs, tau, tau1);
        tau += pc.advance;
        if (pc.tile_end > pc.tile_begin) return pc;
      }
      pc.tile_begin = pc.tile_end = 0;
      return pc;
    };
    // Q of this warp's kv head for a piece: fetched into registers a whole stream ahead ...
    auto load_q = [&](const Piece &pc, uint2 (&qr)[4]) {
      const __nv_bfloat16 *src = static_cast<const __nv_bfloat16 *>(p.q) + pc.b * p.q_stride + (pc.slab * kUHS + j) * g * kHeadDim;
#pragma unroll
      for (int h = 0; h < 4; ++h) qr[h] = h < g ? __ldg(reinterpret_cast<const uint2 *>(src + h * kHeadDim) + lane) : make_uint2(0, 0);
    };
    // ... and written by set 0 as the B operand (buffer = piece parity): per q head a power of two
    // brings the largest element into [128, 256), then hi = top 4 bits, lo = the rest (exact for
    // bf16).  Both sets derive the logit scales from it.
    auto write_q = [&](const Piece &pc, const uint2 (&qr)[4], int buf, float (&sl2h)[4]) {
      unsigned char *q_g = sm + kOffQ + (buf * 2 + hf) * kQSlabB;
      const float ksc = sl2_base * p.k_scale[pc.slab * kUHS + j];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        sl2h[h] = 0.f;
        if (h < g) {
          float x[4] = {bf16_lo(qr[h].x), bf16_hi(qr[h].x), bf16_lo(qr[h].y), bf16_hi(qr[h].y)};
          float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
          int k = 0;
          if (amax > 0.f && amax < INFINITY) k = min(max(7 - (static_cast<int>(__float_as_uint(amax) >> 23) - 127), -100), 100);
          const float mult = __uint_as_float(static_cast<uint32_t>(k + 127) << 23);
          sl2h[h] = ksc * __uint_as_float(static_cast<uint32_t>(127 - k) << 23);
          if (set == 0) {
            float hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              x[e] *= mult;
              hi[e] = top4(x[e]);
              lo[e] = x[e] - hi[e];
            }
            const uint32_t whi = float2_to_e4m3x2(hi[0], hi[1]) | (float2_to_e4m3x2(hi[2], hi[3]) << 16);
            const uint32_t wlo = float2_to_e4m3x2(lo[0], lo[1]) | (float2_to_e4m3x2(lo[2], lo[3]) << 16);
            *reinterpret_cast<uint32_t *>(q_g + sw128_offset(8 * qd + h, lane >> 2) + (lane & 3) * 4) = whi;
            *reinterpret_cast<uint32_t *>(q_g + sw128_offset(8 * qd + 4 + h, lane >> 2) + (lane & 3) * 4) = wlo;
          }
        }
      }
      if (set == 0) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_ready);
      }
    };
    // shared-memory byte of P for (term, q head) of this lane's token: constant per warp but for the term / head
    unsigned char *prow = sm + kOffP + (set * 2 + hf) * kPSlabB + (lane & 15);
    const int chunk = 2 * qd + (lane >> 4);
    float *fac_w = fac_g + set * 64;                      // per set: ring of 2 x [8 kv heads][4 q heads]

    // A wait that runs out marks the warp as failed: it then skips the tile work but still walks
    // through every piece and every CTA barrier below, so that no other warp is left waiting for it.
    Piece pc = next_piece();
    float sl2h[4] = {0.f, 0.f, 0.f, 0.f};
    if (pc.tile_end > pc.tile_begin) {
      if (p.overlap == 2) pdl_wait_prior_grid();   // q may be the preceding kernel's output
      uint2 qr[4];
      load_q(pc, qr);
      write_q(pc, qr, 0, sl2h);
    }
    while (pc.tile_end > pc.tile_begin) {
      const Piece nxt = next_piece();
      const bool more = nxt.tile_end > nxt.tile_begin;
      uint2 qn[4];
      if (more) load_q(nxt, qn);
      const int seq_len = lens[pc.b];
      float m[4], l[4];
      float acc[4][4];        // [kv head 4 hf + jj][q head]: output dim 32 qd + lane, in units of 2^-max / 256
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[jj][h] = 0.f;
      }
      for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
        if (!ok || (it & 1) != set) continue;
        const int kt = it >> 1;                              // this set's tile counter
        // ---- softmax: lane = token ----
        if (!__all_sync(0xffffffffu, mbar_wait(s_full + 8 * set, kt & 1))) { ok = false; continue; }
        tcgen05_fence_after();
        float c[8];
        tmem_ld_32x32b_x8(lane_addr + kColS + set * 64 + hf * 32 + 8 * qd, c);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free + 8 * set);
        const bool valid = tile * kUT + lane < seq_len;
        float fac[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float s = valid ? (c[h] + c[4 + h]) * sl2h[h] : -INFINITY;
          float mx = s;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
          const float mn = fmaxf(m[h], mx);        // finite: the first token of a tile is always valid
          fac[h] = ex2_approx(m[h] - mn);
          m[h] = mn;
          const float pr = ex2_approx(s - mn);
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
          if (lane == h) fac_w[((kt & 1) * 8 + j) * 4 + h] = fac[h];
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 8 * set);
        // ---- accumulate: lane = output dim.  The other set works on its tile while this one
        // waits for the product ----
        if (!__all_sync(0xffffffffu, mbar_wait(o_full + 8 * set, kt & 1))) { ok = false; continue; }
        tcgen05_fence_after();
        // the product completed, so every warp of the set had written its factors (p_full came first)
        const float4 *f4 = reinterpret_cast<const float4 *>(fac_w + ((kt & 1) * 8 + 4 * hf) * 4);
#pragma unroll
        for (int j2 = 0; j2 < 4; j2 += 2) {                  // two kv heads at a time: 32 registers in flight
          float o[2][16];
          tmem_ld_32x32b_x16(lane_addr + kColO + set * 128 + (4 * hf + j2) * 16, o[0]);
          tmem_ld_32x32b_x16(lane_addr + kColO + set * 128 + (4 * hf + j2 + 1) * 16, o[1]);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float4 f = f4[j2 + e];
            acc[j2 + e][0] = fmaf(acc[j2 + e][0], f.x, o[e][0] + o[e][4] + o[e][8]);
            acc[j2 + e][1] = fmaf(acc[j2 + e][1], f.y, o[e][1] + o[e][5] + o[e][9]);
            acc[j2 + e][2] = fmaf(acc[j2 + e][2], f.z, o[e][2] + o[e][6] + o[e][10]);
            acc[j2 + e][3] = fmaf(acc[j2 + e][3], f.w, o[e][3] + o[e][7] + o[e][11]);
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free + 8 * set);
      }
      // The next stream's Q goes out before this one is wrapped up, so that its first products
      // run while these warps publish and merge.
      ++pieces;
      float sl2n[4] = {0.f, 0.f, 0.f, 0.f};
      if (more) write_q(nxt, qn, pieces & 1, sl2n);
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], off);

      // Publish this piece in the scratch format of the merge — per set one row per (kv head, q head):
      // O[128], max, sum; a set that saw no tile publishes (0, -inf, 0) — draw a ticket, and merge
      // the stream if it was the last one.
      if (p.overlap) pdl_wait_prior_grid();   // the scratch is shared with the previous launch
      const int slot_id = first_piece ? 0 : 1;
      float *slot_base = p.fl_part + ((static_cast<size_t>(blockIdx.x) * 2 + slot_id) * kUCWarps + set * kUHS) * 8 * kPartRow;
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
      const int c_first = owner_of(pc.stream_begin + kUCost, total, n_ctas);
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
      if (merger) {
        __threadfence();
        merge_stream<kUCWarps, kUHS, 2, 8, true, false>(p, pc, total, n_ctas, c_first, c_last, warp, lane, g);
        // a stream that lies wholly inside this CTA is published to slot 1 and merged right here; the
        // next piece publishes to slot 1 again, so nobody may run ahead while rows are still being read
        named_bar_sync(1, kUCWarps * 32);
      }
      first_piece = false;
      pc = nxt;
#pragma unroll
      for (int h = 0; h < 4; ++h) sl2h[h] = sl2n[h];
    }
    if (!ok && lane == 0) *failed = 1;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kUCWarps + 2) tmem_dealloc(tmem, kTmemCols);
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
