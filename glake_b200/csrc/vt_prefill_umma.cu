// Causal prefill / prefix-extend attention on the 5th-generation tensor cores:
// tcgen05.mma with operands in shared memory and accumulators in tensor memory.
// Same contract and arithmetic as the mma.sync kernel of vt_prefill.cu (fp32 softmax,
// P applied as hi + lo bf16 halves), needs the per-slot TMA tensor maps.
//
// One CTA per (128-query tile, q head, sequence), six warps:
//   warps 0-3  softmax: thread = query row = TMEM lane.  Reads its row of S with
//              tcgen05.ld (no shuffles: the row's max and sum live in one thread),
//              writes P (hi and lo bf16 halves) back over the same TMEM columns,
//              rescales its row of O in TMEM only when the running maximum grew by more
//              than 2^8 (P then stays <= 256, harmless in fp32), and at the end
//              normalises and stores the row.
//   warp 4     producer: one lane issues the TMA tensor copies of the 64-token K/V
//              tiles (two 32-token boxes per 64-dim half) into a shared-memory ring.
//   warp 5     one lane issues the MMAs: S = Q.K^T (8 steps of K = 16, N = 64) into one of
//              two 64-column S/P buffers, so that the product of tile j+1 runs while the
//              softmax warps work on tile j; O += P_hi.V + P_lo.V (2 x 4 steps, N = 128,
//              P read from TMEM as the A operand, V as the MN-major B operand) into
//              columns [128, 256); tcgen05.commit signals the mbarriers the others wait on.
// Hand-offs (mbarriers, every wait bounded): k/v_full and k/v_empty per ring stage
// (the K slot is released after Q.K^T, the V slot after P.V),
// s_full / p_full per S/P buffer (S ready; P written, 128 arrivals), o_full (P.V of
// a tile done: O may be rescaled), o_last (all of O done).
// Shared memory: Q 32 KB + ring 2 x 32 KB = 96 KB and 256 TMEM columns: two CTAs per SM.
#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_umma.cuh"

namespace vt {
namespace {

constexpr int kUM = 128;                 // query rows per CTA
constexpr int kUN = 64;                  // tokens per K/V tile
constexpr int kUStages = 2;
constexpr int kUThreads = 192;
constexpr int kQSlab = kUM * 128;        // one 64-dim half of Q: [128 rows][128 B]
constexpr int kKVSlab = kUN * 128;       // one 64-dim half of a K (or V) tile: [64 tokens][128 B]
constexpr int kUStage = 4 * kKVSlab;     // K lo, K hi, V lo, V hi
constexpr int kUSmem = 1024 + 2 * kQSlab + kUStages * kUStage + 128;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;   // S/P buffer b at columns [64 b, 64 b + 64): P hi over the first 32, P lo over the rest
constexpr float kRescaleGap = 8.f;       // log2 units

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {      // 2^x, one MUFU op; -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two fp32 lanes per instruction (sm_100 packed fp32 math): halves the FMA / ADD count of the softmax.
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

__global__ void __launch_bounds__(kUThreads, 2) prefill_umma_kernel(PrefillParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, ring_s = q_s + 2 * kQSlab;
  unsigned char *q_g = sm, *ring_g = sm + 2 * kQSlab;
  uint64_t *bars = reinterpret_cast<uint64_t *>(ring_g + kUStages * kUStage);
  // K and V slots of a stage are handed over separately: the K slot is free as soon as Q.K^T of its
  // tile is done, long before P.V releases the V slot, so K of tile j + 2 is fetched ~1.5 tiles ahead.
  const uint32_t k_full = smem_u32(bars), v_full = k_full + 8 * kUStages, k_empty = v_full + 8 * kUStages,
                 v_empty = k_empty + 8 * kUStages, s_full = v_empty + 8 * kUStages, p_full = s_full + 16,
                 o_full = p_full + 16, q_full = o_full + 8, o_last = q_full + 8;
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  // later query tiles see more context: they are scheduled first so that the short ones fill the tail
  const int qt = gridDim.x - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int q_len = p.q_lens[b], seq_len = p.seq_lens[b];
  const int j0 = qt * kUM;
  if (j0 >= q_len) return;                                  // whole CTA: nothing allocated yet
  const int g = p.h / p.kvh, kv_head = hq / g;
  const int pos0 = seq_len - q_len + j0;                    // position of the tile's first query row
  const int kv_end = min(seq_len, pos0 + kUM);              // keys any row of the tile may see
  const int n_tiles = (kv_end + kUN - 1) / kUN;
  if (kv_end <= 0) return;                                  // q_lens > seq_lens: invalid entry, nothing to attend
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // Set-up, overlapped: the producer lane initialises the barriers and at once starts the first K/V
  // copies (nobody else touches a barrier before the CTA-wide sync), warp 5 allocates tensor memory,
  // the softmax warps bring their Q rows into shared memory.
  const int64_t slot = p.slot_ids[b];
  const char *maps = static_cast<const char *>(p.maps) + static_cast<size_t>(slot) * 256;
  // kv = 0: K of tile j, kv = 1: V of tile j (second 32-token box only if it holds context)
  auto load = [&](int j, int kv) -> bool {
    const int s = j % kUStages;
    if (j >= kUStages && !mbar_wait((kv ? v_empty : k_empty) + 8 * s, ((j / kUStages) - 1) & 1)) return false;
    const int t0 = j * kUN;
    const int boxes = (kv_end - t0 > 32) ? 2 : 1;
    const uint32_t dst = ring_s + s * kUStage + kv * 2 * kKVSlab, bar = (kv ? v_full : k_full) + 8 * s;
    const char *map = maps + kv * 128;
    mbar_arrive_expect_tx(bar, static_cast<uint32_t>(boxes) * 2u * 4096u);
    for (int bx = 0; bx < boxes; ++bx) {
      tma_load_3d(dst + bx * 4096, map, 0, kv_head, t0 + 32 * bx, bar);
      tma_load_3d(dst + bx * 4096 + kKVSlab, map, 64, kv_head, t0 + 32 * bx, bar);
    }
    return true;
  };
  const int row = warp * 32 + lane;                         // softmax warps: row of the tile = TMEM lane
  const int jrow = j0 + row;                                // entry-relative query index
  const bool row_ok = jrow < q_len;
  if (warp == 4 && lane == 0) {
    for (int s = 0; s < kUStages; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
    }
    for (int bf = 0; bf < 2; ++bf) {
      mbar_init(s_full + 8 * bf, 1);
      mbar_init(p_full + 8 * bf, kUM);
    }
    mbar_init(o_full, 1);
    mbar_init(o_last, 1);
    mbar_init(q_full, kUM);
    mbar_fence_init();
    failed = 0;
    load(0, 0);                                             // tiles 0 and 1 need no free slot
    if (n_tiles > 1) load(1, 0);
    load(0, 1);
  } else if (warp == 5) {
    tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
    tmem_relinquish();
  } else if (warp < 4) {
    // Q row -> shared memory (zeros beyond q_len), K-major 128-byte swizzle, two 64-dim slabs
    const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.q) +
                                                       (static_cast<int64_t>(p.q_start[b]) + jrow) * p.q_stride + hq * kHeadDim);
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const uint4 v = row_ok ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4 *>(q_g + (c >> 3) * kQSlab + sw128_offset(row, c & 7)) = v;
    }
    fence_proxy_async_smem();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    // ---------------- producer ----------------
    if (lane == 0) {
      // Issue order = the order in which the MMAs free the slots: K(j+1) after Q.K^T(j-1), V(j) after P.V(j-2), ...
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j > 0) ok = load(j, 1);
        if (ok && j + 2 < n_tiles) ok = load(j + 2, 0);
      }
      if (!ok) failed = 1;
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_bf16_f32(kUM, kUN, false, false);
      const uint32_t idesc_pv = umma_idesc_bf16_f32(kUM, kHeadDim, false, true);
      bool ok = mbar_wait(q_full, 0);
      tcgen05_fence_after();
      auto issue_qk = [&](int j) {                          // S of tile j -> buffer j & 1
        const uint32_t st = ring_s + (j % kUStages) * kUStage;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t da = umma_desc_sw128(q_s + (kk >> 2) * kQSlab + (kk & 3) * 32, 0, 1024);
          const uint64_t db = umma_desc_sw128(st + (kk >> 2) * kKVSlab + (kk & 3) * 32, 0, 1024);
          umma_bf16(tmem + kColS + (j & 1) * 64, da, db, idesc_qk, kk > 0);
        }
        umma_commit(k_empty + 8 * (j % kUStages));         // the K slot may be refilled
        umma_commit(s_full + 8 * (j & 1));
      };
      for (int j = 0; ok && j < 2 && j < n_tiles; ++j) {
        ok = mbar_wait(k_full + 8 * (j % kUStages), (j / kUStages) & 1);
        if (ok) {
          tcgen05_fence_after();
          issue_qk(j);
        }
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (!mbar_wait(v_full + 8 * (j % kUStages), (j / kUStages) & 1) || !mbar_wait(p_full + 8 * (j & 1), (j >> 1) & 1)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t st = ring_s + (j % kUStages) * kUStage + 2 * kKVSlab;      // V of this tile
        const uint32_t pa = tmem + kColS + (j & 1) * 64;                           // P hi, then P lo
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = umma_desc_sw128(st + kk * 16 * 128, /*next 64 dims*/ kKVSlab, /*next 8 tokens*/ 1024);
            umma_bf16_ts(tmem + kColO, pa + half * 32 + kk * 8, db, idesc_pv, j > 0 || half > 0 || kk > 0);
          }
        umma_commit(v_empty + 8 * (j % kUStages));        // the V slot may be refilled ...
        umma_commit(o_full);                              // ... and O is quiescent until the next P.V
        if (j == n_tiles - 1) umma_commit(o_last);
        if (j + 2 < n_tiles) {                            // S of tile j + 2 reuses this tile's buffer (after its P.V, in order)
          const int s2 = (j + 2) % kUStages;
          if (!mbar_wait(k_full + 8 * s2, ((j + 2) / kUStages) & 1)) { ok = false; break; }
          tcgen05_fence_after();
          issue_qk(j + 2);
        }
      }
      if (!ok) failed = 1;
    }
  } else {
    // ---------------- softmax warps: thread = query row ----------------
    const int lim = pos0 + row;                             // last visible token
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    mbar_arrive(q_full);                                    // this row of Q was written (and fenced) before the sync
    const float sl2 = p.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t sp = lane_addr + kColS + (j & 1) * 64;   // this tile's S / P buffer
      if (!__all_sync(0xffffffffu, mbar_wait(s_full + 8 * (j & 1), (j >> 1) & 1))) { ok = false; break; }   // warp-uniform: tcgen05.ld follows
      tcgen05_fence_after();
      float x[kUN];
      {                                                     // both halves of the row in flight before the one wait
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(sp, v0);
        tmem_ld_32x32b_x32(sp + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {                      // raw logits; the scale rides in the exponent's FMA
          x[i] = __uint_as_float(v0[i]);
          x[32 + i] = __uint_as_float(v1[i]);
        }
      }
      const int t0 = j * kUN;
      float mx = -INFINITY;
      if (t0 + kUN - 1 > lim) {
#pragma unroll
        for (int i = 0; i < kUN; ++i) x[i] = (t0 + i <= lim) ? x[i] : -INFINITY;
      }
#pragma unroll
      for (int i = 0; i < kUN; i += 2) mx = max3(mx, x[i], x[i + 1]);
      mx *= sl2;                                            // scale > 0 (checked by the launcher): max commutes with it
      // tcgen05.ld / .st are warp-wide instructions: the decision to rescale is taken per warp,
      // every lane then moves its reference to max(old, tile) (a factor of 1 where nothing changed).
      if (__any_sync(0xffffffffu, mx > m_ref + kRescaleGap || (m_ref == -INFINITY && mx != -INFINITY))) {
        const float m_new = fmaxf(m_ref, mx);
        const float f = m_ref == -INFINITY ? 1.f : exp2f(m_ref - m_new);      // O is still empty while m_ref is -inf
        l *= f;
        if (j > 0) {
          // O must be quiescent: P.V of the previous tile done (P.V of this one waits for this thread's P)
          if (!__all_sync(0xffffffffu, mbar_wait(o_full, (j - 1) & 1))) { ok = false; break; }
          tcgen05_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(lane_addr + kColO + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tmem_st_32x32b_x32(lane_addr + kColO + c0, v);
          }
          tmem_st_wait();
        }
        m_ref = m_new;
      }
      const float ref = m_ref == -INFINITY ? 0.f : m_ref;    // nothing visible yet: every x is -inf, every p is 0
      if (kv_end - t0 < kUN) {
        // Ragged last tile: V rows past the context may hold anything (0 * NaN = NaN).  The rows of
        // this thread's share are cleared in both 64-dim halves before the tensor core reads them.
        if (!__all_sync(0xffffffffu, mbar_wait(v_full + 8 * (j % kUStages), (j / kUStages) & 1))) { ok = false; break; }
        unsigned char *vst = ring_g + (j % kUStages) * kUStage + 2 * kKVSlab;
        for (int r = (kv_end - t0) + (row >> 4); r < kUN; r += 8)
          *reinterpret_cast<uint4 *>(vst + ((row >> 3) & 1) * kKVSlab + r * 128 + (row & 7) * 16) = make_uint4(0, 0, 0, 0);
      }
      {                                                     // P hi -> columns [0, 32), P lo -> [32, 64) of the buffer
        uint32_t hi[32], lo[32];
        const uint64_t sl2_2 = f2_pack(sl2, sl2), nref2 = f2_pack(-ref, -ref), minus1 = f2_pack(-1.f, -1.f);
        uint64_t l2 = f2_pack(l, 0.f);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float a0, a1;
          f2_unpack(f2_fma(f2_pack(x[2 * i], x[2 * i + 1]), sl2_2, nref2), a0, a1);
          const float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
          const uint64_t p2 = f2_pack(p0, p1);
          l2 = f2_add(l2, p2);
          hi[i] = pack_bf16x2(p0, p1);
          float r0, r1;
          f2_unpack(f2_fma(f2_pack(bf16_lo(hi[i]), bf16_hi(hi[i])), minus1, p2), r0, r1);   // p - hi, exact
          lo[i] = pack_bf16x2(r0, r1);
        }
        {
          float la, lb;
          f2_unpack(l2, la, lb);
          l = la + lb;
        }
        tmem_st_32x32b_x32(sp, hi);
        tmem_st_32x32b_x32(sp + 32, lo);
        tmem_st_wait();
      }
      fence_proxy_async_smem();        // the cleared V rows of a ragged tile
      tcgen05_fence_before();
      mbar_arrive(p_full + 8 * (j & 1));
    }
    // Not o_full: these threads do not follow its phases tile by tile, and a parity wait can only
    // tell the latest completed phase from the one before it.  o_last completes exactly once.
    if (ok && !__all_sync(0xffffffffu, mbar_wait(o_last, 0))) ok = false;
    tcgen05_fence_after();
    if (__all_sync(0xffffffffu, ok)) {                      // warp-wide TMEM loads; only the stores are per row
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(p.out) +
                                             (static_cast<int64_t>(p.q_start[b]) + jrow) * p.out_stride + hq * kHeadDim);
#pragma unroll
      for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + kColO + c0, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[c0 / 8 + i] = make_uint4(pack_bf16x2(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv),
                                         pack_bf16x2(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv),
                                         pack_bf16x2(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv),
                                         pack_bf16x2(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv));
        }
      }
    }
    if (!ok) failed = 1;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, kTmemCols);
  if (tid == 0 && failed && p.status) atomicExch(p.status, kKernelErrMagic);
}

}  // namespace

int launch_prefill_umma(const PrefillParams &p, int max_q_len, cudaStream_t stream) {
  static SmemOptIn opt_in;
  if (!opt_in.ensure(prefill_umma_kernel, kUSmem)) return VT_ERR_CUDA;
  dim3 grid((max_q_len + kUM - 1) / kUM, p.h, p.batch);
  prefill_umma_kernel<<<grid, kUThreads, kUSmem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

}  // namespace vt
