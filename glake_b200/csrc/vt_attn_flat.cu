// Single-query decode attention, persistent "flat" schedule on the tensor-core
// tile engine of vt_attn_mma.cu (same shared-memory geometry, same per-warp math).
//
// Why: with one CTA per (sequence, token partition) every CTA pays a pipeline
// fill, ragged context lengths leave a tail wave, and a second kernel merges the
// partitions.  Here the whole batch is one list of tiles (16 groups of 1 KiB of
// K and of V): stream (sequence b, kv-head slab) contributes
// ceil(L_b / tile_tokens) tiles, streams are laid end to end, and CTA c of N
// takes tiles [c*T/N, (c+1)*T/N).  N = 2 x SM count CTAs are all resident, each
// moves the same number of bytes, and its copy ring never drains: the producer
// warp simply keeps issuing bulk copies across stream boundaries.
//
// A maximal run of a CTA's tiles inside one stream is a "piece".  A piece that
// covers its whole stream is final.  Otherwise the CTA writes the piece's
// unnormalised state (O[128], running max, running sum per q head and consumer
// warp) to scratch and takes a ticket on the stream's counter; whoever draws the
// last ticket merges all pieces of the stream and writes the output.  Nobody
// waits for anybody, so the kernel cannot hang on a missing peer.  A CTA has at
// most two non-final pieces (its first and its last), hence two scratch slots
// per CTA regardless of context length.
//
// Fused step: when the call carries this step's new K/V rows, the kernel is the
// append as well.  The producer fetches the newest token's row from the input
// tensors instead of the cache (so nothing depends on a prior append kernel), and
// the consumer warp that holds that row in shared memory stores it to the range.
//
// Overlap with the previous step (opt-in): consecutive layers' launches touch
// disjoint ranges, so with programmatic dependent launch a CTA of the next layer
// may take an SM slot as soon as a CTA of this layer exits, and stream its K/V
// while this layer's stragglers and mergers finish.  The only thing the two grids
// share is the scratch buffer; a dependent grid executes griddepcontrol.wait
// before its first access to it.
//
// Roofline: HBM.  Algorithmic bytes per (sequence, kv head): L * 2 * 128 * 2.
#include <algorithm>

#include "../../include/vtensor.h"
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_mma.cuh"
#include "vt_mma_f8.cuh"
#include "vt_attn_flat_sched.cuh"

namespace vt {
namespace {

// Ring depth and residency per engine.  The bf16 engine with one 8-head block runs
// 3 CTAs per SM on 2-stage rings (66 KB, <= 128 registers): with more, shorter-lived
// CTAs the launches of consecutive layers interleave better (measured +5..7 % on the
// decode step); the wider variants keep 3 stages and 2 CTAs per SM (their merge
// buffers and register files need the room).
template <template <int> class W, int NB>
struct FlatCfg {
  static constexpr bool kSmall = W<NB>::kWarps == 4 && NB == 1;
  static constexpr int kStages = kSmall ? 2 : 3;
  static constexpr int kCtasPerSm = kSmall ? 3 : 2;
  static constexpr int kRing = kStages * kStageB;
};

constexpr int kBaseCacheMaxBatch = 256;   // per-sequence base addresses are cached in shared memory up to here

// ring | barriers | flags | prefix[batch + 1] | lens[batch] | (pad to 8) | kbase[batch] | vbase[batch]
__host__ __device__ constexpr int flat_meta_ints(int batch) { return ((2 * batch + 1 + 4) + 1) / 2 * 2; }
__host__ __device__ constexpr int flat_smem_bytes(int batch, int stages) {
  return stages * kStageB + 2 * stages * 8 + flat_meta_ints(batch) * 4 +
         (batch <= kBaseCacheMaxBatch ? batch * 16 : 0);
}

// SM count of the current device, cached.
int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// W = per-warp engine (WarpAttn: bf16 cache, 4 consumer warps; WarpAttnF8: fp8 e4m3
// cache, 8 consumer warps), NB = 8-head blocks per kv head, HS = kv heads per CTA,
// R = consecutive tokens per 1 KiB bulk copy; HS * R = consumer warps.
template <template <int> class W, int NB, int HS, int R>
__global__ void __launch_bounds__((W<NB>::kWarps + 1) * 32, NB == 1 ? FlatCfg<W, NB>::kCtasPerSm : 1)
attn_flat_kernel(AttnParams p) {
  constexpr int kCWarps = W<NB>::kWarps;
  constexpr int kThreads = (kCWarps + 1) * 32;
  constexpr int kStages = FlatCfg<W, NB>::kStages;
  constexpr int kRing = FlatCfg<W, NB>::kRing;
  constexpr int kRowB = W<NB>::kRowBytes;
  constexpr bool kFp8 = kRowB == 128;
  static_assert(HS * R == kCWarps, "one consumer warp per (kv head, row of a group)");
  static_assert(kCWarps * kRowB == kGroupB, "a group is 1 KiB");
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TILE_TOK = kGroupsPerTile * R;
  constexpr int HEADS = NB * 8;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kRing);
  int *flags = reinterpret_cast<int *>(smem + kRing + 2 * kStages * 8);   // [0] = "this CTA merges"
  int *prefix = flags + 4;                                                // [batch + 1]
  int *lens = prefix + p.batch + 1;                                       // [batch] context lengths
  const bool cache_bases = p.batch <= kBaseCacheMaxBatch;
  unsigned long long *kbase_s = reinterpret_cast<unsigned long long *>(flags + flat_meta_ints(p.batch));
  unsigned long long *vbase_s = kbase_s + p.batch;                        // [batch] each, only if cache_bases
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t ring0 = smem_u32(smem);

  const int g = p.h / p.kvh;
  const int slabs = p.kvh / HS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kCWarps);
    }
    mbar_fence_init();
  }
  // tiles per sequence, then an exclusive prefix (batch is small: one warp scans it)
  for (int i = threadIdx.x; i < p.batch; i += kThreads) {
    const int len = max(p.seq_lens[i], 0);
    lens[i] = len;
    prefix[i + 1] = len > 0 ? ((len + TILE_TOK - 1) / TILE_TOK + kBoundaryCost) * slabs : 0;
    if (cache_bases) {   // resolve slot -> range base once, off the producer's critical path
      const int64_t slot = p.slot_ids[i];
      kbase_s[i] = p.k_table[slot];
      vbase_s[i] = p.v_table[slot];
    }
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < p.batch; base += 32) {
      const int i = base + lane;
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
  pdl_launch_dependents();   // the next launch may be scheduled as CTAs of this grid exit
  const long long total = prefix[p.batch];
  // Only min(grid, total) CTAs take part, so that every participating CTA owns at
  // least one tile and the piece count of a stream is a plain difference.
  const int n_ctas = static_cast<int>(min(static_cast<long long>(gridDim.x), total));
  const bool active = static_cast<int>(blockIdx.x) < n_ctas;
  const long long tau0 = active ? total * blockIdx.x / n_ctas : 0;
  const long long tau1 = active ? total * (blockIdx.x + 1) / n_ctas : 0;

  if (warp == kCWarps) {
    // ---------------- producer warp ----------------
    // lanes 0..15 fetch the K groups of a tile, lanes 16..31 the V groups
    const int grp = lane & 15;
    const uint32_t dst_lane = (lane < 16 ? 0 : kTileB) + grp * kPitch;
    const size_t tok_pitch = static_cast<size_t>(p.kvh) * kRowB;
    const uint64_t policy = l2_policy_evict_first();
    int it = 0;  // tiles issued by this CTA: ring position and barrier phase
    for (long long tau = tau0; tau < tau1;) {
      const Piece pc = locate(prefix, p.batch, slabs, tau, tau1);
      const int seq_len = lens[pc.b];
      unsigned long long range;
      if (cache_bases) {
        range = lane < 16 ? kbase_s[pc.b] : vbase_s[pc.b];
      } else {
        const int64_t slot = p.slot_ids[pc.b];
        range = lane < 16 ? p.k_table[slot] : p.v_table[slot];
      }
      const char *base = reinterpret_cast<const char *>(range) + static_cast<size_t>(pc.slab) * HS * kRowB;
      const char *fresh = nullptr;   // this step's row of the slab, when the call is a fused step
      if (p.new_key && p.byte_off[pc.b] >= 0)
        fresh = (lane < 16 ? static_cast<const char *>(p.new_key) + pc.b * p.new_key_stride * 2
                           : static_cast<const char *>(p.new_value) + pc.b * p.new_value_stride * 2) +
                static_cast<size_t>(pc.slab) * HS * kRowB;
      for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
        const int s = it % kStages;
        if (it >= kStages && !mbar_wait(empty0 + 8 * s, ((it / kStages) - 1) & 1)) {
          if (lane == 0) atomicExch(p.status, kKernelErrMagic);
          return;
        }
        const int t0 = tile * TILE_TOK;
        const int nt = min(TILE_TOK, seq_len - t0);
        // fp8 fused step: the newest token's row is quantised into the stage by the consumer
        // warp that owns it, so this tile's copies bring one row less of K and of V
        const int nt_copied = nt - ((kFp8 && fresh && t0 + nt == seq_len) ? 1 : 0);
        if (lane == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2u * nt_copied * HS * kRowB);
        __syncwarp();
        int rows = min(R, nt - grp * R);   // valid token rows of this lane's group
        if (rows > 0) {
          const uint32_t dst = ring0 + s * kStageB + dst_lane;
          if (fresh && t0 + grp * R + rows == seq_len) {
            // the newest token comes straight from this step's input row
            --rows;
            if (p.overlap == 2) pdl_wait_prior_grid();   // ... which the preceding kernel may still be writing
            if (!kFp8) bulk_g2s(dst + rows * HS * kRowB, fresh, HS * kRowB, full0 + 8 * s);
          }
          if (rows > 0)
            bulk_g2s_hint(dst, base + static_cast<size_t>(t0 + grp * R) * tok_pitch, rows * HS * kRowB,
                          full0 + 8 * s, policy);
        }
      }
      tau += pc.advance;
    }
    return;
  }

  // ---------------- consumer warps ----------------
  const int hs = warp % HS, rr = warp / HS;      // kv head within the slab, row within each group
  const uint32_t row_off = (rr * HS + hs) * kRowB;
  const uint32_t k_off = k_lane_offset(lane, row_off), v_off = v_lane_offset(lane, row_off);
  const float sl2_base = p.scale * 1.4426950408889634f;
  const int tid = threadIdx.x;  // 0 .. kCWarps * 32 - 1
  __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);

  // Sequences without context produce zeros; nobody owns a tile of theirs.
  if (blockIdx.x == 0) {
    for (int b = 0; b < p.batch; ++b)
      if (prefix[b + 1] == prefix[b]) {
        for (int i = tid; i < p.h * kHeadDim; i += kCWarps * 32) out[b * p.out_stride + i] = __float2bfloat16(0.f);
        if (p.lse && tid < p.h) p.lse[b * p.h + tid] = -INFINITY;
      }
  }

  // A wait that runs out marks the warp as failed; it then skips the remaining
  // tiles but still walks through every piece and every barrier below, so the
  // other consumer warps are never left waiting for it.
  bool failed = false;
  int it = 0;
  bool first_piece = true;
  for (long long tau = tau0; tau < tau1;) {
    const Piece pc = locate(prefix, p.batch, slabs, tau, tau1);
    if (pc.tile_end <= pc.tile_begin) {   // only phantom positions of this stream fall into the share
      tau += pc.advance;
      continue;
    }
    const int seq_len = lens[pc.b];
    const int kv_head = pc.slab * HS + hs;
    long long append_off = -1;
    char *append_k = nullptr, *append_v = nullptr;
    if (p.new_key) {
      append_off = p.byte_off[pc.b];
      if (cache_bases) {
        append_k = reinterpret_cast<char *>(kbase_s[pc.b]);
        append_v = reinterpret_cast<char *>(vbase_s[pc.b]);
      } else {
        const int64_t slot = p.slot_ids[pc.b];
        append_k = reinterpret_cast<char *>(p.k_table[slot]);
        append_v = reinterpret_cast<char *>(p.v_table[slot]);
      }
    }
    const float sl2 = kFp8 ? sl2_base * p.k_scale[kv_head] : sl2_base;   // fp8: K's scale folded into the logits
    W<NB> st;
    if (p.overlap == 2) pdl_wait_prior_grid();   // q (and the new rows) may be the preceding kernel's output
    st.start(static_cast<const __nv_bfloat16 *>(p.q) + pc.b * p.q_stride + kv_head * g * kHeadDim, g, lane);
    for (int tile = pc.tile_begin; tile < pc.tile_end; ++tile, ++it) {
      const int s = it % kStages;
      if (!failed && !mbar_wait(full0 + 8 * s, (it / kStages) & 1)) failed = true;
      if (failed) continue;
      const int tok0 = tile * TILE_TOK + rr;      // token of fragment row 0
      const int n_rows = min(16, (seq_len - tok0 + R - 1) / R);
      const bool newest_here = append_off >= 0 && (seq_len - 1 - tok0) % R == 0 && seq_len - 1 >= tok0 &&
                               seq_len - 1 < (tile + 1) * TILE_TOK;
      if (newest_here) {
        // Fused step: this warp owns the newest token's row of its kv head; make it part of the cache.
        unsigned char *row = smem + s * kStageB + ((seq_len - 1 - tok0) / R) * kPitch + row_off;
        const size_t dst = static_cast<size_t>(append_off) + static_cast<size_t>(kv_head) * kRowB;
        if constexpr (!kFp8) {
          // the producer fetched it from the step's inputs: 8 bytes per lane for K and for V
          *reinterpret_cast<uint2 *>(append_k + dst + lane * 8) = *reinterpret_cast<const uint2 *>(row + lane * 8);
          *reinterpret_cast<uint2 *>(append_v + dst + lane * 8) = *reinterpret_cast<const uint2 *>(row + kTileB + lane * 8);
        } else {
          // quantise it here (4 elements per lane; true division, as the append kernel does, so the
          // bytes equal sat(x / scale) exactly), into the stage for this step and into the range for good
          const uint2 kx = __ldg(reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(p.new_key) +
                                                                 pc.b * p.new_key_stride + kv_head * kHeadDim) + lane);
          const uint2 vx = __ldg(reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(p.new_value) +
                                                                 pc.b * p.new_value_stride + kv_head * kHeadDim) + lane);
          const float ks = p.k_scale[kv_head], vs = p.v_scale[kv_head];
          const uint32_t kq = float2_to_e4m3x2(bf16_lo(kx.x) / ks, bf16_hi(kx.x) / ks) |
                              (float2_to_e4m3x2(bf16_lo(kx.y) / ks, bf16_hi(kx.y) / ks) << 16);
          const uint32_t vq = float2_to_e4m3x2(bf16_lo(vx.x) / vs, bf16_hi(vx.x) / vs) |
                              (float2_to_e4m3x2(bf16_lo(vx.y) / vs, bf16_hi(vx.y) / vs) << 16);
          *reinterpret_cast<uint32_t *>(row + lane * 4) = kq;
          *reinterpret_cast<uint32_t *>(row + kTileB + lane * 4) = vq;
          *reinterpret_cast<uint32_t *>(append_k + dst + lane * 4) = kq;
          *reinterpret_cast<uint32_t *>(append_v + dst + lane * 4) = vq;
          __syncwarp();
        }
      }
      if (tok0 < seq_len) st.tile(ring0 + s * kStageB, smem + s * kStageB, k_off, v_off, row_off, n_rows, sl2, lane);
      // this warp's own stores into the stage (zeroed rows of a ragged tile, a quantised new row)
      // must be ordered before the copy engine refills the stage
      if (n_rows < 16 || (kFp8 && newest_here)) fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
    st.finish_sums();

    const bool whole = pc.tile_begin == 0 && pc.tile_end == pc.tiles_in_stream;
    if (R == 1 && whole) {
      // This warp saw every token of its kv head: write the result from registers.
      const int r4 = lane >> 2, c4 = lane & 3;
      const float vs = kFp8 ? p.v_scale[kv_head] : 1.0f;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int head = nb * 8 + 2 * c4 + e;
          if (head < g) {
            const float inv = vs / st.lrun[nb][e];   // sum > 0: a stream holds at least one token
            const int hq = kv_head * g + head;
            __nv_bfloat16 *dst = out + pc.b * p.out_stride + hq * kHeadDim;
#pragma unroll
            for (int mb = 0; mb < 8; ++mb) {
              dst[W<NB>::dim_of(mb, 0, r4)] = __float2bfloat16(st.o[nb][mb][e] * inv);
              dst[W<NB>::dim_of(mb, 1, r4)] = __float2bfloat16(st.o[nb][mb][2 + e] * inv);
            }
            if (p.lse && r4 == 0)
              p.lse[pc.b * p.h + hq] = (st.mrun[nb][e] + log2f(st.lrun[nb][e])) * 0.6931471805599453f;
          }
        }
      }
    } else {
      // Publish this piece, draw a ticket, and merge the stream if it was the last one.
      // The scratch is shared with the previous launch: a dependent grid must see
      // that one finished (mergers done reading, counters back to zero) first.
      if (p.overlap) pdl_wait_prior_grid();
      const int slot_id = first_piece ? 0 : 1;
      float *slot_base = p.fl_part + (static_cast<size_t>(blockIdx.x) * 2 + slot_id) * kCWarps * HEADS * kPartRow;
      // the CTA's last piece: whatever is left of the share after this stream is phantom
      const bool last_of_cta = tau1 <= pc.stream_end + kBoundaryCost;
      if (R > 1 && last_of_cta) {
        // The ring is idle after the CTA's last tile: fold the R warps of every kv
        // head together in shared memory first, so the piece publishes one state
        // per head instead of R (fewer bytes out, fewer sources for the merger).
        named_bar_sync(1, kCWarps * 32);                       // all warps are done with the ring
        float *mbuf = reinterpret_cast<float *>(smem);          // [kCWarps][HEADS][kPartRow]
        st.template store<kPartRow>(mbuf + warp * HEADS * kPartRow, lane, g);
        named_bar_sync(1, kCWarps * 32);
        // thread -> (head pair index, output dim): 128 dims x (consumer threads / 128) pairs at a time
        for (int pair = tid >> 7; pair < HS * g; pair += kCWarps * 32 / 128) {
          const int hh = pair / g, head = pair % g, d = tid & 127;
          float M = -INFINITY;
#pragma unroll
          for (int r = 0; r < R; ++r) M = fmaxf(M, mbuf[((r * HS + hh) * HEADS + head) * kPartRow + 128]);
          float L = 0.f, O = 0.f;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float *src = mbuf + ((r * HS + hh) * HEADS + head) * kPartRow;
            const float f = exp2f(src[128] - M);   // M is finite: row 0 of the piece's first tile is valid
            L = fmaf(f, src[129], L);
            O = fmaf(f, src[d], O);
          }
          float *dst = slot_base + (hh * HEADS + head) * kPartRow;
          dst[d] = O;
          if (d == 0) { dst[128] = M; dst[129] = L; }
        }
      } else {
        st.template store<kPartRow>(slot_base + warp * HEADS * kPartRow, lane, g);
      }
      __threadfence();
      named_bar_sync(1, kCWarps * 32);
      // pieces of the stream = CTAs whose shares hold real tiles of it
      const long long s_begin = pc.stream_begin, s_end = pc.stream_end;
      const int c_first = owner_of(s_begin + kBoundaryCost, total, n_ctas), c_last = owner_of(s_end - 1, total, n_ctas);
      const int n_pieces = c_last - c_first + 1;
      if (tid == 0) {
        unsigned *ctr = p.fl_count + pc.b * slabs + pc.slab;
        const unsigned old = atomicAdd(ctr, 1u);
        const int last = old + 1 == static_cast<unsigned>(n_pieces);
        if (last) *ctr = 0u;   // leaves the counters clean for the next launch
        flags[0] = last;
      }
      named_bar_sync(1, kCWarps * 32);
      const bool merger = flags[0] != 0;
      named_bar_sync(1, kCWarps * 32);   // flags[0] may be rewritten by the next piece
      if (merger) {
        merge_stream<kCWarps, HS, R, HEADS, kFp8>(p, pc, total, n_ctas, c_first, c_last, warp, lane, g);
        // With R > 1 a stream that lies wholly inside this CTA is published to slot 1 and
        // merged right here; the next piece publishes to slot 1 again.  No warp may start
        // that store while another still reads this piece's rows (a warp without merge
        // items would otherwise run ahead through a short piece).
        if (R > 1) named_bar_sync(1, kCWarps * 32);
      }
    }
    first_piece = false;
    tau += pc.advance;
  }
  if (failed && lane == 0) atomicExch(p.status, kKernelErrMagic);
}

template <template <int> class W, int NB, int HS, int R>
int launch(const AttnParams &p_in, cudaStream_t stream) {
  constexpr int kThreads = (W<NB>::kWarps + 1) * 32;
  AttnParams p = p_in;
  p.n_ctas = FlatCfg<W, NB>::kCtasPerSm * std::min(sm_count(), kFlatSms);
  const int smem = flat_smem_bytes(p.batch, FlatCfg<W, NB>::kStages);
  static SmemOptIn opt_in;
  if (!opt_in.ensure(attn_flat_kernel<W, NB, HS, R>, smem)) return VT_ERR_CUDA;
  if (p.overlap) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, attn_flat_kernel<W, NB, HS, R>, p) == cudaSuccess ? VT_OK : VT_ERR_CUDA;
  }
  attn_flat_kernel<W, NB, HS, R><<<p.n_ctas, kThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

template <int NB>
int launch_bf16(const AttnParams &p, cudaStream_t stream) {
  if (p.kvh % 4 == 0) return launch<WarpAttn, NB, 4, 1>(p, stream);
  if (p.kvh == 2) return launch<WarpAttn, NB, 2, 2>(p, stream);
  if (p.kvh == 1) return launch<WarpAttn, NB, 1, 4>(p, stream);
  return VT_ERR_UNSUPPORTED;
}

template <int NB>
int launch_fp8(const AttnParams &p, cudaStream_t stream) {
  if (p.kvh % 8 == 0) return launch<WarpAttnF8, NB, 8, 1>(p, stream);
  if (p.kvh == 4) return launch<WarpAttnF8, NB, 4, 2>(p, stream);
  if (p.kvh == 2) return launch<WarpAttnF8, NB, 2, 4>(p, stream);
  if (p.kvh == 1) return launch<WarpAttnF8, NB, 1, 8>(p, stream);
  return VT_ERR_UNSUPPORTED;
}

}  // namespace

bool attn_flat_supports(int batch, int h, int kvh, int kv_dtype) {
  const int g = h / kvh;
  if (batch > kFlatMaxBatch || !(g <= 8 || g == 16)) return false;
  if (kv_dtype == VT_KV_BF16) return kvh % 4 == 0 || kvh == 2 || kvh == 1;
  if (kv_dtype == VT_KV_FP8_E4M3) return kvh % 8 == 0 || kvh == 4 || kvh == 2 || kvh == 1;
  return false;
}

int flat_consumer_warps(int kv_dtype) { return kv_dtype == VT_KV_FP8_E4M3 ? 8 : 4; }

// Largest grid launch() uses for this problem: the scratch holds two piece slots per CTA.
int flat_max_ctas(int h, int kvh, int kv_dtype) {
  const bool nb1 = (h / kvh) <= 8;
  const int per_sm = kv_dtype == VT_KV_FP8_E4M3 ? (nb1 ? FlatCfg<WarpAttnF8, 1>::kCtasPerSm : FlatCfg<WarpAttnF8, 2>::kCtasPerSm)
                                                : (nb1 ? FlatCfg<WarpAttn, 1>::kCtasPerSm : FlatCfg<WarpAttn, 2>::kCtasPerSm);
  return per_sm * kFlatSms;
}

int launch_attn_flat(const AttnParams &p, int kv_dtype, cudaStream_t stream) {
  if (!attn_flat_supports(p.batch, p.h, p.kvh, kv_dtype)) return VT_ERR_UNSUPPORTED;
  const bool nb1 = (p.h / p.kvh) <= 8;
  if (kv_dtype == VT_KV_FP8_E4M3) return nb1 ? launch_fp8<1>(p, stream) : launch_fp8<2>(p, stream);
  return nb1 ? launch_bf16<1>(p, stream) : launch_bf16<2>(p, stream);
}

}  // namespace vt
