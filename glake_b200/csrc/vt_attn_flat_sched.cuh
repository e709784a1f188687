// Scheduling pieces shared by the persistent ("flat") decode attention kernels: how the
// tile list is cut into per-CTA shares, and how the last CTA of a stream merges the
// published piece states.  The engines differ (mma.sync per warp, or tcgen05 per CTA);
// the schedule and the scratch format do not.
#pragma once
#include "vt_device.cuh"
#include "vt_kernels.h"
#include "vt_mma.cuh"

namespace vt {
namespace {

constexpr int kPartRow = kFlatPartRow;   // floats per published (q head, warp) state: O[128], max, sum, pad

// The tile list is cut evenly in COST units, not in tiles: every stream is preceded by
// kBoundaryCost phantom positions that carry no data.  A CTA whose share crosses from one
// stream into the next stops computing for a while (publish the piece, fence, ticket,
// possibly merge, load the next Q): measured 4.4 us against 1.4 us per 32 KB tile, and the
// CTAs with such a crossing were the last to finish by that margin.  With the phantom
// positions inside its share, a crossing CTA gets that many fewer real tiles.
constexpr int kBoundaryCost = 3;

struct Piece {
  int b, slab, tile_begin, tile_end, tiles_in_stream;   // real tiles [tile_begin, tile_end) of the stream (may be empty)
  long long stream_begin;  // position of the stream's first phantom position
  long long stream_end;    // position after the stream's last tile
  int advance;             // positions of the share this piece uses up
};

// Locates the stream holding position `tau` and the run of tiles this CTA owns inside
// it.  prefix[b] = position of sequence b's first stream.
template <int kCost = kBoundaryCost>
__device__ __forceinline__ Piece locate(const int *prefix, int batch, int slabs, long long tau, long long tau_end) {
  int lo = 0, hi = batch;  // largest b with prefix[b] <= tau
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= tau) lo = mid; else hi = mid;
  }
  Piece pc;
  pc.b = lo;
  const int per_slab = (prefix[lo + 1] - prefix[lo]) / slabs;      // phantom positions + tiles
  const int rem = static_cast<int>(tau - prefix[lo]);
  pc.slab = rem / per_slab;
  const int pos = rem % per_slab;
  pc.tiles_in_stream = per_slab - kCost;
  pc.stream_begin = prefix[lo] + static_cast<long long>(pc.slab) * per_slab;
  pc.stream_end = pc.stream_begin + per_slab;
  const int end = static_cast<int>(min(static_cast<long long>(per_slab), pos + (tau_end - tau)));
  pc.advance = end - pos;
  pc.tile_begin = max(pos - kCost, 0);
  pc.tile_end = max(end - kCost, 0);
  return pc;
}

// CTA that owns global tile tau when CTA c starts at floor(c * T / N).
__device__ __forceinline__ int owner_of(long long tau, long long total, int n_ctas) {
  return static_cast<int>(((tau + 1) * n_ctas - 1) / total);
}

// Merge of one stream by the CTA that drew its last ticket.  The caller has published its
// own piece and passed a CTA-wide barrier; every consumer warp of the CTA calls this.
// kCWarps / HS / R / HEADS describe the scratch layout ([cta][2 slots][kCWarps][HEADS] rows;
// consumer warp r * HS + hh holds kv head hh of the slab), kFp8 applies the V scale.
// kFold: pieces that were their CTA's last piece were folded to one row per head before they
// were published (the mma.sync kernel does that in its idle ring); without it every piece
// arrives as R rows per head.
template <int kCWarps, int HS, int R, int HEADS, bool kFp8, bool kFold = true>
__device__ __forceinline__ void merge_stream(const AttnParams &p, const Piece &pc, long long total, int n_ctas,
                                             int c_first, int c_last, int warp, int lane, int g) {
  const long long s_begin = pc.stream_begin, s_end = pc.stream_end;
  const int n_pieces = c_last - c_first + 1;
  __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
  __threadfence();
  // Sources of one q head: (piece c, consumer warp r * HS + hh).  Heads are
  // dealt round-robin to the four warps; inside a warp lane i first fetches
  // (max, sum) of source i, the warp agrees on the stream maximum, then every
  // lane accumulates its 4 output dims over the sources with independent
  // 16-byte loads.  Streams cut into more than 32 sources go in rounds.
  // Pieces that were their CTA's last piece arrive folded (one row per head):
  // that is every piece but, possibly, the one in the stream's last CTA.
  const bool last_folded = R == 1 || total * (c_last + 1) / n_ctas <= s_end + kBoundaryCost;
  const int n_single = !kFold ? 0 : last_folded ? n_pieces : n_pieces - 1;
  const int n_src = R == 1 ? n_pieces : !kFold ? n_pieces * R : n_single + (last_folded ? 0 : R);
  for (int item = warp; item < HS * g; item += kCWarps) {
    const int hh = item / g, head = item % g;
    const float vsc = kFp8 ? __ldg(p.v_scale + pc.slab * HS + hh) : 1.0f;   // in flight with the sources, not after them
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < n_src; s0 += 32) {
      const int i = s0 + lane;
      const float *mine = nullptr;
      float mi = -INFINITY, li = 0.f;
      if (i < n_src) {
        const int c = !kFold ? c_first + i / R : i < n_single ? c_first + i : c_last;
        const int r = !kFold ? i % R : i < n_single ? 0 : i - n_single;
        // the stream is CTA c's first piece iff it already runs at c's first tile
        const int sl = (s_begin <= total * c / n_ctas) ? 0 : 1;
        mine = p.fl_part + (((static_cast<size_t>(c) * 2 + sl) * kCWarps + r * HS + hh) * HEADS + head) * kPartRow;
        mi = __ldcg(mine + 128);
        li = __ldcg(mine + 129);
      }
      // Eight independent 16-byte loads in flight per lane; absent sources carry
      // weight 0 and re-read the lane's own row (or source 0's), never garbage.  The
      // first eight go out together with the (max, sum) loads above: their addresses
      // need no data, only the weights do, so a stream cut into up to eight sources
      // is merged in ONE round trip to L2.
      const unsigned long long mine_bits = reinterpret_cast<unsigned long long>(mine);
      const unsigned long long any_bits = __shfl_sync(0xffffffffu, mine_bits, 0);
      const int cnt = min(32, n_src - s0);
      auto fetch = [&](int j0, float4 (&v)[8]) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          unsigned long long bits = __shfl_sync(0xffffffffu, mine_bits, min(j0 + u, 31));
          if (bits == 0ull) bits = any_bits;
          v[u] = __ldcg(reinterpret_cast<const float4 *>(bits) + lane);
        }
      };
      float4 v[8];
      fetch(0, v);
      float mx = mi;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float Mn = fmaxf(M, mx);
      const float rescale = exp2f(M - Mn);   // 0 on the first round (M = -inf)
      const float fi = i < n_src ? exp2f(mi - Mn) : 0.f;
      float ls = fi * li;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, off);
      L = L * rescale + ls;
      acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
      M = Mn;
      for (int j0 = 0; j0 < cnt; j0 += 8) {
        if (j0 > 0) fetch(j0, v);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float w = j0 + u < cnt ? __shfl_sync(0xffffffffu, fi, min(j0 + u, 31)) : 0.f;
          acc.x = fmaf(w, v[u].x, acc.x); acc.y = fmaf(w, v[u].y, acc.y);
          acc.z = fmaf(w, v[u].z, acc.z); acc.w = fmaf(w, v[u].w, acc.w);
        }
      }
    }
    const int hq = (pc.slab * HS + hh) * g + head;
    const float inv = vsc / L;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2 *>(out + pc.b * p.out_stride + hq * kHeadDim + lane * 4) = packed;
    if (p.lse && lane == 0) p.lse[pc.b * p.h + hq] = (M + log2f(L)) * 0.6931471805599453f;
  }
}

}  // namespace
}  // namespace vt
