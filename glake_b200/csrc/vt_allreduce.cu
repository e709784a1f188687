// Low-latency sum all-reduce of small bf16 messages over NVLink peer memory: the
// model-level reduction after o_proj / down_proj of a tensor-parallel layer, for
// messages too small for a bandwidth-optimised collective to get going.
//
// Every rank owns one buffer that all ranks have mapped (CUDA IPC or any other
// peer mapping): two flag arrays, two staging copies of the message and two result
// copies (double-buffered by call parity).  One kernel launch per call, the same
// fixed grid on every rank; CTA b owns slice b of the message on every rank and
// synchronises only with CTA b of the peers:
//
//   stage     in[slice b] -> own staging[parity]
//   barrier A store the call number into flagsA[b][me] of every rank (release.sys),
//             poll own flagsA[b][r] for every r (acquire.sys, local memory)
//   one-shot  (small messages, or two ranks): out[v] = sum_r staging_r[v], rank order
//   two-shot  reduce sub-slice `me` of slice b from all ranks' staging and PUSH the
//             result into every rank's result copy; barrier B; copy own result -> out
//
// Accumulation is fp32 in rank order 0..world-1 with one rounding to bf16, so all
// ranks hold bit-identical results (the rule of csrc/custom_all_reduce.cuh:173-181,
// :196-197 in the reference).  Flags carry a monotonically increasing call number
// kept per CTA in device memory: nothing is reset, a peer that runs one call ahead
// cannot be misread (the test is flag - call >= 0), and the launch arguments never
// change, so the call can sit inside a CUDA graph.  Why double buffering suffices:
// CTA b reuses staging[parity] two calls later, after it passed barrier A of the
// call in between, which every peer's CTA b signals only after it finished reading.
//
// Messages up to 256 KiB skip the flags altogether ("push" path): every rank stores its
// vectors straight into a per-source slot of every peer's receive buffer and then
// polls its own slots until no 32-bit word holds the sentinel 0x80008000 any more (the
// data is its own flag; an input word equal to the sentinel, two negative zeros, is
// sent as +0, +0).  Three receive buffers rotate: call n uses buffer n % 3 and restores
// the sentinel in the range call n - 1 used, which is safe because a peer can write
// into that buffer again only after it has seen this rank's data of call n + 1.  That
// leaves one NVLink one-way latency plus a local poll on the critical path.
//
// Messages above that and up to 2 MiB take the same idea in two phases ("push2"): the
// ranks scatter-reduce and then broadcast, both times by storing into the receiver's
// sentinel-filled buffers.  CTA b's slice is cut into one sub-slice per rank; every
// rank stores sub-slice r of its input into rank r's scatter buffer (slot = source
// rank), polls its own scatter slots for its sub-slice from every source, sums them
// in rank order, stores the sum into every rank's gather buffer, and finally polls
// its own gather buffer for the other ranks' sums.  Per rank (world - 1) / world of the
// message leaves over NVLink in each phase, and the critical path is two one-way
// latencies plus local polls: no flag round trip, no peer loads.
//
// Every wait is bounded by wall time (%globaltimer); when it runs out the CTA sets
// the status word, keeps signalling so that nobody else waits for it, and returns.
// Peer data moves with plain loads and stores only (no multimem, no TMA).
#include "../../include/vtensor.h"
#include "vt_device.cuh"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <new>

namespace vt {
namespace {

constexpr int kArMaxWorld = 8;
constexpr int kArMaxCtas = 64;
constexpr int kArThreads = 512;
constexpr size_t kArFlagBytes = 4096;                        // one flag array: [64 CTAs][8 ranks] u32 = 2 KiB, padded
constexpr uint32_t kArTimedOut = 0xDEAD0A88u;
constexpr size_t kPushBytes = 256u << 10;                    // largest message of the push path
constexpr uint32_t kSentinel = 0x80008000u;                  // (-0.0, -0.0) in bf16: "not written yet"
constexpr size_t kPush2Bytes = 2u << 20;                     // largest message of the two-phase push path
// scatter area of one rotation: world regions of ceil(message / world) vectors plus per-CTA rounding slack
constexpr size_t kPush2ScatterBytes = kPush2Bytes + kArMaxWorld * (kArMaxCtas + 16) * 16;

struct ArDev {                                               // lives in local device memory
  int rank, world, n_ctas, one_shot_vecs, push_vecs, push2_vecs;
  unsigned long long wait_ns;
  size_t max_bytes;
  char *peer[kArMaxWorld];                                   // shared buffer of every rank, as mapped here
  uint32_t *epoch;                                           // [n_ctas] call numbers (local)
  uint32_t *push_epoch;                                      // [n_ctas] number of push-path calls (local)
  uint32_t *push_prev;                                       // [n_ctas] vectors of the previous push-path call (local)
  uint32_t *push2_epoch, *push2_prev;                        // the same two for the two-phase push path
  uint32_t *status;                                          // local
};

struct ArLaunch {                                            // index = blockIdx.y (0 unless ranks are emulated on one GPU)
  ArDev dev[kArMaxWorld];                                    // by value: no dependent load before the first flag goes out
  const void *in[kArMaxWorld];
  void *out[kArMaxWorld];
};

__device__ __forceinline__ uint32_t *flags_a(char *buf) { return reinterpret_cast<uint32_t *>(buf); }
__device__ __forceinline__ uint32_t *flags_b(char *buf) { return reinterpret_cast<uint32_t *>(buf + kArFlagBytes); }
__device__ __forceinline__ uint4 *staging(char *buf, size_t max_bytes, int parity) {
  return reinterpret_cast<uint4 *>(buf + 2 * kArFlagBytes + parity * max_bytes);
}
__device__ __forceinline__ uint4 *result(char *buf, size_t max_bytes, int parity) {
  return reinterpret_cast<uint4 *>(buf + 2 * kArFlagBytes + (2 + parity) * max_bytes);
}

// push path: receive buffer t (0..2), slot of source rank r
__device__ __forceinline__ uint4 *push_slot(char *buf, size_t max_bytes, int t, int r) {
  return reinterpret_cast<uint4 *>(buf + 2 * kArFlagBytes + 4 * max_bytes + (static_cast<size_t>(t) * kArMaxWorld + r) * kPushBytes);
}

// two-phase push path: scatter area of rotation t (regions by source rank inside), gather buffer of rotation t
__device__ __forceinline__ uint4 *push2_scatter(char *buf, size_t max_bytes, int t) {
  return reinterpret_cast<uint4 *>(buf + 2 * kArFlagBytes + 4 * max_bytes + 3 * kArMaxWorld * kPushBytes +
                                   static_cast<size_t>(t) * kPush2ScatterBytes);
}
__device__ __forceinline__ uint4 *push2_gather(char *buf, size_t max_bytes, int t) {
  return reinterpret_cast<uint4 *>(buf + 2 * kArFlagBytes + 4 * max_bytes + 3 * kArMaxWorld * kPushBytes +
                                   3 * kPush2ScatterBytes + static_cast<size_t>(t) * kPush2Bytes);
}

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys(const uint4 *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Threads r < world: tell rank r that this CTA reached call `e`, then wait until rank r
// said the same.  All threads return true unless some wait ran out of time.
__device__ __forceinline__ bool cta_barrier(const ArDev &d, bool second, uint32_t e, int *timed_out) {
  __syncthreads();                                           // every thread's earlier writes precede the release below
  const int b = blockIdx.x, r = threadIdx.x;
  if (r < d.world) {
    uint32_t *theirs = (second ? flags_b(d.peer[r]) : flags_a(d.peer[r])) + b * kArMaxWorld + d.rank;
    st_release_sys(theirs, e);
    const uint32_t *mine = (second ? flags_b(d.peer[d.rank]) : flags_a(d.peer[d.rank])) + b * kArMaxWorld + r;
    const unsigned long long t0 = global_ns();
    for (unsigned it = 0;; ++it) {
      if (static_cast<int>(ld_acquire_sys(mine) - e) >= 0) break;
      if ((it & 63u) == 63u && global_ns() - t0 > d.wait_ns) {
        *timed_out = 1;
        break;
      }
    }
  }
  __syncthreads();
  return *timed_out == 0;
}

__device__ __forceinline__ void add8(float *acc, const uint4 &v) {
  acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
  acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
// Sums vectors [lo, hi) of all ranks' staging copies, U vectors of every rank in
// flight per thread before the first add (a peer load is a ~2 us round trip), and
// hands each sum to `sink(v, sum)`.
template <int W, typename Sink>
__device__ __forceinline__ void reduce_range(const ArDev &d, int parity, int lo, int hi, Sink sink) {
  constexpr int U = W <= 2 ? 4 : (W <= 4 ? 2 : 1);
  const uint4 *src[W];
#pragma unroll
  for (int r = 0; r < W; ++r) src[r] = staging(d.peer[r], d.max_bytes, parity);
  for (int v0 = lo + threadIdx.x; v0 < hi; v0 += kArThreads * U) {
    uint4 x[U][W];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * kArThreads;
      if (v < hi) {
#pragma unroll
        for (int r = 0; r < W; ++r) x[u][r] = ld_relaxed_sys(src[r] + v);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * kArThreads;
      if (v < hi) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < W; ++r) add8(acc, x[u][r]);
        sink(v, make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7])));
      }
    }
  }
}

template <int W>
__device__ __forceinline__ void all_reduce_body(const ArDev &d, const uint4 *in, uint4 *out, int n_vec, int *timed_out) {
  const int b = blockIdx.x;
  const uint32_t e = d.epoch[b] + 1;
  const int parity = e & 1;
  const int per = (n_vec + d.n_ctas - 1) / d.n_ctas;
  const int lo = min(b * per, n_vec), hi = min(lo + per, n_vec);
  char *me = d.peer[d.rank];
  uint4 *stage = staging(me, d.max_bytes, parity);
  for (int v = lo + threadIdx.x; v < hi; v += kArThreads) stage[v] = in[v];
  bool ok = cta_barrier(d, false, e, timed_out);
  if (n_vec <= d.one_shot_vecs || W == 2) {
    if (ok) reduce_range<W>(d, parity, lo, hi, [&](int v, const uint4 &sum) { out[v] = sum; });
  } else {
    const int q = (hi - lo + W - 1) / W;
    const int s_lo = min(lo + d.rank * q, hi), s_hi = min(s_lo + q, hi);
    if (ok) {
      uint4 *dst[W];
#pragma unroll
      for (int r = 0; r < W; ++r) dst[r] = result(d.peer[r], d.max_bytes, parity);
      reduce_range<W>(d, parity, s_lo, s_hi, [&](int v, const uint4 &sum) {
#pragma unroll
        for (int r = 0; r < W; ++r) dst[r][v] = sum;
      });
    }
    ok = cta_barrier(d, true, e, timed_out) && ok;
    if (ok) {
      const uint4 *res = result(me, d.max_bytes, parity);
      for (int v = lo + threadIdx.x; v < hi; v += kArThreads) out[v] = ld_relaxed_sys(res + v);
    }
  }
  if (threadIdx.x == 0) {
    d.epoch[b] = e;
    if (!ok) atomicExch(d.status, kArTimedOut);
  }
}

template <int W>
__device__ __forceinline__ void push_body(const ArDev &d, const uint4 *in, uint4 *out, int n_vec, int *timed_out) {
  const int b = blockIdx.x;
  const uint32_t e = d.push_epoch[b] + 1;
  const int n_prev = static_cast<int>(d.push_prev[b]);
  const int cur = e % 3, clr = (e + 2) % 3;                  // clr held the data of push call e - 1
  const int per = (n_vec + d.n_ctas - 1) / d.n_ctas;
  const int lo = min(b * per, n_vec), hi = min(lo + per, n_vec);
  char *me = d.peer[d.rank];
  // 1. this rank's vectors into its slot of every rank's buffer
  for (int v = lo + threadIdx.x; v < hi; v += kArThreads) {
    uint4 x = in[v];
    x.x = x.x == kSentinel ? 0u : x.x; x.y = x.y == kSentinel ? 0u : x.y;
    x.z = x.z == kSentinel ? 0u : x.z; x.w = x.w == kSentinel ? 0u : x.w;
#pragma unroll
    for (int r = 0; r < W; ++r) push_slot(d.peer[r], d.max_bytes, cur, d.rank)[v] = x;
  }
  // 2. restore the sentinel where the previous push call landed (this CTA's slice of that extent)
  {
    const int per_p = (n_prev + d.n_ctas - 1) / d.n_ctas;
    const int lo_p = min(b * per_p, n_prev), hi_p = min(lo_p + per_p, n_prev);
    const uint4 s4 = make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
    for (int v = lo_p + threadIdx.x; v < hi_p; v += kArThreads)
#pragma unroll
      for (int r = 0; r < W; ++r) push_slot(me, d.max_bytes, clr, r)[v] = s4;
  }
  // 3. wait for every rank's vector (the data is the flag), sum in rank order
  bool ok = true;
  for (int v = lo + threadIdx.x; v < hi; v += kArThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < W; ++r) {
      const uint4 *src = push_slot(me, d.max_bytes, cur, r) + v;
      uint4 x = ld_relaxed_sys(src);
      if (x.x == kSentinel || x.y == kSentinel || x.z == kSentinel || x.w == kSentinel) {
        const unsigned long long t0 = global_ns();
        for (unsigned it = 0;; ++it) {
          x = ld_relaxed_sys(src);
          if (x.x != kSentinel && x.y != kSentinel && x.z != kSentinel && x.w != kSentinel) break;
          if ((it & 63u) == 63u && global_ns() - t0 > d.wait_ns) {
            ok = false;
            break;
          }
        }
      }
      add8(acc, x);
    }
    if (ok) out[v] = make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7]));
  }
  if (!ok) *timed_out = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    d.push_epoch[b] = e;
    d.push_prev[b] = static_cast<uint32_t>(n_vec);
    if (*timed_out) atomicExch(d.status, kArTimedOut);
  }
}

__device__ __forceinline__ uint4 no_sentinel(uint4 x) {
  x.x = x.x == kSentinel ? 0u : x.x; x.y = x.y == kSentinel ? 0u : x.y;
  x.z = x.z == kSentinel ? 0u : x.z; x.w = x.w == kSentinel ? 0u : x.w;
  return x;
}
__device__ __forceinline__ bool has_sentinel(const uint4 &x) {
  return x.x == kSentinel || x.y == kSentinel || x.z == kSentinel || x.w == kSentinel;
}
// Re-reads *src until no word holds the sentinel; false when the wait ran out.
__device__ __forceinline__ bool poll_vector(const uint4 *src, uint4 *x, unsigned long long wait_ns) {
  if (!has_sentinel(*x)) return true;
  const unsigned long long t0 = global_ns();
  for (unsigned it = 0;; ++it) {
    *x = ld_relaxed_sys(src);
    if (!has_sentinel(*x)) return true;
    if ((it & 63u) == 63u && global_ns() - t0 > wait_ns) return false;
  }
}

// Geometry of one CTA's slice in the two-phase push path: slice [lo, hi) of the message,
// q vectors per rank's sub-slice (the same q in every CTA, so that region offsets agree).
struct Push2Geo {
  int lo, hi, q, region;   // region = vectors per source region of the scatter area
  __device__ __forceinline__ Push2Geo(int n_vec, int n_ctas, int world, int b) {
    const int per = (n_vec + n_ctas - 1) / n_ctas;
    lo = min(b * per, n_vec);
    hi = min(lo + per, n_vec);
    q = (per + world - 1) / world;
    region = n_ctas * q;
  }
  __device__ __forceinline__ int sub_lo(int r) const { return min(lo + r * q, hi); }
  __device__ __forceinline__ int sub_hi(int r) const { return min(sub_lo(r) + q, hi); }
};

template <int W>
__device__ __forceinline__ void push2_body(const ArDev &d, const uint4 *in, uint4 *out, int n_vec, int *timed_out) {
  const int b = blockIdx.x, me_r = d.rank;
  const uint32_t e = d.push2_epoch[b] + 1;
  const int n_prev = static_cast<int>(d.push2_prev[b]);
  const int cur = e % 3, clr = (e + 2) % 3;                  // clr held the data of call e - 1 of this path
  const Push2Geo g(n_vec, d.n_ctas, W, b);
  char *me = d.peer[me_r];
  // 1. scatter: sub-slice r of this rank's input into region `me_r` of rank r's scatter area
  for (int i = threadIdx.x; i < g.hi - g.lo; i += kArThreads) {
    const int r = i / g.q;
    if (r != me_r)
      push2_scatter(d.peer[r], d.max_bytes, cur)[me_r * g.region + b * g.q + (i - r * g.q)] = no_sentinel(in[g.lo + i]);
  }
  // 2. restore the sentinel where the previous call of this path landed in this rank's buffers
  {
    const Push2Geo p(n_prev, d.n_ctas, W, b);
    const uint4 s4 = make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
    const int mine = p.sub_hi(me_r) - p.sub_lo(me_r);
    uint4 *sc = push2_scatter(me, d.max_bytes, clr);
    for (int i = threadIdx.x; i < mine * W; i += kArThreads) {
      const int r = i / max(mine, 1);
      if (r != me_r) sc[r * p.region + b * p.q + (i - r * mine)] = s4;
    }
    uint4 *ga = push2_gather(me, d.max_bytes, clr);
    for (int v = p.lo + threadIdx.x; v < p.hi; v += kArThreads) ga[v] = s4;
  }
  // 3. own sub-slice: wait for every source's vector (the data is the flag), sum in rank order,
  //    hand the sum to every rank's gather buffer
  bool ok = true;
  const int s_lo = g.sub_lo(me_r), s_hi = g.sub_hi(me_r);
  const uint4 *sc = push2_scatter(me, d.max_bytes, cur);
  for (int v = s_lo + threadIdx.x; v < s_hi; v += kArThreads) {
    uint4 x[W];
#pragma unroll
    for (int r = 0; r < W; ++r)
      x[r] = r == me_r ? in[v] : ld_relaxed_sys(sc + r * g.region + b * g.q + (v - s_lo));
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < W; ++r) {
      if (r != me_r) ok = poll_vector(sc + r * g.region + b * g.q + (v - s_lo), &x[r], d.wait_ns) && ok;
      add8(acc, x[r]);
    }
    const uint4 sum = make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7]));
    const uint4 sent = no_sentinel(sum);                     // (-0, -0) travels as (+0, +0)
#pragma unroll
    for (int r = 0; r < W; ++r)
      if (r != me_r) push2_gather(d.peer[r], d.max_bytes, cur)[v] = sent;
    if (ok) out[v] = sent;
  }
  // 4. the other ranks' sums
  {
    const uint4 *ga = push2_gather(me, d.max_bytes, cur);
    constexpr int U = 4;
    const int own = s_hi - s_lo, rest = (g.hi - g.lo) - own;
    for (int i0 = threadIdx.x; i0 < rest; i0 += kArThreads * U) {
      uint4 x[U];
      int vv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * kArThreads;
        vv[u] = g.lo + i + (g.lo + i >= s_lo ? own : 0);      // skip over the own sub-slice
        if (i < rest) x[u] = ld_relaxed_sys(ga + vv[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * kArThreads < rest) {
          ok = poll_vector(ga + vv[u], &x[u], d.wait_ns) && ok;
          if (ok) out[vv[u]] = x[u];
        }
      }
    }
  }
  if (!ok) *timed_out = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    d.push2_epoch[b] = e;
    d.push2_prev[b] = static_cast<uint32_t>(n_vec);
    if (*timed_out) atomicExch(d.status, kArTimedOut);
  }
}

__global__ void __launch_bounds__(kArThreads) fill_words_kernel(uint32_t *p, size_t n, uint32_t value) {
  for (size_t i = blockIdx.x * static_cast<size_t>(kArThreads) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * kArThreads)
    p[i] = value;
}

__global__ void __launch_bounds__(kArThreads, 2) all_reduce_kernel(const __grid_constant__ ArLaunch L, int n_vec) {
  __shared__ int timed_out;
  const ArDev &d = L.dev[blockIdx.y];
  const uint4 *in = static_cast<const uint4 *>(L.in[blockIdx.y]);
  uint4 *out = static_cast<uint4 *>(L.out[blockIdx.y]);
  pdl_launch_dependents();   // a programmatic dependent behind this call may start its own prologue now
  if (threadIdx.x == 0) timed_out = 0;
  __syncthreads();
  const bool push = n_vec <= d.push_vecs, push2 = !push && n_vec <= d.push2_vecs && d.world > 1;
#define VT_AR_CASE(W)                                              \
  case W:                                                          \
    if (push) push_body<W>(d, in, out, n_vec, &timed_out);         \
    else if (push2) push2_body<W>(d, in, out, n_vec, &timed_out);  \
    else all_reduce_body<W>(d, in, out, n_vec, &timed_out);        \
    break;
  switch (d.world) {
    VT_AR_CASE(1) VT_AR_CASE(2) VT_AR_CASE(3) VT_AR_CASE(4) VT_AR_CASE(5) VT_AR_CASE(6) VT_AR_CASE(7)
    default:
      if (push) push_body<8>(d, in, out, n_vec, &timed_out);
      else if (push2) push2_body<8>(d, in, out, n_vec, &timed_out);
      else all_reduce_body<8>(d, in, out, n_vec, &timed_out);
      break;
  }
#undef VT_AR_CASE
}

}  // namespace
}  // namespace vt

struct vt_ar {
  vt::ArDev host;                 // travels by value with every launch
  uint32_t *local = nullptr;      // device memory: epochs + status
  int device = 0;
};

namespace {
size_t push_bytes_total() { return 3 * vt::kArMaxWorld * vt::kPushBytes + 3 * vt::kPush2ScatterBytes + 3 * vt::kPush2Bytes; }
size_t shared_bytes(size_t max_bytes) { return 2 * vt::kArFlagBytes + 4 * max_bytes + push_bytes_total(); }
bool cuda_ok(cudaError_t e) { return e == cudaSuccess; }
}  // namespace

extern "C" {

int vt_ar_buffer_bytes(size_t max_bytes, size_t *bytes) {
  if (!bytes || max_bytes == 0 || max_bytes % 256 != 0) return VT_ERR_INVALID;
  *bytes = shared_bytes(max_bytes);
  return VT_OK;
}

int vt_ar_alloc(size_t bytes, void **buf) {
  if (!buf || bytes == 0) return VT_ERR_INVALID;
  void *p = nullptr;
  if (!cuda_ok(cudaMalloc(&p, bytes))) return VT_ERR_CUDA;
  if (!cuda_ok(cudaMemset(p, 0, bytes)) || !cuda_ok(cudaDeviceSynchronize())) {
    cudaFree(p);
    return VT_ERR_CUDA;
  }
  *buf = p;
  return VT_OK;
}

int vt_ar_free(void *buf) { return cuda_ok(cudaFree(buf)) ? VT_OK : VT_ERR_CUDA; }

int vt_ar_ipc_export(void *buf, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (!buf || !handle) return VT_ERR_INVALID;
  cudaIpcMemHandle_t h;
  if (!cuda_ok(cudaIpcGetMemHandle(&h, buf))) return VT_ERR_CUDA;
  memcpy(handle, &h, 64);
  return VT_OK;
}

int vt_ar_ipc_open(const unsigned char handle[64], void **buf) {
  if (!buf || !handle) return VT_ERR_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return cuda_ok(cudaIpcOpenMemHandle(buf, h, cudaIpcMemLazyEnablePeerAccess)) ? VT_OK : VT_ERR_CUDA;
}

int vt_ar_ipc_close(void *buf) { return cuda_ok(cudaIpcCloseMemHandle(buf)) ? VT_OK : VT_ERR_CUDA; }

int vt_ar_create(int rank, int world, void *const *peer_bufs, size_t max_bytes, int n_ctas, vt_ar **out) {
  if (!out || !peer_bufs || world < 1 || world > vt::kArMaxWorld || rank < 0 || rank >= world) return VT_ERR_INVALID;
  if (max_bytes == 0 || max_bytes % 256 != 0 || max_bytes > (size_t(1) << 30)) return VT_ERR_INVALID;
  if (n_ctas == 0) n_ctas = 32;
  if (n_ctas < 1 || n_ctas > vt::kArMaxCtas) return VT_ERR_INVALID;
  for (int r = 0; r < world; ++r)
    if (!peer_bufs[r] || (reinterpret_cast<uintptr_t>(peer_bufs[r]) & 255) != 0) return VT_ERR_INVALID;
  vt_ar *ar = new (std::nothrow) vt_ar();
  if (!ar) return VT_ERR_CUDA;
  if (!cuda_ok(cudaGetDevice(&ar->device)) ||
      !cuda_ok(cudaMalloc(&ar->local, (5 * vt::kArMaxCtas + 1) * sizeof(uint32_t))) ||
      !cuda_ok(cudaMemset(ar->local, 0, (5 * vt::kArMaxCtas + 1) * sizeof(uint32_t)))) {
    cudaFree(ar->local);
    delete ar;
    return VT_ERR_CUDA;
  }
  vt::ArDev &h = ar->host;
  h.rank = rank; h.world = world; h.n_ctas = n_ctas;
  // One-shot (every rank reads everything) costs ~10 us + 1.8 us per MiB fetched from peers, two-shot ~19 us +
  // 0.5 us per MiB of message (measured, 8 B200s): they cross where (world - 1) * bytes is about 6 MiB.
  h.one_shot_vecs = world > 1 ? static_cast<int>(((6u << 20) / (world - 1)) / 16) : 0;
  h.wait_ns = 1000000000ull;                                  // 1 s
  h.max_bytes = max_bytes;
  for (int r = 0; r < vt::kArMaxWorld; ++r) h.peer[r] = r < world ? static_cast<char *>(peer_bufs[r]) : nullptr;
  h.push_vecs = static_cast<int>(vt::kPushBytes / 16);
  h.epoch = ar->local;
  h.push_epoch = ar->local + vt::kArMaxCtas;
  h.push_prev = ar->local + 2 * vt::kArMaxCtas;
  h.push2_epoch = ar->local + 3 * vt::kArMaxCtas;
  h.push2_prev = ar->local + 4 * vt::kArMaxCtas;
  h.status = ar->local + 5 * vt::kArMaxCtas;
  h.push2_vecs = static_cast<int>(vt::kPush2Bytes / 16);
  // the receive buffers of the push path start out as "nothing written" (own buffer only: every rank does its own)
  char *push0 = static_cast<char *>(peer_bufs[rank]) + 2 * vt::kArFlagBytes + 4 * max_bytes;
  vt::fill_words_kernel<<<64, vt::kArThreads>>>(reinterpret_cast<uint32_t *>(push0), push_bytes_total() / 4, vt::kSentinel);
  if (!cuda_ok(cudaGetLastError()) || !cuda_ok(cudaDeviceSynchronize())) {
    cudaFree(ar->local);
    delete ar;
    return VT_ERR_CUDA;
  }
  *out = ar;
  return VT_OK;
}

int vt_ar_destroy(vt_ar *ar) {
  if (!ar) return VT_OK;
  cudaFree(ar->local);
  delete ar;
  return VT_OK;
}

int vt_ar_configure(vt_ar *ar, long long wait_ns, long long one_shot_bytes, long long push_bytes, long long push2_bytes) {
  if (!ar) return VT_ERR_INVALID;
  if (push2_bytes >= 0)
    ar->host.push2_vecs = static_cast<int>(std::min<long long>(push2_bytes, static_cast<long long>(vt::kPush2Bytes)) / 16);
  if (push_bytes >= 0)
    ar->host.push_vecs = static_cast<int>(std::min<long long>(push_bytes, static_cast<long long>(vt::kPushBytes)) / 16);
  if (wait_ns > 0) ar->host.wait_ns = static_cast<unsigned long long>(wait_ns);
  if (one_shot_bytes >= 0)
    ar->host.one_shot_vecs = static_cast<int>(std::min<long long>(one_shot_bytes / 16, 1 << 30));
  return VT_OK;
}

int vt_ar_status(vt_ar *ar, uint32_t *status) {
  if (!ar || !status) return VT_ERR_INVALID;
  return cuda_ok(cudaMemcpy(status, ar->host.status, sizeof(uint32_t), cudaMemcpyDeviceToHost)) ? VT_OK : VT_ERR_CUDA;
}

static int ar_checks(const vt_ar *ar, const void *in, const void *out, size_t n_elems) {
  if (!ar || !in || !out) return VT_ERR_INVALID;
  if (n_elems % 8 != 0 || ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return VT_ERR_UNSUPPORTED;
  if (n_elems * 2 > ar->host.max_bytes) return VT_ERR_TOO_LARGE;
  return VT_OK;
}

int vt_all_reduce(vt_ar *ar, const void *in, void *out, size_t n_elems, void *stream) {
  if (n_elems == 0) return ar ? VT_OK : VT_ERR_INVALID;
  const int st = ar_checks(ar, in, out, n_elems);
  if (st != VT_OK) return st;
  vt::ArLaunch L{};
  L.dev[0] = ar->host; L.in[0] = in; L.out[0] = out;
  vt::all_reduce_kernel<<<dim3(ar->host.n_ctas, 1), vt::kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      L, static_cast<int>(n_elems / 8));
  return cudaGetLastError() == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

int vt_all_reduce_emulated(vt_ar *const *ars, const void *const *ins, void *const *outs, int world, size_t n_elems,
                           void *stream) {
  if (!ars || !ins || !outs || world < 1 || world > vt::kArMaxWorld) return VT_ERR_INVALID;
  if (n_elems == 0) return VT_OK;
  vt::ArLaunch L{};
  for (int r = 0; r < world; ++r) {
    const int st = ar_checks(ars[r], ins[r], outs[r], n_elems);
    if (st != VT_OK) return st;
    if (ars[r]->host.world != world || ars[r]->host.rank != r || ars[r]->host.n_ctas != ars[0]->host.n_ctas)
      return VT_ERR_INVALID;
    L.dev[r] = ars[r]->host; L.in[r] = ins[r]; L.out[r] = outs[r];
  }
  int n_vec = static_cast<int>(n_elems / 8);
  void *args[] = {&L, &n_vec};
  // All ranks' CTAs wait on one another, so they must be resident together: a
  // cooperative launch refuses (instead of hanging) when they do not fit.
  const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(vt::all_reduce_kernel),
                                                    dim3(ars[0]->host.n_ctas, world), dim3(vt::kArThreads), args, 0,
                                                    static_cast<cudaStream_t>(stream));
  if (e == cudaErrorCooperativeLaunchTooLarge) return VT_ERR_TOO_LARGE;
  return e == cudaSuccess ? VT_OK : VT_ERR_CUDA;
}

}  // extern "C"
