// Device-side helpers shared by the kernels: mbarrier / bulk-copy PTX wrappers
// (sm_90+ async proxy; compiled here for sm_100a only), bf16 / fp8 unpacking.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vt {

constexpr int kHeadDim = 128;
constexpr uint32_t kKernelErrMagic = 0xDEAD0A77u;  // value of the workspace status word after a failed wait
constexpr uint32_t kWaitLimit = 1u << 22;          // try_wait rounds before a wait gives up ...
constexpr unsigned long long kWaitLimitNs = 1000000000ull;   // ... or one second, whichever comes first

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false when the phase did not complete within kWaitLimitNs of wall time
// (a try_wait round may itself block for a hardware-defined time, so rounds are not
// counted; the clock is read only after a round that failed).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > kWaitLimitNs) return false;
  }
  return false;
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later
// async-proxy (bulk copy) accesses to it.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 1-D bulk async copy global -> this CTA's shared memory, completion counted in
// bytes on an mbarrier.  Both addresses 16-byte aligned, bytes a multiple of 16.
// No cluster multicast: the source is always this GPU's own memory and each CTA
// fetches its own tile.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Same with an L2 eviction-priority hint (KV rows are streamed once per step).
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          dst_smem),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Programmatic dependent launch (sm_90+): let the next kernel on the stream start
// once every CTA of this grid has passed this point (or exited) ...
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// ... and, in that next kernel, wait until the previous grid has completed and its
// writes are visible.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// two bf16 packed in a 32-bit word -> two floats (exact)
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// four e4m3 bytes packed in a 32-bit word -> four floats (exact)
__device__ __forceinline__ void e4m3x4_to_float(uint32_t w, float *f) {
  uint32_t h01, h23;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"(static_cast<unsigned short>(w & 0xffffu)));
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"(static_cast<unsigned short>(w >> 16)));
  float2 a = __half22float2(*reinterpret_cast<__half2 *>(&h01));
  float2 b = __half22float2(*reinterpret_cast<__half2 *>(&h23));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// float -> e4m3 byte, round-to-nearest-even, saturating to +-448
__device__ __forceinline__ uint32_t float2_to_e4m3x2(float lo, float hi) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// 16 bytes of cache -> floats: 8 (bf16) or 16 (fp8)
template <bool FP8>
struct Unpack;
template <>
struct Unpack<false> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void run(const uint4 &v, float *f) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
  }
};
template <>
struct Unpack<true> {
  static constexpr int N = 16;
  __device__ __forceinline__ static void run(const uint4 &v, float *f) {
    e4m3x4_to_float(v.x, f); e4m3x4_to_float(v.y, f + 4); e4m3x4_to_float(v.z, f + 8); e4m3x4_to_float(v.w, f + 12);
  }
};

}  // namespace vt
