// Probe: one 128-row tcgen05.mma tile with operands written to shared memory in the
// 128-byte-swizzle canonical layouts, accumulator in tensor memory, read back with
// tcgen05.ld and compared with a host reference.  Two cases:
//   1. D[128 x 64]  = A[128 x 128] . B[64 x 128]^T   A and B K-major (the Q.K^T shape)
//   2. D[128 x 128] = A[128 x 64]  . B[64 x 128]     B MN-major     (the P.V shape)
// Build: make -C glake_b200/csrc probe ; run: glake_b200/csrc/probe/umma_tile
// Every wait is bounded; on a timeout the kernel reports it and still frees its
// tensor memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../vt_device.cuh"
#include "../vt_umma.cuh"

using namespace vt;

// A: row-major [128][K].  B: K-major -> [N][K] row-major; MN-major -> [K][N] row-major.
template <bool B_MN>
__global__ void __launch_bounds__(128) umma_probe(const __nv_bfloat16 *A, const __nv_bfloat16 *B, float *D, int N, int K,
                                                  int *status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_slot;
  const uint32_t s0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *s = smem_raw + (s0 - smem_u32(smem_raw));
  const int a_slabs = (K + 63) / 64;
  unsigned char *sa = s;                         // a_slabs x [128 rows][128 B]
  unsigned char *sb = s + a_slabs * 128 * 128;   // K-major: K/64 x [N][128 B]; MN-major: N/64 x [K][128 B]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i < 128 * (K / 8); i += 128) {           // 16-byte chunks of A
    const int r = i / (K / 8), ck = i % (K / 8), slab = ck / 8, c = ck % 8;
    *reinterpret_cast<uint4 *>(sa + slab * 128 * 128 + sw128_offset(r, c)) =
        *reinterpret_cast<const uint4 *>(A + static_cast<size_t>(r) * K + ck * 8);
  }
  if (!B_MN) {
    for (int i = tid; i < N * (K / 8); i += 128) {
      const int r = i / (K / 8), ck = i % (K / 8), slab = ck / 8, c = ck % 8;
      *reinterpret_cast<uint4 *>(sb + slab * N * 128 + sw128_offset(r, c)) =
          *reinterpret_cast<const uint4 *>(B + static_cast<size_t>(r) * K + ck * 8);
    }
  } else {
    for (int i = tid; i < K * (N / 8); i += 128) {
      const int r = i / (N / 8), cn = i % (N / 8), slab = cn / 8, c = cn % 8;   // r = k index (row), cn = 8-element chunk of n
      *reinterpret_cast<uint4 *>(sb + slab * K * 128 + sw128_offset(r, c)) =
          *reinterpret_cast<const uint4 *>(B + static_cast<size_t>(r) * N + cn * 8);
    }
  }
  if (tid == 0) {
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  const uint32_t cols = N < 32 ? 32 : N;
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), cols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();            // the generic-proxy stores above must be visible to the tensor core's reads
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = tmem_base_slot;

  if (tid == 0) {
    const uint32_t idesc = umma_idesc_bf16_f32(128, N, /*a_mn=*/false, /*b_mn=*/B_MN);
    for (int kk = 0; kk < K / 16; ++kk) {
      const uint64_t da = umma_desc_sw128(smem_u32(sa) + (kk / 4) * 128 * 128 + (kk % 4) * 32, /*lbo=*/0, /*sbo=*/1024);
      uint64_t db;
      if (!B_MN) db = umma_desc_sw128(smem_u32(sb) + (kk / 4) * N * 128 + (kk % 4) * 32, 0, 1024);
      else db = umma_desc_sw128(smem_u32(sb) + kk * 16 * 128, /*lbo = next 64 n*/ K * 128, /*sbo = next 8 k*/ 1024);
      umma_bf16(tmem, da, db, idesc, kk > 0);
    }
    umma_commit(smem_u32(&bar));
  }
  const bool ok = mbar_wait(smem_u32(&bar), 0);
  tcgen05_fence_after();
  if (ok) {
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      tmem_ld_wait();
      for (int j = 0; j < 32; ++j) D[static_cast<size_t>(warp * 32 + lane) * N + c0 + j] = __uint_as_float(v[j]);
    }
  } else if (tid == 0) {
    *status = 1;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, cols);
}

static float bf(float x) { return __bfloat162float(__float2bfloat16(x)); }

template <bool B_MN>
static int run_case(int N, int K, const char *name) {
  std::vector<float> a(128 * K), b(static_cast<size_t>(N) * K), ref(128 * N, 0.f);
  srand(7 + N);
  for (auto &x : a) x = bf((rand() % 2001 - 1000) / 500.f);
  for (auto &x : b) x = bf((rand() % 2001 - 1000) / 500.f);
  for (int m = 0; m < 128; ++m)
    for (int n = 0; n < N; ++n) {
      double acc = 0;
      for (int k = 0; k < K; ++k) acc += static_cast<double>(a[m * K + k]) * (B_MN ? b[static_cast<size_t>(k) * N + n] : b[static_cast<size_t>(n) * K + k]);
      ref[m * N + n] = static_cast<float>(acc);
    }
  std::vector<__nv_bfloat16> ah(a.size()), bh(b.size());
  for (size_t i = 0; i < a.size(); ++i) ah[i] = __float2bfloat16(a[i]);
  for (size_t i = 0; i < b.size(); ++i) bh[i] = __float2bfloat16(b[i]);
  __nv_bfloat16 *da, *db;
  float *dd;
  int *ds;
  cudaMalloc(&da, ah.size() * 2); cudaMalloc(&db, bh.size() * 2); cudaMalloc(&dd, ref.size() * 4); cudaMalloc(&ds, 4);
  cudaMemcpy(da, ah.data(), ah.size() * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(db, bh.data(), bh.size() * 2, cudaMemcpyHostToDevice);
  cudaMemset(dd, 0, ref.size() * 4); cudaMemset(ds, 0, 4);
  const int smem = 1024 + ((K + 63) / 64) * 128 * 128 + (B_MN ? (N / 64) * K * 128 : ((K + 63) / 64) * N * 128);
  cudaFuncSetAttribute(umma_probe<B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  umma_probe<B_MN><<<1, 128, smem>>>(da, db, dd, N, K, ds);
  const cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { printf("%s: CUDA error %s\n", name, cudaGetErrorString(e)); return 2; }
  std::vector<float> out(ref.size());
  int st = 0;
  cudaMemcpy(out.data(), dd, out.size() * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(&st, ds, 4, cudaMemcpyDeviceToHost);
  double max_err = 0, max_ref = 0;
  for (size_t i = 0; i < ref.size(); ++i) { max_err = fmax(max_err, fabs(out[i] - ref[i])); max_ref = fmax(max_ref, fabs(ref[i])); }
  printf("%s: N %d K %d  status %d  max|err| %.3e  max|ref| %.3e  d[0][0..3] %.3f %.3f %.3f %.3f ref %.3f %.3f %.3f %.3f -> %s\n", name, N, K,
         st, max_err, max_ref, out[0], out[1], out[2], out[3], ref[0], ref[1], ref[2], ref[3],
         (st == 0 && max_err <= 1e-3 * max_ref) ? "OK" : "MISMATCH");
  cudaFree(da); cudaFree(db); cudaFree(dd); cudaFree(ds);
  return (st == 0 && max_err <= 1e-3 * max_ref) ? 0 : 1;
}

int main() {
  int bad = 0;
  bad += run_case<false>(64, 128, "K-major B (Q.K^T shape)");
  bad += run_case<true>(128, 64, "MN-major B (P.V shape)");
  bad += run_case<true>(128, 32, "MN-major B, 32 tokens");
  return bad;
}
