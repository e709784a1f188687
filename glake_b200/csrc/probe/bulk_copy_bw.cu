// Diagnostic, not part of libvtensor: read bandwidth of a cp.async.bulk shared-memory
// ring as a function of the bytes moved per request, next to a plain ld.global
// stream.  This measurement is why every bulk copy in the attention kernels moves
// 1 KiB: on B200 the copy engine sustains ~7.3 TB/s with requests >= 1 KiB, ~6.0 TB/s
// at 512 B and ~3.3 TB/s at 256 B.
// Build: make -C glake_b200/csrc probe     Run: glake_b200/csrc/probe/bulk_copy_bw
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cuda_runtime.h>
#include "../vt_device.cuh"
using namespace vt;

template<int STAGES>
__global__ void bulk_ring(const char* src, size_t bytes_per_cta, int stage_bytes, int copy_bytes, unsigned* sink, int use_hint, size_t src_stride) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* bars = (uint64_t*)(smem + (size_t)STAGES*stage_bytes);
  uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars+STAGES), ring0 = smem_u32(smem);
  int warp = threadIdx.x>>5, lane = threadIdx.x&31;
  int ncw = (blockDim.x>>5)-1;
  if (threadIdx.x==0){ for(int s=0;s<STAGES;++s){ mbar_init(full0+8*s,1); mbar_init(empty0+8*s,ncw);} mbar_fence_init(); }
  __syncthreads();
  const char* base = src + (size_t)blockIdx.x * bytes_per_cta;
  int ntiles = bytes_per_cta / stage_bytes;
  int per = stage_bytes / copy_bytes;
  if (warp==ncw){
    uint64_t pol = l2_policy_evict_first();
    for(int t=0;t<ntiles;++t){ int s=t%STAGES; if(t>=STAGES && !mbar_wait(empty0+8*s, ((t/STAGES)-1)&1)) return;
      if(lane==0) mbar_arrive_expect_tx(full0+8*s, stage_bytes); __syncwarp();
      for(int c=lane;c<per;c+=32){ const char* g = base + ((size_t)t*per + c)*src_stride; uint32_t d = ring0 + s*stage_bytes + c*copy_bytes;
        if(use_hint) bulk_g2s_hint(d,g,copy_bytes,full0+8*s,pol); else bulk_g2s(d,g,copy_bytes,full0+8*s);} }
    return;
  }
  unsigned acc=0;
  for(int t=0;t<ntiles;++t){ int s=t%STAGES; if(!mbar_wait(full0+8*s,(t/STAGES)&1)) return;
    // touch: each consumer thread reads 16B per 512B
    const uint4* p = (const uint4*)(smem + s*stage_bytes);
    for(int i=threadIdx.x; i<stage_bytes/16; i+=ncw*32) { uint4 v=p[i]; acc += v.x^v.y^v.z^v.w; }
    __syncwarp(); if(lane==0) mbar_arrive(empty0+8*s); }
  if(acc==0x12345678) sink[0]=acc;
}

__global__ void ldg_stream(const uint4* src, size_t n16, unsigned* sink){
  size_t i = (size_t)blockIdx.x*blockDim.x + threadIdx.x; size_t stride=(size_t)gridDim.x*blockDim.x; unsigned acc=0;
  #pragma unroll 8
  for(; i<n16; i+=stride){ uint4 v = __ldcs(src+i); acc += v.x^v.y^v.z^v.w; }
  if(acc==0x12345678) sink[0]=acc;
}

int main(int argc,char**argv){
  size_t total = (size_t)4<<30; char* buf; cudaMalloc(&buf,total); cudaMemset(buf,1,total); unsigned* sink; cudaMalloc(&sink,4);
  cudaEvent_t a,z; cudaEventCreate(&a); cudaEventCreate(&z);
  auto timeit=[&](auto fn){ fn(); cudaDeviceSynchronize(); float best=1e9; for(int r=0;r<5;++r){ cudaEventRecord(a); fn(); cudaEventRecord(z); cudaEventSynchronize(z); float ms; cudaEventElapsedTime(&ms,a,z); if(ms<best)best=ms;} return best; };
  { float ms=timeit([&]{ ldg_stream<<<148*8,512>>>((const uint4*)buf,total/16,sink);}); printf("ldg stream: %.0f GB/s\n", total/ms/1e6); }
  cudaError_t e;
  int cfgs[][5] = { // stage_bytes, copy_bytes, ctas_per_sm(target via smem), consumer warps, stages
    {16384,256,3,4,4},{16384,512,3,4,4},{16384,1024,3,4,4},{16384,2048,3,4,4},{16384,4096,3,4,4},{16384,16384,3,4,4},
    {32768,256,1,4,4},{32768,32768,1,4,4},{32768,16384,1,4,4},{32768,1024,1,4,4},
    {8192,256,6,4,4},{8192,8192,6,4,4},{65536,65536,1,8,3},{32768,32768,2,4,3},{16384,128,3,4,4}};
  for(auto& c: cfgs){ int stage=c[0], copy=c[1], cw=c[3], st=c[4]; size_t smem=(size_t)st*stage+128;
    size_t per_cta = (size_t)2<<20; int ctas = total/per_cta;
    for (int hint=0; hint<2; ++hint){
    float ms;
    if(st==4){ cudaFuncSetAttribute(bulk_ring<4>,cudaFuncAttributeMaxDynamicSharedMemorySize,(int)smem); ms=timeit([&]{ bulk_ring<4><<<ctas,(cw+1)*32,smem>>>(buf,per_cta,stage,copy,sink,hint,copy);}); }
    else { cudaFuncSetAttribute(bulk_ring<3>,cudaFuncAttributeMaxDynamicSharedMemorySize,(int)smem); ms=timeit([&]{ bulk_ring<3><<<ctas,(cw+1)*32,smem>>>(buf,per_cta,stage,copy,sink,hint,copy);}); }
    e=cudaGetLastError(); printf("stage %6d copy %6d stages %d cwarps %d hint %d smem %zu: %.0f GB/s %s\n", stage,copy,st,cw,hint,smem,total/ms/1e6, e?cudaGetErrorString(e):""); }
  }
  return 0; }
