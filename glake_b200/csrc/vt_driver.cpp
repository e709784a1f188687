#include "vt_driver.h"

#include <dlfcn.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <thread>

namespace vt {
namespace {

// ---------------------------------------------------------------------------
// real driver: entry points looked up by name in libcuda.so.1
// ---------------------------------------------------------------------------
struct Api {
  void *lib = nullptr;
  CUresult (*cuInit)(unsigned) = nullptr;
  CUresult (*cuDeviceGet)(CUdevice *, int) = nullptr;
  CUresult (*cuDevicePrimaryCtxRetain)(CUcontext *, CUdevice) = nullptr;
  CUresult (*cuDevicePrimaryCtxRelease)(CUdevice) = nullptr;
  CUresult (*cuCtxSetCurrent)(CUcontext) = nullptr;
  CUresult (*cuCtxGetCurrent)(CUcontext *) = nullptr;
  CUresult (*cuMemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *,
                                            CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *,
                          unsigned long long) = nullptr;
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*cuMemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr,
                                  unsigned long long) = nullptr;
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                       unsigned long long) = nullptr;
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemAlloc)(CUdeviceptr *, size_t) = nullptr;
  CUresult (*cuMemFree)(CUdeviceptr) = nullptr;
  CUresult (*cuMemcpyHtoD)(CUdeviceptr, const void *, size_t) = nullptr;
  CUresult (*cuMemcpyDtoH)(void *, CUdeviceptr, size_t) = nullptr;
  CUresult (*cuGetErrorString)(CUresult, const char **) = nullptr;
};

template <typename F>
bool sym(void *lib, const char *name, F *out, std::string *why) {
  *out = reinterpret_cast<F>(dlsym(lib, name));
  if (!*out && why) *why = std::string("libcuda lacks ") + name;
  return *out != nullptr;
}

Api *load_api(std::string *why) {
  static std::mutex mu;
  static Api *api = nullptr;
  static std::string err;
  std::lock_guard<std::mutex> g(mu);
  if (api) return api;
  if (!err.empty()) { if (why) *why = err; return nullptr; }
  void *lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) { err = std::string("dlopen libcuda.so.1: ") + dlerror(); if (why) *why = err; return nullptr; }
  Api *a = new Api;
  a->lib = lib;
  bool ok = sym(lib, "cuInit", &a->cuInit, &err) && sym(lib, "cuDeviceGet", &a->cuDeviceGet, &err) &&
            sym(lib, "cuDevicePrimaryCtxRetain", &a->cuDevicePrimaryCtxRetain, &err) &&
            sym(lib, "cuDevicePrimaryCtxRelease_v2", &a->cuDevicePrimaryCtxRelease, &err) &&
            sym(lib, "cuCtxSetCurrent", &a->cuCtxSetCurrent, &err) &&
            sym(lib, "cuCtxGetCurrent", &a->cuCtxGetCurrent, &err) &&
            sym(lib, "cuMemGetAllocationGranularity", &a->cuMemGetAllocationGranularity, &err) &&
            sym(lib, "cuMemCreate", &a->cuMemCreate, &err) && sym(lib, "cuMemRelease", &a->cuMemRelease, &err) &&
            sym(lib, "cuMemAddressReserve", &a->cuMemAddressReserve, &err) &&
            sym(lib, "cuMemAddressFree", &a->cuMemAddressFree, &err) && sym(lib, "cuMemMap", &a->cuMemMap, &err) &&
            sym(lib, "cuMemSetAccess", &a->cuMemSetAccess, &err) && sym(lib, "cuMemUnmap", &a->cuMemUnmap, &err) &&
            sym(lib, "cuMemAlloc_v2", &a->cuMemAlloc, &err) && sym(lib, "cuMemFree_v2", &a->cuMemFree, &err) &&
            sym(lib, "cuMemcpyHtoD_v2", &a->cuMemcpyHtoD, &err) &&
            sym(lib, "cuMemcpyDtoH_v2", &a->cuMemcpyDtoH, &err) &&
            sym(lib, "cuGetErrorString", &a->cuGetErrorString, &err);
  if (!ok) { delete a; if (why) *why = err; return nullptr; }
  api = a;
  return api;
}

class RealDriver final : public Driver {
 public:
  explicit RealDriver(Api *a) : a_(a) {}
  ~RealDriver() override {
    if (ctx_) a_->cuDevicePrimaryCtxRelease(dev_);
  }
  CUresult init(int device) override {
    CUresult r = a_->cuInit(0);
    if (r != CUDA_SUCCESS) return r;
    if ((r = a_->cuDeviceGet(&dev_, device)) != CUDA_SUCCESS) return r;
    // The primary context is the one the CUDA runtime (and torch) use for this
    // device, so addresses mapped here are valid in the caller's kernels.
    if ((r = a_->cuDevicePrimaryCtxRetain(&ctx_, dev_)) != CUDA_SUCCESS) return r;
    device_ = device;
    return a_->cuCtxSetCurrent(ctx_);
  }
  CUresult bind_thread() override {
    CUcontext cur = nullptr;
    CUresult r = a_->cuCtxGetCurrent(&cur);
    if (r == CUDA_SUCCESS && cur == ctx_) return r;
    return a_->cuCtxSetCurrent(ctx_);
  }
  CUmemAllocationProp prop() const {
    CUmemAllocationProp p;
    std::memset(&p, 0, sizeof(p));
    p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    p.location.id = device_;
    return p;
  }
  CUresult granularity(size_t *out) override {
    CUmemAllocationProp p = prop();
    return a_->cuMemGetAllocationGranularity(out, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  }
  CUresult mem_create(CUmemGenericAllocationHandle *h, size_t bytes) override {
    CUmemAllocationProp p = prop();
    return a_->cuMemCreate(h, bytes, &p, 0);
  }
  CUresult mem_release(CUmemGenericAllocationHandle h) override { return a_->cuMemRelease(h); }
  CUresult address_reserve(CUdeviceptr *p, size_t bytes, size_t align) override {
    return a_->cuMemAddressReserve(p, bytes, align, 0, 0);
  }
  CUresult address_free(CUdeviceptr p, size_t bytes) override { return a_->cuMemAddressFree(p, bytes); }
  CUresult mem_map(CUdeviceptr p, size_t bytes, CUmemGenericAllocationHandle h) override {
    return a_->cuMemMap(p, bytes, 0, h, 0);
  }
  CUresult set_access_rw(CUdeviceptr p, size_t bytes) override {
    CUmemAccessDesc d;
    std::memset(&d, 0, sizeof(d));
    d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    d.location.id = device_;
    d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    return a_->cuMemSetAccess(p, bytes, &d, 1);
  }
  CUresult mem_unmap(CUdeviceptr p, size_t bytes) override { return a_->cuMemUnmap(p, bytes); }
  CUresult mem_alloc(CUdeviceptr *p, size_t bytes) override { return a_->cuMemAlloc(p, bytes); }
  CUresult mem_free(CUdeviceptr p) override { return a_->cuMemFree(p); }
  CUresult memcpy_htod(CUdeviceptr dst, const void *src, size_t bytes) override {
    return a_->cuMemcpyHtoD(dst, src, bytes);
  }
  CUresult memcpy_dtoh(void *dst, CUdeviceptr src, size_t bytes) override {
    return a_->cuMemcpyDtoH(dst, src, bytes);
  }
  const char *error_string(CUresult r) override {
    const char *s = nullptr;
    if (a_->cuGetErrorString(r, &s) != CUDA_SUCCESS || !s) return "unknown CUDA driver error";
    return s;
  }

 private:
  Api *a_;
  CUdevice dev_ = 0;
  CUcontext ctx_ = nullptr;
  int device_ = 0;
};

// ---------------------------------------------------------------------------
// mock driver
// ---------------------------------------------------------------------------
std::mutex g_mock_mu;
std::map<std::string, int> g_fail_nth;  // call name -> remaining calls until failure
std::atomic<int> g_map_delay_us{0};

bool mock_should_fail(const char *call) {
  std::lock_guard<std::mutex> g(g_mock_mu);
  auto it = g_fail_nth.find(call);
  if (it == g_fail_nth.end() || it->second <= 0) return false;
  if (--it->second == 0) { g_fail_nth.erase(it); return true; }
  return false;
}

class MockDriver final : public Driver {
 public:
  bool is_mock() const override { return true; }
  CUresult init(int) override { return CUDA_SUCCESS; }
  CUresult bind_thread() override { return CUDA_SUCCESS; }
  CUresult granularity(size_t *out) override { *out = 2u << 20; return CUDA_SUCCESS; }
  CUresult mem_create(CUmemGenericAllocationHandle *h, size_t bytes) override {
    if (mock_should_fail("cuMemCreate")) return CUDA_ERROR_OUT_OF_MEMORY;
    std::lock_guard<std::mutex> g(mu_);
    *h = next_handle_++;
    handles_[*h] = bytes;
    return CUDA_SUCCESS;
  }
  CUresult mem_release(CUmemGenericAllocationHandle h) override {
    std::lock_guard<std::mutex> g(mu_);
    return handles_.erase(h) ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
  }
  CUresult address_reserve(CUdeviceptr *p, size_t bytes, size_t align) override {
    if (mock_should_fail("cuMemAddressReserve")) return CUDA_ERROR_OUT_OF_MEMORY;
    std::lock_guard<std::mutex> g(mu_);
    if (align == 0) align = 2u << 20;
    next_va_ = (next_va_ + align - 1) / align * align;
    *p = next_va_;
    reservations_[next_va_] = bytes;
    next_va_ += bytes + align;
    return CUDA_SUCCESS;
  }
  CUresult address_free(CUdeviceptr p, size_t bytes) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reservations_.find(p);
    if (it == reservations_.end() || it->second != bytes) return CUDA_ERROR_INVALID_VALUE;
    for (auto &m : maps_)
      if (m.first >= p && m.first < p + bytes) return CUDA_ERROR_INVALID_VALUE;  // still mapped
    reservations_.erase(it);
    return CUDA_SUCCESS;
  }
  CUresult mem_map(CUdeviceptr p, size_t bytes, CUmemGenericAllocationHandle h) override {
    int d = g_map_delay_us.load();
    if (d > 0) std::this_thread::sleep_for(std::chrono::microseconds(d));
    if (mock_should_fail("cuMemMap")) return CUDA_ERROR_INVALID_VALUE;
    std::lock_guard<std::mutex> g(mu_);
    auto hi = handles_.find(h);
    if (hi == handles_.end() || hi->second != bytes) return CUDA_ERROR_INVALID_VALUE;
    if (!inside_reservation(p, bytes) || overlaps(p, bytes) || mapped_handles_.count(h))
      return CUDA_ERROR_INVALID_VALUE;
    maps_[p] = {bytes, h};
    mapped_handles_.insert(h);
    return CUDA_SUCCESS;
  }
  CUresult set_access_rw(CUdeviceptr p, size_t bytes) override {
    if (mock_should_fail("cuMemSetAccess")) return CUDA_ERROR_INVALID_VALUE;
    std::lock_guard<std::mutex> g(mu_);
    // every byte of [p, p + bytes) must be mapped
    CUdeviceptr cur = p;
    while (cur < p + bytes) {
      auto it = maps_.find(cur);
      if (it == maps_.end()) return CUDA_ERROR_INVALID_VALUE;
      cur += it->second.bytes;
    }
    return cur == p + bytes ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
  }
  CUresult mem_unmap(CUdeviceptr p, size_t bytes) override {
    if (mock_should_fail("cuMemUnmap")) return CUDA_ERROR_INVALID_VALUE;
    std::lock_guard<std::mutex> g(mu_);
    // must cover whole mappings exactly
    CUdeviceptr cur = p;
    while (cur < p + bytes) {
      auto it = maps_.find(cur);
      if (it == maps_.end() || cur + it->second.bytes > p + bytes) return CUDA_ERROR_INVALID_VALUE;
      cur += it->second.bytes;
    }
    for (auto it = maps_.lower_bound(p); it != maps_.end() && it->first < p + bytes;) {
      mapped_handles_.erase(it->second.handle);
      it = maps_.erase(it);
    }
    return CUDA_SUCCESS;
  }
  CUresult mem_alloc(CUdeviceptr *p, size_t bytes) override {
    if (mock_should_fail("cuMemAlloc")) return CUDA_ERROR_OUT_OF_MEMORY;
    void *m = calloc(1, bytes ? bytes : 1);  // host memory: tables are readable in tests
    *p = reinterpret_cast<CUdeviceptr>(m);
    return m ? CUDA_SUCCESS : CUDA_ERROR_OUT_OF_MEMORY;
  }
  CUresult mem_free(CUdeviceptr p) override { free(reinterpret_cast<void *>(p)); return CUDA_SUCCESS; }
  CUresult memcpy_htod(CUdeviceptr dst, const void *src, size_t bytes) override {
    if (mock_should_fail("cuMemcpyHtoD")) return CUDA_ERROR_INVALID_VALUE;
    std::memcpy(reinterpret_cast<void *>(dst), src, bytes);
    return CUDA_SUCCESS;
  }
  CUresult memcpy_dtoh(void *dst, CUdeviceptr src, size_t bytes) override {
    std::memcpy(dst, reinterpret_cast<const void *>(src), bytes);  // tables only: ranges are synthetic
    return CUDA_SUCCESS;
  }
  const char *error_string(CUresult r) override {
    switch (r) {
      case CUDA_SUCCESS: return "no error";
      case CUDA_ERROR_OUT_OF_MEMORY: return "out of memory (mock)";
      case CUDA_ERROR_INVALID_VALUE: return "invalid argument (mock)";
      default: return "mock driver error";
    }
  }

 private:
  struct Mapping { size_t bytes; CUmemGenericAllocationHandle handle; };
  bool inside_reservation(CUdeviceptr p, size_t bytes) {
    auto it = reservations_.upper_bound(p);
    if (it == reservations_.begin()) return false;
    --it;
    return p >= it->first && p + bytes <= it->first + it->second;
  }
  bool overlaps(CUdeviceptr p, size_t bytes) {
    auto it = maps_.lower_bound(p);
    if (it != maps_.end() && it->first < p + bytes) return true;
    if (it != maps_.begin()) { --it; if (it->first + it->second.bytes > p) return true; }
    return false;
  }
  std::mutex mu_;
  CUmemGenericAllocationHandle next_handle_ = 1;
  CUdeviceptr next_va_ = 0x7f0000000000ull;
  std::map<CUmemGenericAllocationHandle, size_t> handles_;
  std::map<CUdeviceptr, size_t> reservations_;
  std::map<CUdeviceptr, Mapping> maps_;
  std::set<CUmemGenericAllocationHandle> mapped_handles_;
};

}  // namespace

Driver *make_real_driver(std::string *why) {
  Api *a = load_api(why);
  return a ? new RealDriver(a) : nullptr;
}
Driver *make_mock_driver() { return new MockDriver; }

void mock_fail_nth(const char *call, int nth) {
  std::lock_guard<std::mutex> g(g_mock_mu);
  if (nth <= 0) g_fail_nth.erase(call); else g_fail_nth[call] = nth;
}
void mock_map_delay_us(int us) { g_map_delay_us.store(us < 0 ? 0 : us); }

}  // namespace vt
