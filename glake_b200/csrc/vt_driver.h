// Driver-call seam of the allocator.  The real implementation resolves the
// CUDA driver's virtual-memory-management entry points from libcuda.so.1 at run
// time (the library therefore loads on machines without a GPU); the mock keeps
// the same bookkeeping in host memory so that pool exhaustion, map failures and
// slow maps can be produced on the host without touching a GPU.
#pragma once
#include <cuda.h>

#include <cstddef>
#include <cstdint>
#include <string>

namespace vt {

class Driver {
 public:
  virtual ~Driver() = default;
  virtual CUresult init(int device) = 0;  // cuInit + retain/bind the primary context
  virtual CUresult bind_thread() = 0;     // make the context current on this thread
  virtual CUresult granularity(size_t *out) = 0;
  virtual CUresult mem_create(CUmemGenericAllocationHandle *h, size_t bytes) = 0;
  virtual CUresult mem_release(CUmemGenericAllocationHandle h) = 0;
  virtual CUresult address_reserve(CUdeviceptr *p, size_t bytes, size_t align) = 0;
  virtual CUresult address_free(CUdeviceptr p, size_t bytes) = 0;
  virtual CUresult mem_map(CUdeviceptr p, size_t bytes, CUmemGenericAllocationHandle h) = 0;
  virtual CUresult set_access_rw(CUdeviceptr p, size_t bytes) = 0;
  virtual CUresult mem_unmap(CUdeviceptr p, size_t bytes) = 0;
  virtual CUresult mem_alloc(CUdeviceptr *p, size_t bytes) = 0;
  virtual CUresult mem_free(CUdeviceptr p) = 0;
  virtual CUresult memcpy_htod(CUdeviceptr dst, const void *src, size_t bytes) = 0;
  virtual CUresult memcpy_dtoh(void *dst, CUdeviceptr src, size_t bytes) = 0;
  virtual const char *error_string(CUresult r) = 0;
  virtual bool is_mock() const { return false; }
};

// nullptr (and *why filled) when libcuda cannot be loaded.
Driver *make_real_driver(std::string *why);
Driver *make_mock_driver();

// Mock controls (process-wide, affect every mock driver instance).
void mock_fail_nth(const char *call, int nth);
void mock_map_delay_us(int us);

}  // namespace vt
