// Chunk pool, per-slot virtual ranges and pointer tables (C++ side of the C ABI).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "../../include/vtensor.h"
#include "vt_driver.h"

struct vt_pool {
  vt::Driver *drv = nullptr;
  int device = 0;
  size_t chunk_bytes = 0;
  size_t total = 0;

  std::mutex mu;  // free list
  std::vector<CUmemGenericAllocationHandle> free_list;

  struct Request { vt_seg *seg; int n_chunks; uint64_t epoch; };
  std::mutex qmu;
  std::condition_variable qcv;
  std::deque<Request> queue;
  bool stop = false;
  std::thread worker;

  std::atomic<uint64_t> map_calls{0}, unmap_calls{0}, set_access_calls{0}, map_ns{0}, access_ns{0};
  std::atomic<uint64_t> async_requests{0}, async_completed{0}, async_failed{0};
  std::atomic<int64_t> segments{0}, tables{0};
};

struct vt_seg {
  vt_pool *pool = nullptr;
  int n_layers = 0;
  size_t reserve = 0;  // bytes per range, multiple of the chunk size
  CUdeviceptr base = 0;

  std::mutex op_mu;  // serialises structural changes (grow / release / destroy)
  std::mutex mu;     // guards the fields below
  std::condition_variable cv;
  size_t mapped = 0;  // per range
  size_t used = 0;    // per range
  int pending = 0;    // queued or running background growths
  int async_status = VT_OK;
  uint64_t epoch = 0;  // bumped by release: queued growths of older epochs are dropped
  // A release whose cuMemUnmap failed part-way leaves the ranges mapped to different
  // frontiers; until a later release / destroy completes, growth and row bookkeeping are refused.
  bool poisoned = false;
  // chunks[r] = handles mapped into range r (r = 2 * layer + {0: K, 1: V}), in address order
  std::vector<std::vector<CUmemGenericAllocationHandle>> chunks;
};

struct vt_table {
  vt_pool *pool = nullptr;
  int n_slots = 0;
  CUdeviceptr dptr = 0;
};

namespace vt {
void set_last_driver_error(int r);
int grow_chunks(vt_seg *seg, size_t n_chunks);  // caller holds seg->op_mu
}  // namespace vt
