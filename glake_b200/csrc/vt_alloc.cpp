// VMM allocator: physical 2 MiB chunks are created once, then only mapped into
// and unmapped from per-slot virtual ranges.  A sequence's K (or V) cache of one
// layer is therefore one contiguous address range for its whole life; growing
// it never copies and never changes its base address, which is what lets the
// attention kernel stream it with bulk copies and lets CUDA graphs replay.
#include "vt_alloc.h"

#include <chrono>
#include <cstring>
#include <new>

namespace vt {

static thread_local int g_last_driver_error = 0;
void set_last_driver_error(int r) { g_last_driver_error = r; }
int last_driver_error() { return g_last_driver_error; }

static std::atomic<bool> g_use_mock{false};

static inline uint64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch()).count();
}

#define VT_DRV(pool, expr)                                  \
  do {                                                      \
    CUresult _r = (expr);                                   \
    if (_r != CUDA_SUCCESS) {                               \
      vt::set_last_driver_error(static_cast<int>(_r));      \
      return VT_ERR_DRIVER;                                 \
    }                                                       \
  } while (0)

static inline CUdeviceptr range_base(const vt_seg *s, size_t r) { return s->base + r * s->reserve; }

// Maps n more chunks at the mapped frontier of every range of the segment.
// All-or-nothing: on any failure everything mapped by this call is unmapped and
// the chunks go back to the pool.
int grow_chunks(vt_seg *seg, size_t n) {
  if (n == 0) return VT_OK;
  vt_pool *pool = seg->pool;
  Driver *drv = pool->drv;
  const size_t cb = pool->chunk_bytes;
  const size_t ranges = 2 * static_cast<size_t>(seg->n_layers);
  size_t mapped;
  {
    std::lock_guard<std::mutex> g(seg->mu);
    if (seg->poisoned) return VT_ERR_STATE;
    mapped = seg->mapped;
  }
  if (mapped + n * cb > seg->reserve) return VT_ERR_RESERVE;

  std::vector<CUmemGenericAllocationHandle> take;
  {
    std::lock_guard<std::mutex> g(pool->mu);
    if (pool->free_list.size() < ranges * n) return VT_ERR_POOL_EMPTY;
    take.assign(pool->free_list.end() - ranges * n, pool->free_list.end());
    pool->free_list.resize(pool->free_list.size() - ranges * n);
  }
  CUresult err = CUDA_SUCCESS;
  if ((err = drv->bind_thread()) != CUDA_SUCCESS) {
    std::lock_guard<std::mutex> g(pool->mu);
    pool->free_list.insert(pool->free_list.end(), take.begin(), take.end());
    set_last_driver_error(err);
    return VT_ERR_DRIVER;
  }
  const uint64_t t0 = now_ns();
  size_t done_maps = 0;  // handles take[0 .. done_maps) are mapped
  for (size_t r = 0; r < ranges && err == CUDA_SUCCESS; ++r) {
    CUdeviceptr at = range_base(seg, r) + mapped;
    for (size_t j = 0; j < n; ++j) {
      err = drv->mem_map(at + j * cb, cb, take[r * n + j]);
      pool->map_calls++;
      if (err != CUDA_SUCCESS) break;
      ++done_maps;
    }
    if (err == CUDA_SUCCESS) {
      const uint64_t ta = now_ns();
      err = drv->set_access_rw(at, n * cb);
      pool->access_ns += now_ns() - ta;
      pool->set_access_calls++;
    }
  }
  pool->map_ns += now_ns() - t0;
  if (err != CUDA_SUCCESS) {
    set_last_driver_error(err);
    for (size_t i = 0; i < done_maps; ++i) {
      size_t r = i / n, j = i % n;
      drv->mem_unmap(range_base(seg, r) + mapped + j * cb, cb);
      pool->unmap_calls++;
    }
    std::lock_guard<std::mutex> g(pool->mu);
    pool->free_list.insert(pool->free_list.end(), take.begin(), take.end());
    return VT_ERR_DRIVER;
  }
  std::lock_guard<std::mutex> g(seg->mu);
  for (size_t r = 0; r < ranges; ++r)
    seg->chunks[r].insert(seg->chunks[r].end(), take.begin() + r * n, take.begin() + (r + 1) * n);
  seg->mapped = mapped + n * cb;
  return VT_OK;
}

static void worker_main(vt_pool *pool) {
  pool->drv->bind_thread();
  for (;;) {
    vt_pool::Request rq;
    {
      std::unique_lock<std::mutex> lk(pool->qmu);
      pool->qcv.wait(lk, [&] { return pool->stop || !pool->queue.empty(); });
      if (pool->queue.empty()) return;  // stop requested and drained
      rq = pool->queue.front();
      pool->queue.pop_front();
    }
    vt_seg *seg = rq.seg;
    int st = VT_OK;
    bool ran = false;
    {
      std::lock_guard<std::mutex> op(seg->op_mu);
      bool stale;
      { std::lock_guard<std::mutex> g(seg->mu); stale = rq.epoch != seg->epoch; }
      if (!stale) { st = grow_chunks(seg, static_cast<size_t>(rq.n_chunks)); ran = true; }
    }
    if (ran) { if (st == VT_OK) pool->async_completed++; else pool->async_failed++; }
    {
      std::lock_guard<std::mutex> g(seg->mu);
      if (ran) seg->async_status = st;
      seg->pending--;
      // Notify under the lock: vt_seg_destroy may delete the segment as soon as
      // it observes pending == 0.
      seg->cv.notify_all();
    }
  }
}

}  // namespace vt

using vt::Driver;

extern "C" {

int vt_last_driver_error(void) { return vt::last_driver_error(); }

int vt_use_mock_driver(int enable) { vt::g_use_mock.store(enable != 0); return VT_OK; }
int vt_mock_fail_nth(const char *call, int nth) {
  if (!call) return VT_ERR_INVALID;
  vt::mock_fail_nth(call, nth);
  return VT_OK;
}
int vt_mock_map_delay_us(int us) { vt::mock_map_delay_us(us); return VT_OK; }

int vt_pool_create(int device, size_t n_chunks, size_t chunk_bytes, vt_pool **out) {
  if (!out || device < 0) return VT_ERR_INVALID;
  *out = nullptr;
  if (chunk_bytes == 0) chunk_bytes = 2u << 20;
  Driver *drv = nullptr;
  if (vt::g_use_mock.load()) {
    drv = vt::make_mock_driver();
  } else {
    std::string why;
    drv = vt::make_real_driver(&why);
    if (!drv) return VT_ERR_NO_DRIVER;
  }
  CUresult r = drv->init(device);
  size_t gran = 0;
  if (r == CUDA_SUCCESS) r = drv->granularity(&gran);
  if (r != CUDA_SUCCESS) { vt::set_last_driver_error(r); delete drv; return VT_ERR_DRIVER; }
  if (gran == 0 || chunk_bytes % gran != 0) { delete drv; return VT_ERR_INVALID; }
  vt_pool *p = new (std::nothrow) vt_pool;
  if (!p) { delete drv; return VT_ERR_INVALID; }
  p->drv = drv;
  p->device = device;
  p->chunk_bytes = chunk_bytes;
  p->free_list.reserve(n_chunks);
  for (size_t i = 0; i < n_chunks; ++i) {
    CUmemGenericAllocationHandle h;
    r = drv->mem_create(&h, chunk_bytes);
    if (r != CUDA_SUCCESS) {
      vt::set_last_driver_error(r);
      for (auto hh : p->free_list) drv->mem_release(hh);
      delete p;
      delete drv;
      return VT_ERR_DRIVER;
    }
    p->free_list.push_back(h);
  }
  p->total = n_chunks;
  p->worker = std::thread(vt::worker_main, p);
  *out = p;
  return VT_OK;
}

int vt_pool_destroy(vt_pool *pool) {
  if (!pool) return VT_ERR_INVALID;
  if (pool->segments.load() != 0 || pool->tables.load() != 0) return VT_ERR_STATE;
  {
    std::lock_guard<std::mutex> g(pool->qmu);
    pool->stop = true;
  }
  pool->qcv.notify_all();
  if (pool->worker.joinable()) pool->worker.join();
  pool->drv->bind_thread();
  int st = VT_OK;
  for (auto h : pool->free_list) {
    CUresult r = pool->drv->mem_release(h);
    if (r != CUDA_SUCCESS) { vt::set_last_driver_error(r); st = VT_ERR_DRIVER; }
  }
  delete pool->drv;
  delete pool;
  return st;
}

int vt_pool_free_chunks(vt_pool *pool, size_t *out) {
  if (!pool || !out) return VT_ERR_INVALID;
  std::lock_guard<std::mutex> g(pool->mu);
  *out = pool->free_list.size();
  return VT_OK;
}

int vt_pool_stats(vt_pool *pool, vt_stats *out) {
  if (!pool || !out) return VT_ERR_INVALID;
  std::memset(out, 0, sizeof(*out));
  { std::lock_guard<std::mutex> g(pool->mu); out->chunks_free = pool->free_list.size(); }
  out->chunks_total = pool->total;
  out->chunk_bytes = pool->chunk_bytes;
  out->map_calls = pool->map_calls;
  out->unmap_calls = pool->unmap_calls;
  out->set_access_calls = pool->set_access_calls;
  out->map_ns = pool->map_ns;
  out->access_ns = pool->access_ns;
  out->async_requests = pool->async_requests;
  out->async_completed = pool->async_completed;
  out->async_failed = pool->async_failed;
  out->segments = static_cast<uint64_t>(pool->segments.load());
  return VT_OK;
}

int vt_seg_create(vt_pool *pool, int n_layers, size_t reserve_bytes, size_t premap_bytes, vt_seg **out) {
  if (!pool || !out || n_layers <= 0 || reserve_bytes == 0) return VT_ERR_INVALID;
  *out = nullptr;
  const size_t cb = pool->chunk_bytes;
  const size_t reserve = (reserve_bytes + cb - 1) / cb * cb;
  if (premap_bytes > reserve) return VT_ERR_RESERVE;
  VT_DRV(pool, pool->drv->bind_thread());
  vt_seg *s = new (std::nothrow) vt_seg;
  if (!s) return VT_ERR_INVALID;
  s->pool = pool;
  s->n_layers = n_layers;
  s->reserve = reserve;
  s->chunks.resize(2 * static_cast<size_t>(n_layers));
  CUresult r = pool->drv->address_reserve(&s->base, reserve * 2 * n_layers, cb);
  if (r != CUDA_SUCCESS) { vt::set_last_driver_error(r); delete s; return VT_ERR_DRIVER; }
  pool->segments++;
  if (premap_bytes) {
    int st;
    { std::lock_guard<std::mutex> op(s->op_mu); st = vt::grow_chunks(s, (premap_bytes + cb - 1) / cb); }
    if (st != VT_OK) { vt_seg_destroy(s); return st; }
  }
  *out = s;
  return VT_OK;
}

static int release_locked(vt_seg *seg, size_t keep_bytes) {  // caller holds op_mu
  vt_pool *pool = seg->pool;
  const size_t cb = pool->chunk_bytes;
  size_t keep = (keep_bytes + cb - 1) / cb * cb;
  size_t mapped;
  {
    std::lock_guard<std::mutex> g(seg->mu);
    seg->epoch++;  // drops growths still queued for the old occupant of the slot
    seg->used = 0;
    mapped = seg->mapped;
  }
  if (keep >= mapped) return VT_OK;
  VT_DRV(pool, pool->drv->bind_thread());
  const size_t keep_chunks = keep / cb;
  int st = VT_OK;
  std::vector<CUmemGenericAllocationHandle> back;
  for (size_t r = 0; r < seg->chunks.size(); ++r) {
    // a range that an earlier, partly failed release already cut back
    if (seg->chunks[r].size() <= keep_chunks) continue;
    CUresult e = pool->drv->mem_unmap(vt::range_base(seg, r) + keep, seg->chunks[r].size() * cb - keep);
    pool->unmap_calls++;
    if (e != CUDA_SUCCESS) { vt::set_last_driver_error(e); st = VT_ERR_DRIVER; break; }
    std::lock_guard<std::mutex> g(seg->mu);
    auto &v = seg->chunks[r];
    // LIFO hand-back so the most recently touched chunks are reused first
    for (size_t j = v.size(); j > keep_chunks; --j) back.push_back(v[j - 1]);
    v.resize(keep_chunks);
  }
  {
    std::lock_guard<std::mutex> g(pool->mu);
    pool->free_list.insert(pool->free_list.end(), back.begin(), back.end());
  }
  {
    // On failure the ranges before the failing one are already cut back to `keep`
    // while the others still reach `mapped`: the segment stays unusable for growth,
    // bookkeeping and table fills until a later release or destroy gets through.
    std::lock_guard<std::mutex> g(seg->mu);
    seg->poisoned = st != VT_OK;
    if (st == VT_OK) seg->mapped = keep;
  }
  return st;
}

int vt_seg_release(vt_seg *seg, size_t keep_bytes) {
  if (!seg) return VT_ERR_INVALID;
  std::lock_guard<std::mutex> op(seg->op_mu);
  return release_locked(seg, keep_bytes);
}

int vt_seg_destroy(vt_seg *seg) {
  if (!seg) return VT_ERR_INVALID;
  vt_pool *pool = seg->pool;
  int st;
  {
    std::lock_guard<std::mutex> op(seg->op_mu);
    st = release_locked(seg, 0);
  }
  {  // queued growths were made stale above; wait until the worker has dropped them
    std::unique_lock<std::mutex> lk(seg->mu);
    seg->cv.wait(lk, [&] { return seg->pending == 0; });
  }
  if (st != VT_OK) return st;  // still mapped: keep the object alive rather than leak silently
  CUresult r = pool->drv->address_free(seg->base, seg->reserve * 2 * seg->n_layers);
  if (r != CUDA_SUCCESS) { vt::set_last_driver_error(r); return VT_ERR_DRIVER; }
  pool->segments--;
  delete seg;
  return VT_OK;
}

int vt_seg_k_ptr(vt_seg *seg, int layer, uint64_t *dptr) {
  if (!seg || !dptr || layer < 0 || layer >= seg->n_layers) return VT_ERR_INVALID;
  *dptr = vt::range_base(seg, 2 * static_cast<size_t>(layer));
  return VT_OK;
}
int vt_seg_v_ptr(vt_seg *seg, int layer, uint64_t *dptr) {
  if (!seg || !dptr || layer < 0 || layer >= seg->n_layers) return VT_ERR_INVALID;
  *dptr = vt::range_base(seg, 2 * static_cast<size_t>(layer) + 1);
  return VT_OK;
}
int vt_seg_used(vt_seg *seg, size_t *bytes) {
  if (!seg || !bytes) return VT_ERR_INVALID;
  std::lock_guard<std::mutex> g(seg->mu);
  *bytes = seg->used;
  return VT_OK;
}
int vt_seg_set_used(vt_seg *seg, size_t bytes) {
  if (!seg) return VT_ERR_INVALID;
  std::lock_guard<std::mutex> g(seg->mu);
  if (bytes > seg->reserve) return VT_ERR_RESERVE;
  seg->used = bytes;
  return VT_OK;
}
int vt_seg_mapped(vt_seg *seg, size_t *bytes) {
  if (!seg || !bytes) return VT_ERR_INVALID;
  std::lock_guard<std::mutex> g(seg->mu);
  *bytes = seg->mapped;
  return VT_OK;
}
int vt_seg_reserved(vt_seg *seg, size_t *bytes) {
  if (!seg || !bytes) return VT_ERR_INVALID;
  *bytes = seg->reserve;
  return VT_OK;
}

int vt_seg_grow(vt_seg *seg, size_t bytes_needed) {
  if (!seg) return VT_ERR_INVALID;
  if (bytes_needed > seg->reserve) return VT_ERR_RESERVE;
  std::lock_guard<std::mutex> op(seg->op_mu);
  size_t mapped;
  { std::lock_guard<std::mutex> g(seg->mu); mapped = seg->mapped; }
  if (bytes_needed <= mapped) return VT_OK;
  const size_t cb = seg->pool->chunk_bytes;
  return vt::grow_chunks(seg, (bytes_needed - mapped + cb - 1) / cb);
}

int vt_seg_grow_async(vt_seg *seg, int n_chunks) {
  if (!seg || n_chunks <= 0) return VT_ERR_INVALID;
  vt_pool *pool = seg->pool;
  uint64_t epoch;
  {
    std::lock_guard<std::mutex> g(seg->mu);
    // Early answer for the common mistake; the worker re-checks against the
    // frontier it finds when the request runs.
    if (seg->mapped + static_cast<size_t>(n_chunks) * pool->chunk_bytes > seg->reserve) return VT_ERR_RESERVE;
    seg->pending++;
    epoch = seg->epoch;
  }
  {
    std::lock_guard<std::mutex> g(pool->qmu);
    pool->queue.push_back({seg, n_chunks, epoch});
  }
  pool->async_requests++;
  pool->qcv.notify_one();
  return VT_OK;
}

int vt_seg_ready(vt_seg *seg, int *ready) {
  if (!seg || !ready) return VT_ERR_INVALID;
  std::lock_guard<std::mutex> g(seg->mu);
  *ready = seg->pending == 0;
  return VT_OK;
}

int vt_seg_wait(vt_seg *seg, uint64_t timeout_us) {
  if (!seg) return VT_ERR_INVALID;
  std::unique_lock<std::mutex> lk(seg->mu);
  if (!seg->cv.wait_for(lk, std::chrono::microseconds(timeout_us), [&] { return seg->pending == 0; }))
    return VT_ERR_TIMEOUT;
  int st = seg->async_status;
  seg->async_status = VT_OK;
  return st;
}

int vt_extend_batch(vt_seg *const *segs, int n, const int64_t *set_used_tokens,
                    const uint64_t *token_bytes, uint64_t kv_size, int gen, uint64_t wait_us,
                    int64_t *out_offsets) {
  if (!segs || !token_bytes || !out_offsets || n < 0) return VT_ERR_INVALID;
  // pass 1: make sure every entry's rows fit into mapped memory
  for (int i = 0; i < n; ++i) {
    vt_seg *s = segs[i];
    if (!s) return VT_ERR_INVALID;
    size_t used, mapped;
    int pending;
    {
      std::lock_guard<std::mutex> g(s->mu);
      if (s->poisoned) return VT_ERR_STATE;
      used = (set_used_tokens && set_used_tokens[i] > 0) ? static_cast<size_t>(set_used_tokens[i]) * kv_size : s->used;
      mapped = s->mapped;
      pending = s->pending;
    }
    size_t need = used + token_bytes[i];
    if (need > s->reserve) return VT_ERR_RESERVE;
    if (need <= mapped) continue;
    if (gen && pending > 0) {  // a background growth is on its way: bounded wait
      int st = vt_seg_wait(s, wait_us);
      if (st != VT_OK) return st;
    }
    int st = vt_seg_grow(s, need);  // no-op when the background growth covered it
    if (st != VT_OK) return st;
  }
  // pass 2: commit
  for (int i = 0; i < n; ++i) {
    vt_seg *s = segs[i];
    std::lock_guard<std::mutex> g(s->mu);
    if (set_used_tokens && set_used_tokens[i] > 0) s->used = static_cast<size_t>(set_used_tokens[i]) * kv_size;
    out_offsets[i] = static_cast<int64_t>(s->used);
    s->used += token_bytes[i];
  }
  return VT_OK;
}

int vt_table_create(vt_pool *pool, int n_slots, vt_table **out) {
  if (!pool || !out || n_slots <= 0) return VT_ERR_INVALID;
  *out = nullptr;
  VT_DRV(pool, pool->drv->bind_thread());
  vt_table *t = new (std::nothrow) vt_table;
  if (!t) return VT_ERR_INVALID;
  t->pool = pool;
  t->n_slots = n_slots;
  CUresult r = pool->drv->mem_alloc(&t->dptr, static_cast<size_t>(n_slots) * 8);
  if (r != CUDA_SUCCESS) { vt::set_last_driver_error(r); delete t; return VT_ERR_DRIVER; }
  std::vector<uint64_t> zero(n_slots, 0);
  r = pool->drv->memcpy_htod(t->dptr, zero.data(), zero.size() * 8);
  if (r != CUDA_SUCCESS) { vt::set_last_driver_error(r); pool->drv->mem_free(t->dptr); delete t; return VT_ERR_DRIVER; }
  pool->tables++;
  *out = t;
  return VT_OK;
}

int vt_table_destroy(vt_table *tbl) {
  if (!tbl) return VT_ERR_INVALID;
  vt_pool *pool = tbl->pool;
  VT_DRV(pool, pool->drv->bind_thread());
  VT_DRV(pool, pool->drv->mem_free(tbl->dptr));
  pool->tables--;
  delete tbl;
  return VT_OK;
}

int vt_table_set(vt_table *tbl, int slot, uint64_t dptr) {
  if (!tbl || slot < 0 || slot >= tbl->n_slots) return VT_ERR_INVALID;
  VT_DRV(tbl->pool, tbl->pool->drv->bind_thread());
  VT_DRV(tbl->pool, tbl->pool->drv->memcpy_htod(tbl->dptr + static_cast<size_t>(slot) * 8, &dptr, 8));
  return VT_OK;
}

int vt_table_fill(vt_table *k_tbl, vt_table *v_tbl, vt_seg *const *segs, int n, int layer) {
  if (!k_tbl || !v_tbl || !segs || n < 0 || n > k_tbl->n_slots || n > v_tbl->n_slots) return VT_ERR_INVALID;
  std::vector<uint64_t> k(n), v(n);
  for (int i = 0; i < n; ++i) {
    int st = vt_seg_k_ptr(segs[i], layer, &k[i]);
    if (st == VT_OK) st = vt_seg_v_ptr(segs[i], layer, &v[i]);
    if (st != VT_OK) return st;
  }
  if (n == 0) return VT_OK;
  VT_DRV(k_tbl->pool, k_tbl->pool->drv->bind_thread());
  VT_DRV(k_tbl->pool, k_tbl->pool->drv->memcpy_htod(k_tbl->dptr, k.data(), k.size() * 8));
  VT_DRV(v_tbl->pool, v_tbl->pool->drv->memcpy_htod(v_tbl->dptr, v.data(), v.size() * 8));
  return VT_OK;
}

int vt_pool_read(vt_pool *pool, void *dst_host, uint64_t src_dptr, size_t bytes) {
  if (!pool || !dst_host || !src_dptr) return VT_ERR_INVALID;
  VT_DRV(pool, pool->drv->bind_thread());
  VT_DRV(pool, pool->drv->memcpy_dtoh(dst_host, src_dptr, bytes));
  return VT_OK;
}

int vt_pool_write(vt_pool *pool, uint64_t dst_dptr, const void *src_host, size_t bytes) {
  if (!pool || !src_host || !dst_dptr) return VT_ERR_INVALID;
  VT_DRV(pool, pool->drv->bind_thread());
  VT_DRV(pool, pool->drv->memcpy_htod(dst_dptr, src_host, bytes));
  return VT_OK;
}

int vt_table_dptr(vt_table *tbl, uint64_t *dptr) {
  if (!tbl || !dptr) return VT_ERR_INVALID;
  *dptr = tbl->dptr;
  return VT_OK;
}

}  // extern "C"
