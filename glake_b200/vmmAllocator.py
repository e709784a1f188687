"""Drop-in for the reference's pybind11 module ``vmmAllocator``
(GLakeServe/vmm_allocator/vmm_allocator.h:190-219): same function and class
names, argument order and return types, implemented on libvtensor's C ABI.

Differences a caller can observe, all deliberate:
* state is per process (no ``/my_shm`` POSIX segment shared by every process on
  the machine, vmm_allocator.cpp:114-133), and the slot count is not capped at 1000;
* driver failures raise ``VTensorError`` instead of printing and ``assert(0)``
  (vmm_allocator.h:19-42); ``init_physical_handle`` still returns ``False`` on failure;
* a decode-step ``extend_kv_cache_batch`` whose rows would land in unmapped memory
  first waits (bounded) for the slot's pending background growth and otherwise
  maps synchronously, where the reference would let the kernel fault.
"""
import ctypes
from ctypes import byref, c_int, c_int64, c_size_t, c_uint64, c_void_p

from ._lib import VT_ERR_TIMEOUT, VTensorError, check, lib

granularitySize = 2 * 1024 * 1024  # vmm_allocator.h:45
WAIT_US = 2_000_000                # bound of every wait for a background growth

_pool = None
_slot_registry = {}  # slot id -> (segment, token_bytes) of the last eagerExtend


def _require_pool():
    if _pool is None:
        raise RuntimeError("vmmAllocator.init_physical_handle has not been called")
    return _pool


def set_chunk_bytes(nbytes):
    """Size of a physical chunk for pools created from now on (default 2 MiB, the reference's
    ``granularitySize``, vmm_allocator.h:45): a multiple of 2 MiB.  The driver's cost of a growth is
    per CHUNK, not per byte (measured on B200: cuMemCreate 0.075 ms and cuMemSetAccess 0.15 ms per
    handle whether it holds 2 or 32 MiB), so 8 MiB chunks make pool creation and growth 4 x cheaper
    per byte at the price of up to 8 MiB of slack per range.  Only while no pool exists.  Updates
    ``granularitySize`` here and the copy the host-side accounting (``chunk_manager.PHY_GRAN``) keeps."""
    from . import chunk_manager
    global granularitySize
    nbytes = int(nbytes)
    if _pool is not None:
        raise RuntimeError("set_chunk_bytes: a pool exists already (call shutdown first)")
    if nbytes <= 0 or nbytes % (2 * 1024 * 1024) != 0:
        raise ValueError("chunk size must be a positive multiple of 2 MiB")
    granularitySize = nbytes
    chunk_manager.PHY_GRAN = nbytes


def init_physical_handle(num_blocks, device_id):
    """Pre-creates ``num_blocks`` physical chunks (2 MiB unless :func:`set_chunk_bytes` said otherwise) on ``device_id`` and starts
    the growth worker (vmm_allocator.cpp:113-151).  Calling it again adds a fresh
    pool only if the previous one was shut down with :func:`shutdown`."""
    global _pool
    if _pool is not None:
        return True
    h = c_void_p()
    st = lib.vt_pool_create(int(device_id if device_id >= 0 else 0), int(num_blocks), granularitySize, byref(h))
    if st != 0:
        return False
    _pool = h
    return True


def shutdown():
    """Releases the pool (no counterpart in the reference, which never frees)."""
    global _pool
    if _pool is not None:
        check(lib.vt_pool_destroy(_pool), "vt_pool_destroy")
        _pool = None
        _slot_registry.clear()


def showFreeBlocks():
    n = c_size_t()
    check(lib.vt_pool_free_chunks(_require_pool(), byref(n)), "vt_pool_free_chunks")
    return n.value


def stats():
    from ._lib import Stats
    s = Stats()
    check(lib.vt_pool_stats(_require_pool(), byref(s)), "vt_pool_stats")
    return {k: getattr(s, k) for k, _ in Stats._fields_}


class KVCache:
    """Device array of per-slot base addresses (vmm_allocator.cpp:458-470)."""

    def __init__(self, num_seqs):
        self.num_seqs = num_seqs
        self._h = c_void_p()
        check(lib.vt_table_create(_require_pool(), int(num_seqs), byref(self._h)), "vt_table_create")
        p = c_uint64()
        check(lib.vt_table_dptr(self._h, byref(p)), "vt_table_dptr")
        self.kv_cache_ptr = p.value

    def getKVCachePtr(self):
        return self.kv_cache_ptr

    def AddKVCache(self, slot, dptr):
        check(lib.vt_table_set(self._h, int(slot), int(dptr)), "vt_table_set")

    def close(self):
        if self._h:
            check(lib.vt_table_destroy(self._h), "vt_table_destroy")
            self._h = None


class KVcacheSegment:
    """One sequence slot's K and V ranges for every layer (vmm_allocator.cpp:177-211)."""

    def __init__(self, layer_num, context_max_size, expand_size, expand):
        self.layer_num = layer_num
        self.context_max_size = context_max_size
        self.expand_size = expand_size
        self._h = c_void_p()
        premap = expand_size if expand else 0
        check(lib.vt_seg_create(_require_pool(), int(layer_num), int(context_max_size), int(premap), byref(self._h)),
              "vt_seg_create")

    # -- pointers ------------------------------------------------------
    def getKeyDevicePtr(self, layer_index):
        p = c_uint64()
        check(lib.vt_seg_k_ptr(self._h, int(layer_index), byref(p)), "vt_seg_k_ptr")
        return p.value

    def getValueDevicePtr(self, layer_index):
        p = c_uint64()
        check(lib.vt_seg_v_ptr(self._h, int(layer_index), byref(p)), "vt_seg_v_ptr")
        return p.value

    # -- fill ----------------------------------------------------------
    def get_used_slot(self):
        n = c_size_t()
        check(lib.vt_seg_used(self._h, byref(n)), "vt_seg_used")
        return n.value

    def set_used_size(self, used_size):
        check(lib.vt_seg_set_used(self._h, int(used_size)), "vt_seg_set_used")

    @property
    def used_size(self):
        return self.get_used_slot()

    @property
    def actual_size(self):
        n = c_size_t()
        check(lib.vt_seg_mapped(self._h, byref(n)), "vt_seg_mapped")
        return n.value

    # -- growth --------------------------------------------------------
    def expandMultiSegment(self, expand_num):
        """Synchronous growth by ``expand_num`` chunks per range (vmm_allocator.cpp:214-297)."""
        st = lib.vt_seg_grow(self._h, self.actual_size + int(expand_num) * granularitySize)
        return st == 0

    def ensure_mapped(self, nbytes):
        """Synchronous growth until at least ``nbytes`` of every range are mapped (whole
        chunks); no-op when they already are.  Used at admission to map a sequence's
        logical reservation (prompt + headroom) in one go."""
        check(lib.vt_seg_grow(self._h, int(nbytes)), "vt_seg_grow")

    def eagerExtend(self, token_size, seq_id):
        """Queue one chunk per range on the worker thread (vmm_allocator.cpp:307-320)."""
        _slot_registry[int(seq_id)] = (self, int(token_size))
        if self.context_max_size > self.actual_size:
            check(lib.vt_seg_grow_async(self._h, 1), "vt_seg_grow_async")

    def copy_kv_cache(self, token_size, kv_size):
        """Prefill-side growth + advance (vmm_allocator.cpp:322-337)."""
        used = self.get_used_slot()
        check(lib.vt_seg_grow(self._h, used + int(token_size)), "vt_seg_grow")
        self.set_used_size(used + int(token_size))

    def ready(self):
        r = c_int()
        check(lib.vt_seg_ready(self._h, byref(r)), "vt_seg_ready")
        return bool(r.value)

    def wait(self, timeout_us=WAIT_US):
        check(lib.vt_seg_wait(self._h, int(timeout_us)), "vt_seg_wait")

    # -- lifecycle -----------------------------------------------------
    def release_seq(self, seq_id):
        """End of sequence: keep the pre-cached ``expand_size`` prefix mapped when
        the slot has at least that much, else unmap everything
        (vmm_allocator.cpp:383-421)."""
        _slot_registry.pop(int(seq_id), None)
        keep = self.expand_size if self.actual_size >= self.expand_size else 0
        check(lib.vt_seg_release(self._h, int(keep)), "vt_seg_release")

    def preempt_seq(self, seq_id):
        """Unmap everything (vmm_allocator.cpp:348-381)."""
        _slot_registry.pop(int(seq_id), None)
        check(lib.vt_seg_release(self._h, 0), "vt_seg_release")

    def write_string(self, data):
        """Debug helper (vmm_allocator.cpp:423-433): copies the bytes of ``data`` to the
        fill position of layer 0's K range and advances the fill.  The target must be mapped."""
        raw = data.encode() if isinstance(data, str) else bytes(data)
        used = self.get_used_slot()
        if used + len(raw) > self.actual_size:
            raise RuntimeError("write_string: beyond the mapped part of the range")
        if raw:
            buf = ctypes.create_string_buffer(raw, len(raw))
            check(lib.vt_pool_write(_require_pool(), self.getKeyDevicePtr(0) + used, buf, len(raw)), "vt_pool_write")
            self.set_used_size(used + len(raw))

    def read_string(self):
        """Debug helper (vmm_allocator.cpp:435-446): prints layer 0's K range up to the fill
        position, as the reference does, and also returns it."""
        used = self.get_used_slot()
        buf = ctypes.create_string_buffer(max(used, 1))
        if used:
            check(lib.vt_pool_read(_require_pool(), buf, self.getKeyDevicePtr(0), used), "vt_pool_read")
        text = buf.raw[:used].decode(errors="replace")
        print(text)
        return text

    def show_info(self, seq_id):
        return [int(seq_id), self.actual_size, self.get_used_slot(), int(self.ready()), 0]

    def close(self):
        if self._h:
            for slot in [k for k, (seg, _) in _slot_registry.items() if seg is self]:
                del _slot_registry[slot]
            check(lib.vt_seg_destroy(self._h), "vt_seg_destroy")
            self._h = None


def _seg_array(segments):
    arr = (c_void_p * len(segments))()
    for i, s in enumerate(segments):
        arr[i] = s._h
    return arr


def extend_kv_cache_batch(k_cache_batch, v_cache_batch, slot_mapping, token_size, segment, set_used_size,
                          kv_size, gen):
    """Per-step bookkeeping (vmm_allocator.h:138-168): returns each entry's byte
    offset and advances its fill; prefill (``gen`` false) also maps what it needs."""
    n = len(slot_mapping)
    out = (c_int64 * n)()
    su = (c_int64 * n)(*[int(x) for x in set_used_size]) if set_used_size is not None else None
    tb = (c_uint64 * n)(*[int(x) for x in token_size])
    check(lib.vt_extend_batch(_seg_array(segment), n, su, tb, int(kv_size), 1 if gen else 0, WAIT_US, out),
          "vt_extend_batch")
    return list(out)


def copy_kv_cache(k_cache_batch, v_cache_batch, segment):
    """Fill every layer's K/V pointer table, table index = position in ``segment``
    (vmm_allocator.h:170-182)."""
    segs = _seg_array(segment)
    for layer, (k, v) in enumerate(zip(k_cache_batch, v_cache_batch)):
        check(lib.vt_table_fill(k._h, v._h, segs, len(segment), layer), "vt_table_fill")


def query_shm(seq_ids):
    """True when no listed slot has a background growth in flight (vmm_allocator.cpp:85-92)."""
    return all(_slot_registry[s][0].ready() for s in seq_ids if s in _slot_registry)


def query_cycle(seq_ids):
    """True when the caller has to wait now: some listed slot's next row would not
    fit into what is mapped and its growth has not finished.  (The reference
    counts 100 calls down before it starts checking, vmm_allocator.cpp:95-103.)"""
    for s in seq_ids:
        ent = _slot_registry.get(s)
        if ent is None:
            continue
        seg, tok = ent
        if not seg.ready() and seg.get_used_slot() + tok > seg.actual_size:
            return True
    return False


def wait_ready(seq_ids, timeout_us=WAIT_US):
    """Bounded replacement for ``while not query_shm(...)`` (llama.py:324-325)."""
    for s in seq_ids:
        ent = _slot_registry.get(s)
        if ent is not None:
            ent[0].wait(timeout_us)


def query_unmap(seq_ids):
    """Per slot: True when no unmap of it is in flight (vmm_allocator.cpp:105-111 returns
    ``!unmap_ptr[slot]``, a flag the reference initialises to 0 and never sets).  Here
    ``release_seq`` / ``preempt_seq`` unmap synchronously before they return, so there is
    never one in flight by the time a caller can ask."""
    return [True for _ in seq_ids]


def print_shm_state(seq_ids):
    return [int(_slot_registry[s][0].ready()) if s in _slot_registry else 1 for s in seq_ids]
