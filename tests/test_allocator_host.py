"""Host-side tests of the VMM allocator against the in-process mock driver:
growth, release-to-watermark, preempt, pool exhaustion, reserve overflow,
failure injection with rollback, the bounded wait, and the decode/prefill
bookkeeping compared with a Python restatement of the reference's
extend_kv_cache_batch (GLakeServe/vmm_allocator/vmm_allocator.h:138-168)."""
import ctypes
import threading
from ctypes import byref, c_int, c_int64, c_size_t, c_uint64, c_void_p

import pytest

from glake_b200 import _lib
from glake_b200._lib import lib

MiB = 1 << 20
CH = 2 * MiB


@pytest.fixture()
def pool():
    lib.vt_use_mock_driver(1)
    lib.vt_mock_map_delay_us(0)
    h = c_void_p()
    assert lib.vt_pool_create(0, 64, 0, byref(h)) == 0
    yield h
    st = lib.vt_pool_destroy(h)
    lib.vt_use_mock_driver(0)
    assert st == 0


def free_chunks(pool):
    n = c_size_t()
    assert lib.vt_pool_free_chunks(pool, byref(n)) == 0
    return n.value


def seg_create(pool, layers, reserve, premap=0):
    s = c_void_p()
    st = lib.vt_seg_create(pool, layers, reserve, premap, byref(s))
    return st, s


def mapped(s):
    n = c_size_t()
    assert lib.vt_seg_mapped(s, byref(n)) == 0
    return n.value


def used(s):
    n = c_size_t()
    assert lib.vt_seg_used(s, byref(n)) == 0
    return n.value


def test_layout_k_v_ranges_are_disjoint_and_chunk_aligned(pool):
    st, s = seg_create(pool, 3, 5 * MiB)  # rounds up to 6 MiB per range
    assert st == 0
    r = c_size_t()
    lib.vt_seg_reserved(s, byref(r))
    assert r.value == 6 * MiB
    ptrs = []
    for layer in range(3):
        k, v = c_uint64(), c_uint64()
        assert lib.vt_seg_k_ptr(s, layer, byref(k)) == 0 and lib.vt_seg_v_ptr(s, layer, byref(v)) == 0
        ptrs += [k.value, v.value]
    assert all(p % CH == 0 for p in ptrs)
    assert ptrs == sorted(ptrs) and all(b - a == 6 * MiB for a, b in zip(ptrs, ptrs[1:]))
    assert lib.vt_seg_k_ptr(s, 3, byref(c_uint64())) == _lib.VT_ERR_INVALID
    assert lib.vt_seg_destroy(s) == 0


def test_grow_release_preempt_accounting(pool):
    st, s = seg_create(pool, 2, 16 * MiB, premap=2 * MiB)
    assert st == 0 and mapped(s) == CH and free_chunks(pool) == 64 - 4
    assert lib.vt_seg_grow(s, 5 * MiB) == 0          # -> 3 chunks per range
    assert mapped(s) == 3 * CH and free_chunks(pool) == 64 - 12
    assert lib.vt_seg_grow(s, 1) == 0 and mapped(s) == 3 * CH   # already covered
    lib.vt_seg_set_used(s, 4 * MiB)
    assert lib.vt_seg_release(s, 2 * MiB) == 0        # keep the pre-cached prefix
    assert mapped(s) == CH and used(s) == 0 and free_chunks(pool) == 64 - 4
    assert lib.vt_seg_release(s, 0) == 0              # preempt
    assert mapped(s) == 0 and free_chunks(pool) == 64
    assert lib.vt_seg_release(s, 0) == 0              # double release is harmless
    st = _lib.Stats()
    lib.vt_pool_stats(pool, byref(st))
    assert st.map_calls == 12 and st.set_access_calls == 8 and st.unmap_calls == 8 and st.segments == 1
    assert lib.vt_pool_destroy(pool) == _lib.VT_ERR_STATE   # live segment
    assert lib.vt_seg_destroy(s) == 0


def test_pool_exhaustion_and_reserve_overflow(pool):
    st, a = seg_create(pool, 4, 64 * MiB)
    assert st == 0
    assert lib.vt_seg_grow(a, 7 * CH) == 0 and free_chunks(pool) == 64 - 56
    # 8 chunks left, next growth of one chunk per range needs 8: ok; then empty
    assert lib.vt_seg_grow(a, 8 * CH) == 0 and free_chunks(pool) == 0
    assert lib.vt_seg_grow(a, 9 * CH) == _lib.VT_ERR_POOL_EMPTY
    assert mapped(a) == 8 * CH                         # nothing half-done
    assert lib.vt_seg_grow(a, 65 * MiB) == _lib.VT_ERR_RESERVE
    st, b = seg_create(pool, 1, 4 * MiB, premap=6 * MiB)
    assert st == _lib.VT_ERR_RESERVE
    st, b = seg_create(pool, 1, 4 * MiB, premap=2 * MiB)
    assert st == _lib.VT_ERR_POOL_EMPTY                # and the failed create left nothing behind
    assert lib.vt_seg_destroy(a) == 0 and free_chunks(pool) == 64


@pytest.mark.parametrize("call,nth", [("cuMemMap", 3), ("cuMemSetAccess", 2), ("cuMemMap", 1)])
def test_injected_driver_failure_rolls_back(pool, call, nth):
    st, s = seg_create(pool, 2, 16 * MiB, premap=CH)
    assert st == 0
    before = free_chunks(pool)
    lib.vt_mock_fail_nth(call.encode(), nth)
    assert lib.vt_seg_grow(s, 3 * CH) == _lib.VT_ERR_DRIVER
    assert lib.vt_last_driver_error() != 0
    assert mapped(s) == CH and free_chunks(pool) == before
    # the same growth succeeds afterwards: the rollback unmapped what it had mapped
    assert lib.vt_seg_grow(s, 3 * CH) == 0 and mapped(s) == 3 * CH
    assert lib.vt_seg_destroy(s) == 0


def test_failed_unmap_poisons_the_segment_until_a_release_gets_through(pool):
    """A cuMemUnmap that fails part-way through a release leaves some ranges cut back
    and others not: no growth or row bookkeeping may succeed on that slot (a later
    growth at the stale frontier would leave an unmapped hole that kernels would
    read), and a second release or destroy finishes the job with every chunk back."""
    st, s = seg_create(pool, 2, 16 * MiB)
    assert st == 0 and lib.vt_seg_grow(s, 3 * CH) == 0 and free_chunks(pool) == 64 - 12
    lib.vt_mock_fail_nth(b"cuMemUnmap", 3)                      # ranges 0 and 1 succeed, range 2 fails
    assert lib.vt_seg_release(s, CH) == _lib.VT_ERR_DRIVER
    assert free_chunks(pool) == 64 - 12 + 4                     # two ranges handed two chunks back each
    assert lib.vt_seg_grow(s, 4 * CH) == _lib.VT_ERR_STATE
    assert lib.vt_seg_grow_async(s, 1) == 0 and lib.vt_seg_wait(s, 1_000_000) == _lib.VT_ERR_STATE
    out = (c_int64 * 1)()
    segs = (c_void_p * 1)(s)
    tb = (c_uint64 * 1)(8192)
    assert lib.vt_extend_batch(segs, 1, None, tb, 8192, 1, 1000, out) == _lib.VT_ERR_STATE
    assert lib.vt_seg_release(s, 0) == 0                        # a different watermark than the failed attempt
    assert mapped(s) == 0 and free_chunks(pool) == 64
    assert lib.vt_seg_grow(s, 2 * CH) == 0 and mapped(s) == 2 * CH   # usable again
    assert lib.vt_seg_destroy(s) == 0 and free_chunks(pool) == 64


def test_pool_create_failure_is_reported():
    lib.vt_use_mock_driver(1)
    lib.vt_mock_fail_nth(b"cuMemCreate", 5)
    h = c_void_p()
    assert lib.vt_pool_create(0, 16, 0, byref(h)) == _lib.VT_ERR_DRIVER and not h.value
    lib.vt_use_mock_driver(0)


def test_async_growth_ready_flag_and_bounded_wait(pool):
    st, s = seg_create(pool, 2, 16 * MiB)
    assert st == 0
    lib.vt_mock_map_delay_us(50_000)                   # 4 maps x 50 ms
    assert lib.vt_seg_grow_async(s, 1) == 0
    r = c_int()
    lib.vt_seg_ready(s, byref(r))
    assert r.value == 0
    assert lib.vt_seg_wait(s, 1_000) == _lib.VT_ERR_TIMEOUT   # bounded: gives up, no hang
    assert lib.vt_seg_wait(s, 5_000_000) == 0
    lib.vt_seg_ready(s, byref(r))
    assert r.value == 1 and mapped(s) == CH
    lib.vt_mock_map_delay_us(0)
    # background failure is reported by the next wait, and nothing is half-mapped
    lib.vt_mock_fail_nth(b"cuMemMap", 2)
    assert lib.vt_seg_grow_async(s, 1) == 0
    assert lib.vt_seg_wait(s, 5_000_000) == _lib.VT_ERR_DRIVER
    assert mapped(s) == CH
    assert lib.vt_seg_grow_async(s, 100) == _lib.VT_ERR_RESERVE
    assert lib.vt_seg_destroy(s) == 0


def test_release_drops_queued_growths(pool):
    st, s = seg_create(pool, 1, 32 * MiB)
    assert st == 0
    lib.vt_mock_map_delay_us(20_000)
    for _ in range(4):
        assert lib.vt_seg_grow_async(s, 1) == 0
    assert lib.vt_seg_release(s, 0) == 0               # sequence finished while growths were queued
    assert lib.vt_seg_wait(s, 5_000_000) in (0,)
    lib.vt_mock_map_delay_us(0)
    assert mapped(s) <= CH                              # at most the one that was already running
    assert lib.vt_seg_destroy(s) == 0 and free_chunks(pool) == 64


def ref_extend_kv_cache_batch(state, set_used, token_size, kv_size, gen, chunk=CH):
    """Python restatement of vmm_allocator.h:138-168 on (used, mapped) pairs; the
    prefill branch maps exactly what is needed (no 100-token headroom)."""
    out = []
    for i, st in enumerate(state):
        if set_used[i] > 0:
            st["used"] = set_used[i] * kv_size
        out.append(st["used"])
        need = st["used"] + token_size[i]
        if need > st["mapped"]:
            st["mapped"] = (need + chunk - 1) // chunk * chunk
        st["used"] += token_size[i]
    return out


def test_extend_batch_matches_reference_bookkeeping(pool):
    kv = 8192                                          # 32 kv heads x 128 x bf16
    segs, state = [], []
    for _ in range(3):
        st, s = seg_create(pool, 1, 16 * MiB)
        assert st == 0
        segs.append(s)
        state.append({"used": 0, "mapped": 0})
    arr = (c_void_p * 3)(*[s for s in segs])
    out = (c_int64 * 3)()

    def call(set_used, tok, gen):
        su = (c_int64 * 3)(*set_used)
        tb = (c_uint64 * 3)(*tok)
        assert lib.vt_extend_batch(arr, 3, su, tb, kv, gen, 1_000_000, out) == 0
        want = ref_extend_kv_cache_batch(state, set_used, tok, kv, gen)
        assert list(out) == want
        assert [used(s) for s in segs] == [s["used"] for s in state]
        assert [mapped(s) for s in segs] == [s["mapped"] for s in state]

    call([0, 0, 0], [300 * kv, 1 * kv, 256 * kv], 0)            # prefill: 3 / 1 / 1 chunks
    for _ in range(5):
        call([0, 0, 0], [kv, kv, kv], 1)                          # decode steps; seq 2 crosses a chunk
    call([0, 7, 0], [kv, kv, kv], 1)                              # set_used_size rewinds entry 1 to 7 tokens
    # exceeding the reservation is an error and changes nothing
    su = (c_int64 * 3)(0, 0, 0)
    tb = (c_uint64 * 3)(kv, 17 * MiB, kv)
    before = [used(s) for s in segs]
    assert lib.vt_extend_batch(arr, 3, su, tb, kv, 1, 1000, out) == _lib.VT_ERR_RESERVE
    assert [used(s) for s in segs] == before
    for s in segs:
        assert lib.vt_seg_destroy(s) == 0


def test_decode_extend_waits_for_pending_growth(pool):
    kv = 8192
    st, s = seg_create(pool, 1, 16 * MiB, premap=CH)
    assert st == 0
    lib.vt_seg_set_used(s, CH - kv)                   # one row left in the mapped chunk
    arr = (c_void_p * 1)(s)
    out = (c_int64 * 1)()
    tb = (c_uint64 * 1)(kv)
    assert lib.vt_extend_batch(arr, 1, None, tb, kv, 1, 1000, out) == 0 and out[0] == CH - kv
    lib.vt_mock_map_delay_us(100_000)
    assert lib.vt_seg_grow_async(s, 1) == 0
    # next row needs the chunk that is still being mapped: a 1 ms budget runs out ...
    assert lib.vt_extend_batch(arr, 1, None, tb, kv, 1, 1_000, out) == _lib.VT_ERR_TIMEOUT
    assert used(s) == CH
    # ... a generous one succeeds once the worker is done
    assert lib.vt_extend_batch(arr, 1, None, tb, kv, 1, 5_000_000, out) == 0 and out[0] == CH
    lib.vt_mock_map_delay_us(0)
    assert mapped(s) == 2 * CH
    assert lib.vt_seg_destroy(s) == 0


def test_tables_hold_segment_bases(pool):
    segs = []
    for _ in range(4):
        st, s = seg_create(pool, 2, 4 * MiB)
        assert st == 0
        segs.append(s)
    kt, vt_ = c_void_p(), c_void_p()
    assert lib.vt_table_create(pool, 6, byref(kt)) == 0 and lib.vt_table_create(pool, 6, byref(vt_)) == 0
    arr = (c_void_p * 4)(*segs)
    assert lib.vt_table_fill(kt, vt_, arr, 4, 1) == 0
    assert lib.vt_table_fill(kt, vt_, arr, 4, 2) == _lib.VT_ERR_INVALID
    p = c_uint64()
    lib.vt_table_dptr(kt, byref(p))
    host = (c_uint64 * 6).from_address(p.value)        # mock tables live in host memory
    for i, s in enumerate(segs):
        k = c_uint64()
        lib.vt_seg_k_ptr(s, 1, byref(k))
        assert host[i] == k.value
    assert host[4] == 0 and host[5] == 0
    assert lib.vt_table_set(kt, 5, 0xABC000) == 0 and host[5] == 0xABC000
    assert lib.vt_table_set(kt, 6, 1) == _lib.VT_ERR_INVALID
    assert lib.vt_table_destroy(kt) == 0 and lib.vt_table_destroy(vt_) == 0
    for s in segs:
        assert lib.vt_seg_destroy(s) == 0


def test_concurrent_growth_and_release_keep_the_pool_consistent(pool):
    """Caller threads and the worker thread hammer the same pool; chunk
    conservation must hold at the end (the reference mutates its pool from both
    threads without a lock, vmm_allocator.cpp:222-228 vs :409-413)."""
    segs = []
    for _ in range(4):
        st, s = seg_create(pool, 2, 8 * MiB)
        assert st == 0
        segs.append(s)
    errors = []

    def worker(s, seed):
        for it in range(60):
            st = lib.vt_seg_grow_async(s, 1) if (it + seed) % 3 else lib.vt_seg_grow(s, ((it % 4) + 1) * CH)
            if st not in (0, _lib.VT_ERR_RESERVE, _lib.VT_ERR_POOL_EMPTY):
                errors.append(st)
            if it % 7 == 6:
                lib.vt_seg_wait(s, 2_000_000)
                if lib.vt_seg_release(s, 0) != 0:
                    errors.append(-1)
    ts = [threading.Thread(target=worker, args=(s, i)) for i, s in enumerate(segs)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors
    for s in segs:
        assert lib.vt_seg_wait(s, 5_000_000) in (0, _lib.VT_ERR_RESERVE, _lib.VT_ERR_POOL_EMPTY)
    total_mapped = sum(mapped(s) // CH * 4 for s in segs)
    assert total_mapped + free_chunks(pool) == 64
    for s in segs:
        assert lib.vt_seg_destroy(s) == 0
    assert free_chunks(pool) == 64


def test_python_mirror_of_the_reference_module():
    """vmmAllocator keeps the reference's names and call shapes (vmm_allocator.h:190-219)."""
    from glake_b200 import vmmAllocator as A
    from glake_b200.vmm_allocator.vmm_allocator import KV_cache
    lib.vt_use_mock_driver(1)
    try:
        assert A.init_physical_handle(40, 0) is True
        assert A.showFreeBlocks() == 40
        segs = [A.KVcacheSegment(2, 8 * MiB, CH, i < 1) for i in range(3)]   # slot 0 pre-cached
        assert A.showFreeBlocks() == 36 and segs[0].actual_size == CH and segs[1].actual_size == 0
        caches = [(KV_cache(3, l), KV_cache(3, l)) for l in range(2)]
        A.copy_kv_cache([k.kv_cache for k, _ in caches], [v.kv_cache for _, v in caches], segs)
        assert caches[1][0].vmm_ptr == caches[1][0].kv_cache.getKVCachePtr() and caches[1][1].layer_index == 1
        kv = 1024
        off = A.extend_kv_cache_batch(None, None, [0, 1, 2], [5 * kv, 3000 * kv, kv], segs, [0, 0, 0], kv, False)
        assert off == [0, 0, 0] and [s.get_used_slot() for s in segs] == [5 * kv, 3000 * kv, kv]
        assert segs[1].actual_size == 2 * CH
        segs[2].eagerExtend(kv, 2)
        A.wait_ready([2])
        assert A.query_shm([0, 1, 2]) and not A.query_cycle([2]) and segs[2].actual_size == 2 * CH
        off = A.extend_kv_cache_batch(None, None, [0, 1, 2], [kv] * 3, segs, [0, 2, 0], kv, True)
        assert off == [5 * kv, 2 * kv, kv]
        assert segs[0].show_info(0)[:3] == [0, CH, 6 * kv]
        segs[0].release_seq(0)                      # keeps its pre-cached chunk
        segs[1].release_seq(1)                      # mapped >= expand_size: keeps expand_size too
        segs[2].preempt_seq(2)
        assert [s.actual_size for s in segs] == [CH, CH, 0]
        assert A.query_unmap([0, 1]) == [True, True] and A.print_shm_state([0, 2]) == [1, 1]
        for k, v in caches:
            k.kv_cache.close(), v.kv_cache.close()
        for s in segs:
            s.close()
        assert A.showFreeBlocks() == 40
    finally:
        A.shutdown()
        lib.vt_use_mock_driver(0)
