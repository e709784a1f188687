"""Model-based test of the VMM allocator on the mock driver: random sequences of
create / grow / background growth / wait / release / preempt / set_used / destroy
and injected driver failures are replayed against a few lines of Python that state
what the C++ allocator promises — all-or-nothing growth, chunk conservation, stable
base addresses, mapped <= reserved, release-to-watermark and preempt semantics
(GLakeServe/vmm_allocator/vmm_allocator.cpp:151-337, vmm_allocator.h:60-136)."""
from ctypes import byref, c_int, c_size_t, c_uint64, c_void_p

import hypothesis.strategies as st
from hypothesis import settings
from hypothesis.stateful import RuleBasedStateMachine, invariant, precondition, rule

from glake_b200 import _lib
from glake_b200._lib import lib

CH = 2 << 20
POOL = 20


class Seg:
    def __init__(self, handle, layers, reserve_chunks, mapped_chunks, bases):
        self.h, self.layers, self.reserve, self.mapped, self.bases = handle, layers, reserve_chunks, mapped_chunks, bases
        self.used = 0


class AllocatorMachine(RuleBasedStateMachine):
    def __init__(self):
        super().__init__()
        lib.vt_use_mock_driver(1)
        lib.vt_mock_map_delay_us(0)
        self.pool = c_void_p()
        assert lib.vt_pool_create(0, POOL, 0, byref(self.pool)) == 0
        self.segs = []

    def teardown(self):
        for s in self.segs:
            assert lib.vt_seg_destroy(s.h) == 0
        assert self._free() == POOL
        assert lib.vt_pool_destroy(self.pool) == 0
        lib.vt_use_mock_driver(0)

    # ---- helpers ----
    def _free(self):
        n = c_size_t()
        assert lib.vt_pool_free_chunks(self.pool, byref(n)) == 0
        return n.value

    def _mapped(self, s):
        n = c_size_t()
        assert lib.vt_seg_mapped(s.h, byref(n)) == 0
        return n.value // CH

    def _bases(self, s):
        out = []
        for layer in range(s.layers):
            k, v = c_uint64(), c_uint64()
            assert lib.vt_seg_k_ptr(s.h, layer, byref(k)) == 0 and lib.vt_seg_v_ptr(s.h, layer, byref(v)) == 0
            out += [k.value, v.value]
        return out

    def _model_free(self):
        return POOL - sum(2 * s.layers * s.mapped for s in self.segs)

    # ---- rules ----
    @rule(layers=st.integers(1, 3), reserve=st.integers(1, 6), premap=st.integers(0, 2))
    def create(self, layers, reserve, premap):
        premap = min(premap, reserve)
        h = c_void_p()
        status = lib.vt_seg_create(self.pool, layers, reserve * CH, premap * CH, byref(h))
        if 2 * layers * premap > self._model_free():
            assert status == _lib.VT_ERR_POOL_EMPTY
            return
        assert status == 0
        s = Seg(h, layers, reserve, premap, None)
        s.bases = self._bases(s)
        self.segs.append(s)

    @precondition(lambda self: self.segs)
    @rule(data=st.data(), chunks=st.integers(1, 7), background=st.booleans())
    def grow(self, data, chunks, background):
        s = data.draw(st.sampled_from(self.segs))
        want = max(s.mapped, chunks)
        need = 2 * s.layers * (want - s.mapped)
        if background:
            status = lib.vt_seg_grow_async(s.h, want - s.mapped) if want > s.mapped else 0
            if status == 0 and want > s.mapped:
                status = lib.vt_seg_wait(s.h, 2_000_000)
        else:
            status = lib.vt_seg_grow(s.h, want * CH - 5)            # any byte count inside the last chunk
        if want > s.reserve:
            assert status == _lib.VT_ERR_RESERVE
        elif need > self._model_free():
            assert status == _lib.VT_ERR_POOL_EMPTY
        else:
            assert status == 0
            s.mapped = want

    @precondition(lambda self: self.segs)
    @rule(data=st.data(), call=st.sampled_from([b"cuMemMap", b"cuMemSetAccess"]), nth=st.integers(1, 4))
    def failed_growth_rolls_back(self, data, call, nth):
        s = data.draw(st.sampled_from(self.segs))
        if s.mapped >= s.reserve or 2 * s.layers > self._model_free():
            return
        calls = 2 * s.layers if call == b"cuMemMap" else 2 * s.layers
        lib.vt_mock_fail_nth(call, nth)
        status = lib.vt_seg_grow(s.h, (s.mapped + 1) * CH)
        lib.vt_mock_fail_nth(call, 0)
        if nth <= calls:
            assert status == _lib.VT_ERR_DRIVER                      # nothing of the growth stays behind
        else:
            assert status == 0
            s.mapped += 1

    @precondition(lambda self: self.segs)
    @rule(data=st.data(), keep=st.integers(0, 3))
    def release(self, data, keep):
        s = data.draw(st.sampled_from(self.segs))
        assert lib.vt_seg_release(s.h, keep * CH) == 0
        s.mapped = min(s.mapped, keep)
        s.used = 0

    @precondition(lambda self: self.segs)
    @rule(data=st.data(), frac=st.floats(0, 1))
    def set_used(self, data, frac):
        s = data.draw(st.sampled_from(self.segs))
        target = int(frac * s.mapped * CH)
        assert lib.vt_seg_set_used(s.h, target) == 0
        s.used = target

    @precondition(lambda self: self.segs)
    @rule(data=st.data())
    def destroy(self, data):
        s = data.draw(st.sampled_from(self.segs))
        assert lib.vt_seg_destroy(s.h) == 0
        self.segs.remove(s)

    # ---- what must always hold ----
    @invariant()
    def chunks_are_conserved(self):
        assert self._free() == self._model_free()

    @invariant()
    def segments_match_the_model(self):
        for s in self.segs:
            assert self._mapped(s) == s.mapped <= s.reserve
            assert self._bases(s) == s.bases                         # growth and release never move a range
            u, r = c_size_t(), c_int()
            assert lib.vt_seg_used(s.h, byref(u)) == 0 and u.value == s.used
            assert lib.vt_seg_ready(s.h, byref(r)) == 0 and r.value == 1


TestAllocatorModel = AllocatorMachine.TestCase
TestAllocatorModel.settings = settings(max_examples=60, stateful_step_count=30, deadline=None)
