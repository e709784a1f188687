"""vt_decode_attn_static: the decode-attention entry point for hosts that may not
allocate device memory (plugins inside another runtime's callback, processes with
a fixed and policed memory budget, allocator-free hot paths).  Its scratch is a
fixed array inside the library instead of a caller-provided buffer.

Checked here, through the C ABI: two calls in a row give the same output as the
regular entry point (vt_decode_attn with a caller-allocated workspace) within the
2e-3 tolerance the other attention tests use, although the shared scratch still
holds the previous call's contents; problems whose scratch would not fit are
refused with VT_ERR_TOO_LARGE.  This file is collected last on purpose, and passes
both alone in a fresh process and after the rest of the suite.
"""
import ctypes
from ctypes import c_void_p

import pytest
import torch

from tests import synth
from tests.test_oracle import SCALE

pytestmark = pytest.mark.gpu


def _static_call(q, kv, out, lse=None, num_splits=0):
    from glake_b200._lib import lib
    b, h, d = q.shape
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.vt_decode_attn_static(
        c_void_p(out.data_ptr()), out.stride(0), c_void_p(q.data_ptr()), q.stride(0), c_void_p(kv.k_table),
        c_void_p(kv.v_table), c_void_p(kv.meta.slot_mapping.data_ptr()), c_void_p(kv.meta.seq_lens_tensor.data_ptr()),
        b, h, kv.kvh, d, kv.meta.max_seq_len, ctypes.c_float(SCALE), 0, None, None,
        c_void_p(lse.data_ptr()) if lse is not None else None, num_splits, stream)


@pytest.mark.parametrize("h,kvh,lens", [(8, 8, [700, 33, 1500, 1]), (16, 2, [2100, 900]), (8, 1, [4096, 5000, 64])])
def test_static_scratch_matches_regular_entry_point_twice(h, kvh, lens):
    from tests import gpu_util
    q, k, v = synth.make_case(900 + h + kvh, lens, h, kvh)
    kv = gpu_util.GpuKV(k, v, kvh)
    try:
        want = kv.attend(q, SCALE)                      # regular entry point, caller-allocated workspace
        qd = q.cuda()
        for call in range(2):                           # second call reuses the dirty shared scratch
            out = torch.full_like(qd, float("nan"))
            assert _static_call(qd, kv, out) == 0
            torch.cuda.synchronize()
            got = out.cpu()
            assert (got.float() - want.float()).abs().max() <= 2e-3, f"call {call}"
        # forced split-K path through the same static scratch
        want3 = kv.attend(q, SCALE, num_splits=3)
        out = torch.full_like(qd, float("nan"))
        assert _static_call(qd, kv, out, num_splits=3) == 0
        torch.cuda.synchronize()
        assert (out.cpu().float() - want3.float()).abs().max() <= 2e-3
    finally:
        kv.close()


def test_static_scratch_refuses_what_does_not_fit():
    from glake_b200 import _lib
    q = torch.zeros(1, 16, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    one = torch.ones(1, dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int64, device="cuda")
    # a query group of 16 needs more piece scratch than the built-in buffer holds
    st = _lib.lib.vt_decode_attn_static(
        c_void_p(out.data_ptr()), 16 * 128, c_void_p(q.data_ptr()), 16 * 128, c_void_p(1 << 20), c_void_p(1 << 20),
        c_void_p(slot.data_ptr()), c_void_p(one.data_ptr()), 1, 16, 1, 128, 1, ctypes.c_float(1.0), 0, None, None, None,
        0, None)
    assert st == _lib.VT_ERR_TOO_LARGE
    assert b"static" in _lib.lib.vt_strerror(st)
