"""vt_decode_attn_static: the decode-attention entry point for hosts that may not
allocate device memory (plugins inside another runtime's callback, processes with
a fixed and policed memory budget, allocator-free hot paths).  Its scratch is a
fixed array inside the library instead of a caller-provided buffer.

Checked here, through the C ABI: two calls in a row give bit-identical output to
the regular entry point (vt_decode_attn with a caller-allocated workspace) and agree
with the CPU oracle within the tolerances the other attention tests use (2e-3 for a
bf16 cache, 1e-2 for fp8), although the shared scratch still holds the previous
call's contents; an fp8 problem whose default schedule does not fit the array falls
back to split-K and still matches; problems that fit no schedule are refused with
VT_ERR_TOO_LARGE.  This file is collected last on purpose, and passes both alone in
a fresh process and after the rest of the suite.
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
    ks = c_void_p(kv.k_scale.data_ptr()) if kv.fp8 else None
    vs = c_void_p(kv.v_scale.data_ptr()) if kv.fp8 else None
    return lib.vt_decode_attn_static(
        c_void_p(out.data_ptr()), out.stride(0), c_void_p(q.data_ptr()), q.stride(0), c_void_p(kv.k_table),
        c_void_p(kv.v_table), c_void_p(kv.meta.slot_mapping.data_ptr()), c_void_p(kv.meta.seq_lens_tensor.data_ptr()),
        b, h, kv.kvh, d, kv.meta.max_seq_len, ctypes.c_float(SCALE), 1 if kv.fp8 else 0, ks, vs,
        c_void_p(lse.data_ptr()) if lse is not None else None, num_splits, stream)


def _oracle_result(oracle, q, k, v, lens, kvh, ks=None, vs=None):
    r = oracle.fill_ranges(k, v, k_scale=ks, v_scale=vs)
    return oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh, SCALE,
                                   ks, vs)


@pytest.mark.parametrize("h,kvh,lens", [(8, 8, [700, 33, 1500, 1]), (16, 2, [2100, 900]), (8, 1, [4096, 5000, 64]),
                                         (16, 1, [3000, 517])])
def test_static_scratch_matches_regular_entry_point_twice(oracle, h, kvh, lens):
    from tests import gpu_util
    q, k, v = synth.make_case(900 + h + kvh, lens, h, kvh)
    kv = gpu_util.GpuKV(k, v, kvh)
    try:
        want = kv.attend(q, SCALE)                      # regular entry point, caller-allocated workspace
        port = _oracle_result(oracle, q, k, v, lens, kvh)
        tol = torch.maximum(torch.full_like(port.float(), 2e-3), port.float().abs() * 2.0 ** -7)
        qd = q.cuda()
        for call in range(2):                           # second call reuses the dirty shared scratch
            out = torch.full_like(qd, float("nan"))
            assert _static_call(qd, kv, out) == 0
            torch.cuda.synchronize()
            got = out.cpu()
            assert torch.equal(got, want), f"call {call}: differs from the regular entry point"
            assert bool(((got.float() - port.float()).abs() <= tol).all()), f"call {call}: differs from the oracle"
        # forced split-K path through the same static scratch
        want3 = kv.attend(q, SCALE, num_splits=3)
        out = torch.full_like(qd, float("nan"))
        assert _static_call(qd, kv, out, num_splits=3) == 0
        torch.cuda.synchronize()
        assert (out.cpu().float() - want3.float()).abs().max() <= 2e-3
        assert bool(((out.cpu().float() - port.float()).abs() <= tol).all())
    finally:
        kv.close()


@pytest.mark.parametrize("h,kvh,lens,same_schedule", [
    (8, 8, [700, 33, 1500, 2], True),        # fp8, default schedule fits the array
    (32, 8, [2100, 900, 4100], True),
    (16, 1, [3000, 517], False),             # fp8 with a query group of 16: falls back to split-K
])
def test_static_scratch_fp8_cache(oracle, h, kvh, lens, same_schedule):
    from glake_b200 import ops
    from tests import gpu_util
    q, k, v = synth.make_case(950 + h + kvh, lens, h, kvh)
    ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
    vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = gpu_util.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    try:
        want = kv.attend(q, SCALE)
        port = _oracle_result(oracle, q, k, v, lens, kvh, ks.cpu(), vs.cpu())
        tol = torch.maximum(torch.full_like(port.float(), 1e-2), port.float().abs() * 2.0 ** -6)
        qd = q.cuda()
        for call in range(2):
            out = torch.full_like(qd, float("nan"))
            assert _static_call(qd, kv, out) == 0
            torch.cuda.synchronize()
            got = out.cpu()
            if same_schedule:
                assert torch.equal(got, want), f"call {call}"
            else:
                assert (got.float() - want.float()).abs().max() <= 1e-2, f"call {call}"
            assert bool(((got.float() - port.float()).abs() <= tol).all()), f"call {call}: differs from the oracle"
    finally:
        kv.close()


def test_static_scratch_refuses_what_does_not_fit():
    from glake_b200 import _lib
    b, h = 64, 32
    q = torch.zeros(b, h, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    one = torch.ones(b, dtype=torch.int32, device="cuda")
    slot = torch.zeros(b, dtype=torch.int64, device="cuda")
    # 64 forced partitions x 64 sequences x 32 heads of fp32 partials: 68 MB, beyond the built-in array;
    # refused before anything is launched (the table addresses below are never dereferenced)
    st = _lib.lib.vt_decode_attn_static(
        c_void_p(out.data_ptr()), h * 128, c_void_p(q.data_ptr()), h * 128, c_void_p(1 << 20), c_void_p(1 << 20),
        c_void_p(slot.data_ptr()), c_void_p(one.data_ptr()), b, h, 8, 128, 32768, ctypes.c_float(1.0), 0, None, None,
        None, 64, None)
    assert st == _lib.VT_ERR_TOO_LARGE
    assert b"static" in _lib.lib.vt_strerror(st)
