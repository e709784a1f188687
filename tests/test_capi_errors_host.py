"""Argument checking of the kernel entry points, exercised without a GPU: every
case below must be refused by the C ABI before anything is launched, with the
status the header documents."""
import ctypes

import pytest
import torch

from glake_b200 import _lib
from glake_b200._lib import (VT_ERR_INVALID, VT_ERR_TOO_LARGE, VT_ERR_UNSUPPORTED, VT_KV_BF16, VT_KV_FP8_E4M3, lib)

P = ctypes.c_void_p
BUF = (ctypes.c_ubyte * 4096)()
A = ctypes.addressof(BUF)
A16 = A + (-A) % 256            # an aligned, non-null dummy address; nothing dereferences it in these calls


def test_rope_append_argument_checks():
    def call(rot_dim=128, d=128, q=A16, stride=1024, kv_dtype=VT_KV_BF16, flags=0, max_seq_len=1, batch=1):
        return lib.vt_rope_append(P(A16), P(q), stride, 8, P(A16), P(A16), 1024, 1024, P(A16), rot_dim, 1, P(A16), P(A16),
                                  P(A16), P(A16), None, None, max_seq_len, batch, 8, d, kv_dtype, None, None, flags, None)
    assert call(rot_dim=24) == VT_ERR_UNSUPPORTED          # not a multiple of 16
    assert call(rot_dim=256) == VT_ERR_UNSUPPORTED         # beyond the head size
    assert call(d=64) == VT_ERR_UNSUPPORTED
    assert call(q=A16 + 2) == VT_ERR_UNSUPPORTED           # 16-byte vector accesses
    assert call(stride=1020) == VT_ERR_INVALID             # narrower than the heads it holds
    assert call(kv_dtype=VT_KV_FP8_E4M3) == VT_ERR_INVALID  # fp8 without scales
    assert call(flags=2) == VT_ERR_INVALID
    assert call(max_seq_len=5) == VT_ERR_INVALID           # prefill without seq_lens / cache_seq_lens
    assert call(batch=0) == 0


def test_norm_argument_checks():
    assert lib.vt_rms_norm(P(A16), P(A16), P(A16), 1e-5, 2, 12, 12, 12, None) == VT_ERR_UNSUPPORTED      # hidden % 8
    assert lib.vt_rms_norm(P(A16), P(A16), P(A16), 1e-5, 2, 16392, 16392, 16392, None) == VT_ERR_UNSUPPORTED
    assert lib.vt_rms_norm(P(A16), P(A16), P(A16), 1e-5, 2, 64, 60, 64, None) == VT_ERR_UNSUPPORTED      # stride < hidden
    assert lib.vt_rms_norm(P(A16), None, P(A16), 1e-5, 2, 64, 64, 64, None) == VT_ERR_INVALID
    assert lib.vt_fused_add_rms_norm(P(A16), None, P(A16), 1e-5, 2, 64, None) == VT_ERR_INVALID
    assert lib.vt_fused_add_rms_norm(P(A16), P(A16), P(A16), 1e-5, 0, 64, None) == 0


def test_all_reduce_argument_checks():
    need = ctypes.c_size_t()
    assert lib.vt_ar_buffer_bytes(1 << 20, ctypes.byref(need)) == 0
    push2 = 3 * ((2 << 20) + 8 * (64 + 16) * 16) + 3 * (2 << 20)             # two-phase push: 3 scatter areas + 3 gather buffers
    assert need.value == 2 * 4096 + 4 * (1 << 20) + 3 * 8 * (256 << 10) + push2   # flags, 2 staging + 2 result copies, push buffers
    assert lib.vt_ar_buffer_bytes(1000, ctypes.byref(need)) == VT_ERR_INVALID          # not a multiple of 256
    out = P()
    peers = (P * 9)(*[A16] * 9)
    assert lib.vt_ar_create(0, 9, peers, 1 << 20, 0, ctypes.byref(out)) == VT_ERR_INVALID
    assert lib.vt_ar_create(2, 2, peers, 1 << 20, 0, ctypes.byref(out)) == VT_ERR_INVALID
    assert lib.vt_ar_create(0, 2, peers, 1 << 20, 65, ctypes.byref(out)) == VT_ERR_INVALID
    bad = (P * 2)(A16, A16 + 16)
    assert lib.vt_ar_create(0, 2, bad, 1 << 20, 0, ctypes.byref(out)) == VT_ERR_INVALID  # 256-byte aligned buffers
    assert lib.vt_all_reduce(None, P(A16), P(A16), 8, None) == VT_ERR_INVALID


def test_prefill_map_argument_checks():
    bases = (ctypes.c_uint64 * 2)(1 << 30, 2 << 30)
    host = P(A16)
    assert lib.vt_prefill_maps_encode(bases, bases, 2, 3, 128, 4096, host) == VT_ERR_UNSUPPORTED    # 3 kv heads
    assert lib.vt_prefill_maps_encode(bases, bases, 2, 512, 128, 4096, host) == VT_ERR_UNSUPPORTED  # box would straddle chunks
    assert lib.vt_prefill_maps_encode(bases, bases, 2, 8, 64, 4096, host) == VT_ERR_UNSUPPORTED
    assert lib.vt_prefill_maps_encode(bases, bases, 2, 8, 128, 4096, P(A16 + 8)) == VT_ERR_INVALID  # 64-byte aligned table
    args = [P(A16), 1024, P(A16), 1024, P(A16), P(A16), P(A16), P(A16), P(A16), P(A16), 1, 8, 3, 128, 16, 0.1, VT_KV_BF16, None]
    assert lib.vt_prefill_attn_tma(*args, P(A16), None) == VT_ERR_UNSUPPORTED                     # 8 q heads over 3 kv heads
    args[12] = 2
    assert lib.vt_prefill_attn_tma(*args, None, None) == VT_ERR_INVALID                           # maps required
    args[2] = P(A16 + 4)
    assert lib.vt_prefill_attn(*args, None) == VT_ERR_UNSUPPORTED                                 # q rows are read 16 bytes at a time


def test_decode_map_argument_checks():
    """vt_decode_maps_encode / vt_decode_step_tma (the tcgen05 decode path of an fp8 cache): argument
    errors come back as status codes before anything touches a GPU."""
    bases = (ctypes.c_uint64 * 2)(1 << 30, 2 << 30)
    host = P(A16)
    assert lib.vt_decode_maps_encode(bases, bases, 2, 8, 128, VT_KV_BF16, 4096, host) == VT_ERR_UNSUPPORTED       # fp8 ranges only
    assert lib.vt_decode_maps_encode(bases, bases, 2, 6, 128, VT_KV_FP8_E4M3, 4096, host) == VT_ERR_UNSUPPORTED   # 6 kv heads
    assert lib.vt_decode_maps_encode(bases, bases, 2, 8, 64, VT_KV_FP8_E4M3, 4096, host) == VT_ERR_UNSUPPORTED
    assert lib.vt_decode_maps_encode(bases, bases, 2, 8, 128, VT_KV_FP8_E4M3, 0, host) == VT_ERR_INVALID
    assert lib.vt_decode_maps_encode(bases, bases, 2, 8, 128, VT_KV_FP8_E4M3, 4096, P(A16 + 8)) == VT_ERR_INVALID # 64-byte aligned table
    assert lib.vt_decode_maps_encode(None, bases, 2, 8, 128, VT_KV_FP8_E4M3, 4096, host) == VT_ERR_INVALID
    # out, stride, q, stride, key, value, strides, byte_off, tables, slot ids, seq lens, batch, h, kvh, d, max len, scale, dtype, scales, lse, ws, bytes, flags
    args = [P(A16), 1024, P(A16), 1024, P(A16), P(A16), 1024, 1024, P(A16), P(A16), P(A16), P(A16), P(A16), 1, 8, 8, 128, 64,
            0.1, VT_KV_FP8_E4M3, P(A16), P(A16), None, P(A16), 1 << 20, 0]
    assert lib.vt_decode_step_tma(*args, None, None) == VT_ERR_INVALID                       # maps required
    assert lib.vt_decode_step_tma(*args, P(A16 + 8), None) == VT_ERR_INVALID                 # 64-byte aligned table
    bad = list(args); bad[25] = 8
    assert lib.vt_decode_step_tma(*bad, P(A16), None) == VT_ERR_INVALID                      # unknown flag
    bad = list(args); bad[4] = None; bad[5] = None; bad[25] = 1
    assert lib.vt_decode_step_tma(*bad, P(A16), None) == VT_ERR_INVALID                      # overlap forms need the fused step
    bad = list(args); bad[5] = None
    assert lib.vt_decode_step_tma(*bad, P(A16), None) == VT_ERR_INVALID                      # key without value
    bad = list(args); bad[16] = 64
    assert lib.vt_decode_step_tma(*bad, P(A16), None) == VT_ERR_UNSUPPORTED                  # head size


def test_python_ops_refuse_cpu_tensors():
    from glake_b200 import ops
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.rms_norm(torch.empty_like(x), x, x[0], 1e-5)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fused_add_rms_norm(x, x.clone(), x[0], 1e-5)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.rotary_embedding_and_cache(torch.zeros(2, dtype=torch.int64), x, x, x, 128, x, True, x, x, x, x, None, None, 1, 1)
    assert ops.prefill_tma_supported(8) and ops.prefill_tma_supported(1) and ops.prefill_tma_supported(256)
    assert not ops.prefill_tma_supported(3) and not ops.prefill_tma_supported(512)
    assert VT_ERR_TOO_LARGE == 11 and _lib.VT_OK == 0
