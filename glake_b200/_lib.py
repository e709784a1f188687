"""ctypes binding of libvtensor.so (the C ABI declared in include/vtensor.h).

There is no fallback: if the shared library is missing the import raises, and
every non-zero status from the library becomes a VTensorError.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvtensor.so")

VT_OK = 0
VT_ERR_INVALID, VT_ERR_DRIVER, VT_ERR_POOL_EMPTY, VT_ERR_RESERVE, VT_ERR_TIMEOUT = 1, 2, 3, 4, 5
VT_ERR_UNSUPPORTED, VT_ERR_CUDA, VT_ERR_STATE, VT_ERR_NO_DRIVER, VT_ERR_KERNEL = 6, 7, 8, 9, 10
VT_ERR_TOO_LARGE = 11
VT_STATIC_SCRATCH_BYTES = 24 << 20
VT_STEP_OVERLAP = 1
VT_STEP_EARLY_KV = 2
VT_STEP_CLEAN_SCRATCH = 4
VT_KV_BF16, VT_KV_FP8_E4M3 = 0, 1


class VTensorError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        drv = lib.vt_last_driver_error() if status == VT_ERR_DRIVER else 0
        msg = lib.vt_strerror(status).decode()
        super().__init__(f"{where}: {msg} (status {status}" + (f", CUresult {drv})" if drv else ")"))


class Stats(ctypes.Structure):
    _fields_ = [(n, c_uint64) for n in (
        "chunks_total", "chunks_free", "chunk_bytes", "map_calls", "unmap_calls", "set_access_calls",
        "map_ns", "access_ns", "async_requests", "async_completed", "async_failed", "segments")]


def _load():
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(or __graft_entry__.build()); glake_b200 has no CPU or PyTorch fallback")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz = c_void_p, c_size_t
    sigs = {
        "vt_strerror": (c_char_p, [c_int]),
        "vt_version": (c_char_p, []),
        "vt_last_driver_error": (c_int, []),
        "vt_use_mock_driver": (c_int, [c_int]),
        "vt_mock_fail_nth": (c_int, [c_char_p, c_int]),
        "vt_mock_map_delay_us": (c_int, [c_int]),
        "vt_pool_create": (c_int, [c_int, sz, sz, POINTER(vp)]),
        "vt_pool_destroy": (c_int, [vp]),
        "vt_pool_free_chunks": (c_int, [vp, POINTER(sz)]),
        "vt_pool_stats": (c_int, [vp, POINTER(Stats)]),
        "vt_seg_create": (c_int, [vp, c_int, sz, sz, POINTER(vp)]),
        "vt_seg_destroy": (c_int, [vp]),
        "vt_seg_k_ptr": (c_int, [vp, c_int, POINTER(c_uint64)]),
        "vt_seg_v_ptr": (c_int, [vp, c_int, POINTER(c_uint64)]),
        "vt_seg_used": (c_int, [vp, POINTER(sz)]),
        "vt_seg_set_used": (c_int, [vp, sz]),
        "vt_seg_mapped": (c_int, [vp, POINTER(sz)]),
        "vt_seg_reserved": (c_int, [vp, POINTER(sz)]),
        "vt_seg_grow": (c_int, [vp, sz]),
        "vt_seg_grow_async": (c_int, [vp, c_int]),
        "vt_seg_ready": (c_int, [vp, POINTER(c_int)]),
        "vt_seg_wait": (c_int, [vp, c_uint64]),
        "vt_seg_release": (c_int, [vp, sz]),
        "vt_extend_batch": (c_int, [POINTER(vp), c_int, POINTER(c_int64), POINTER(c_uint64), c_uint64, c_int,
                                    c_uint64, POINTER(c_int64)]),
        "vt_table_create": (c_int, [vp, c_int, POINTER(vp)]),
        "vt_table_destroy": (c_int, [vp]),
        "vt_table_set": (c_int, [vp, c_int, c_uint64]),
        "vt_table_fill": (c_int, [vp, vp, POINTER(vp), c_int, c_int]),
        "vt_table_dptr": (c_int, [vp, POINTER(c_uint64)]),
        "vt_pool_read": (c_int, [vp, vp, c_uint64, sz]),
        "vt_pool_write": (c_int, [vp, c_uint64, vp, sz]),
        "vt_append": (c_int, [vp, vp, c_int64, c_int64, vp, vp, vp, vp, vp, vp, c_int, c_int, c_int, c_int, c_int,
                              vp, vp, vp]),
        "vt_kv_scales": (c_int, [vp, c_int64, c_int, c_int, c_int, vp, vp]),
        "vt_kv_widen": (c_int, [vp, vp, vp, vp, c_int, c_int, c_int, c_int, vp, vp, vp, vp, vp]),
        "vt_rope_append": (c_int, [vp, vp, c_int64, c_int, vp, vp, c_int64, c_int64, vp, c_int, c_int, vp, vp, vp, vp,
                                   vp, vp, c_int, c_int, c_int, c_int, c_int, vp, vp, ctypes.c_uint, vp]),
        "vt_ar_buffer_bytes": (c_int, [sz, POINTER(sz)]),
        "vt_ar_alloc": (c_int, [sz, POINTER(vp)]),
        "vt_ar_free": (c_int, [vp]),
        "vt_ar_ipc_export": (c_int, [vp, vp]),
        "vt_ar_ipc_open": (c_int, [vp, POINTER(vp)]),
        "vt_ar_ipc_close": (c_int, [vp]),
        "vt_ar_create": (c_int, [c_int, c_int, POINTER(vp), sz, c_int, POINTER(vp)]),
        "vt_ar_destroy": (c_int, [vp]),
        "vt_ar_configure": (c_int, [vp, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong]),
        "vt_ar_status": (c_int, [vp, POINTER(ctypes.c_uint32)]),
        "vt_all_reduce": (c_int, [vp, vp, vp, sz, vp]),
        "vt_all_reduce_emulated": (c_int, [POINTER(vp), POINTER(vp), POINTER(vp), c_int, sz, vp]),
        "vt_rms_norm": (c_int, [vp, vp, vp, c_float, c_int, c_int, c_int64, c_int64, vp]),
        "vt_fused_add_rms_norm": (c_int, [vp, vp, vp, c_float, c_int, c_int, vp]),
        "vt_decode_attn_workspace_bytes": (c_int, [c_int, c_int, c_int, c_int, POINTER(sz)]),
        "vt_decode_attn": (c_int, [vp, c_int64, vp, c_int64, vp, vp, vp, vp, c_int, c_int, c_int, c_int, c_int,
                                   c_float, c_int, vp, vp, vp, vp, sz, c_int, vp]),
        "vt_decode_step": (c_int, [vp, c_int64, vp, c_int64, vp, vp, c_int64, c_int64, vp, vp, vp, vp, vp, c_int, c_int,
                                   c_int, c_int, c_int, c_float, c_int, vp, vp, vp, vp, sz, ctypes.c_uint, vp]),
        "vt_decode_step_tma": (c_int, [vp, c_int64, vp, c_int64, vp, vp, c_int64, c_int64, vp, vp, vp, vp, vp, c_int, c_int,
                                       c_int, c_int, c_int, c_float, c_int, vp, vp, vp, vp, sz, ctypes.c_uint, vp, vp]),
        "vt_decode_maps_encode": (c_int, [vp, vp, c_int, c_int, c_int, c_int, c_uint64, vp]),
        "vt_prefill_attn": (c_int, [vp, c_int64, vp, c_int64, vp, vp, vp, vp, vp, vp, c_int, c_int, c_int, c_int, c_int,
                                    c_float, c_int, vp, vp]),
        "vt_prefill_attn_tma": (c_int, [vp, c_int64, vp, c_int64, vp, vp, vp, vp, vp, vp, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_int, vp, vp, vp]),
        "vt_prefill_maps_encode": (c_int, [vp, vp, c_int, c_int, c_int, c_uint64, vp]),
        "vt_decode_attn_static": (c_int, [vp, c_int64, vp, c_int64, vp, vp, vp, vp, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, vp, vp, vp, c_int, vp]),
        "vt_decode_attn_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int),
                                        POINTER(c_int)]),
        "vt_attn_set_tuning": (c_int, [c_int, c_int]),
        "vt_decode_attn_status": (c_int, [vp, vp, POINTER(c_int)]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name)  # AttributeError here means the .so is stale: rebuild
        fn.restype, fn.argtypes = res, args
    L._vt_symbols = tuple(sigs)
    return L


lib = _load()


def check(status, where=""):
    if status != VT_OK:
        raise VTensorError(status, where)
