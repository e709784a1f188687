"""The C-ABI library loads without a GPU and exports every symbol that
include/vtensor.h declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vtensor.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vt_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from glake_b200 import _lib
    syms = declared_symbols()
    assert len(syms) >= 30
    raw = ctypes.CDLL(_lib.LIB_PATH)
    missing = [s for s in syms if not hasattr(raw, s)]
    assert not missing, f"declared in vtensor.h but not exported: {missing}"
    # and the Python binding covers all of them
    assert sorted(_lib.lib._vt_symbols) == syms


def test_status_strings_and_version():
    from glake_b200 import _lib
    assert _lib.lib.vt_strerror(0) == b"ok"
    assert b"pool" in _lib.lib.vt_strerror(_lib.VT_ERR_POOL_EMPTY)
    assert b"sm_100a" in _lib.lib.vt_version()


def test_argument_validation_needs_no_gpu():
    """Entry points reject bad arguments before touching the device."""
    from glake_b200 import _lib
    L = _lib.lib
    n = ctypes.c_size_t()
    assert L.vt_decode_attn_workspace_bytes(8, 32, 64, 2048, ctypes.byref(n)) == _lib.VT_ERR_UNSUPPORTED
    assert L.vt_decode_attn_workspace_bytes(8, 32, 128, 2048, ctypes.byref(n)) == 0 and n.value > 0
    assert L.vt_decode_attn(None, 0, None, 0, None, None, None, None, 4, 8, 2, 128, 100, 1.0, 0, None, None, None,
                            None, 0, 0, None) == _lib.VT_ERR_INVALID
    assert L.vt_append(None, None, 0, 0, None, None, None, None, None, None, 1, 4, 2, 128, 0, None, None,
                       None) == _lib.VT_ERR_INVALID
    assert L.vt_append(None, None, 0, 0, None, None, None, None, None, None, 1, 0, 2, 128, 0, None, None, None) == 0
    assert L.vt_pool_create(0, 1, 12345, ctypes.byref(ctypes.c_void_p())) in (_lib.VT_ERR_INVALID,
                                                                               _lib.VT_ERR_NO_DRIVER,
                                                                               _lib.VT_ERR_DRIVER)
