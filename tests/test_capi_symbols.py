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


def test_header_is_plain_c_and_links_against_the_library(tmp_path):
    """include/vtensor.h must be consumable from C (the reference's FFI side may be C, cgo, JNI ...):
    a C99 translation unit including it compiles without warnings and links against libvtensor.so."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        import pytest
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "use_header.c"
    src.write_text('#include "vtensor.h"\n#include <stdio.h>\n'
                   'int main(void) { size_t b = 0; if (vt_ar_buffer_bytes(1u << 20, &b) != VT_OK) return 2;\n'
                   '  printf("%s %zu %s\\n", vt_version(), b, vt_strerror(VT_ERR_TOO_LARGE)); return 0; }\n')
    exe = tmp_path / "use_header"
    lib_dir = os.path.join(root, "glake_b200")
    res = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(root, "include"),
                          str(src), "-o", str(exe), "-L", lib_dir, "-l:libvtensor.so", f"-Wl,-rpath,{lib_dir}"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and "sm_100a" in run.stdout, run.stdout + run.stderr
