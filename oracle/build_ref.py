"""TEST INFRASTRUCTURE — builds the reference's own CPU kernels as a checker.

Compiles GLakeServe/csrc/cpu/attention.cpp, cache.cpp, pos_encoding.cpp and
layernorm.cpp (unmodified, read from the reference checkout) together with oracle/ref_shim.cpp into a Python
extension under oracle/_ref/.  Two variants are produced because the machine
that later loads the prebuilt file may lack the AVX512-BF16 extension:

    oracle/_ref/vt_ref_bf16.so     -mavx512bf16 (what cmake/cpu_extension.cmake:39-49 picks here)
    oracle/_ref/vt_ref_nobf16.so   plain AVX-512 path (cpu_types.hpp:332-346)

Flags follow GLakeServe/cmake/cpu_extension.cmake:15-17 and :39-49.  The
reference's own build system is not run.  Nothing under oracle/ is imported by
the product; only tests, the smoke check and the CPU-baseline leg of the bench
load these files.

Usage:  python oracle/build_ref.py [--reference /path/to/glake]
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

BASE_FLAGS = ["-O3", "-fopenmp", "-DVLLM_CPU_EXTENSION", "-std=c++17",
              "-mavx512f", "-mavx512vl", "-mavx512bw", "-mavx512dq"]
VARIANTS = {"vt_ref_bf16": BASE_FLAGS + ["-mavx512bf16"],
            "vt_ref_nobf16": BASE_FLAGS}


def reference_root():
    """The reference checkout: $GLAKE_REFERENCE, else a directory named "reference"
    beside this repository; None when neither holds the GLakeServe sources."""
    for cand in (os.environ.get("GLAKE_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "GLakeServe", "csrc", "cpu")):
            return os.path.abspath(cand)
    return None


def build(reference_root, verbose=False):
    cpu_dir = os.path.join(reference_root, "GLakeServe", "csrc", "cpu")
    srcs = [os.path.join(HERE, "ref_shim.cpp"),
            os.path.join(cpu_dir, "attention.cpp"),
            os.path.join(cpu_dir, "cache.cpp"),
            os.path.join(cpu_dir, "pos_encoding.cpp"),
            os.path.join(cpu_dir, "layernorm.cpp")]
    for s in srcs:
        if not os.path.isfile(s):
            raise FileNotFoundError(s)
    # /opt/gcc/bin/g++ lacks libgomp.spec, so link with -lgomp through the system g++.
    os.environ["CXX"] = "/usr/bin/g++"
    from torch.utils import cpp_extension
    os.makedirs(OUT, exist_ok=True)
    built = []
    for name, flags in VARIANTS.items():
        target = os.path.join(OUT, name + ".so")
        if os.path.isfile(target) and all(
                os.path.getmtime(target) >= os.path.getmtime(s) for s in srcs):
            built.append(target)
            continue
        bdir = os.path.join(OUT, "build_" + name)
        os.makedirs(bdir, exist_ok=True)
        cpp_extension.load(name=name, sources=srcs, extra_cflags=flags,
                           extra_ldflags=["-lgomp"], build_directory=bdir,
                           is_python_module=False, verbose=verbose)
        shutil.copyfile(os.path.join(bdir, name + ".so"), target)
        shutil.rmtree(bdir, ignore_errors=True)
        built.append(target)
    return built


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=reference_root())
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        sys.exit("no reference checkout: pass --reference or set GLAKE_REFERENCE")
    for p in build(a.reference, a.verbose):
        print("built", p)
    sys.exit(0)
