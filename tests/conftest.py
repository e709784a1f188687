import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")
    # The package refuses to import without its CUDA library (there is no fallback), so
    # build it when the tree is fresh; nvcc cross-compiles for sm_100a without a GPU.
    so = os.path.join(ROOT, "glake_b200", "libvtensor.so")
    if not os.path.isfile(so):
        import subprocess
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "glake_b200", "csrc"), "-j8"],
                              stdout=subprocess.DEVNULL)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.load_port()
    return O
