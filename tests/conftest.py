import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_sessionstart(session):
    """The shared library is a build product (not in version control): compile it when a fresh checkout has
    none and nvcc is there.  Without it the package refuses to import, which is what the tests would report."""
    from fgms_b200 import build as lib_build

    if not os.path.exists(lib_build.LIB) and os.path.exists(os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")):
        lib_build.build()


def golden_names():
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.endswith(".npz"))


@pytest.fixture(params=golden_names())
def golden(request):
    import numpy as np

    with np.load(os.path.join(GOLDEN_DIR, request.param + ".npz")) as z:
        d = {k: z[k] for k in z.files}
    d["name"] = request.param
    return d
