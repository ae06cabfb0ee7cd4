"""Build recipe for the reference's own CUDA extension.  TEST INFRASTRUCTURE ONLY.

Compiles the two source files of hkeee21/FGMS's extension (``backend/pybind_cuda.cpp``, ``backend/spconv.cu``,
listed in its ``setup.py:5-6``) where they lie in a checkout of the reference, for sm_100a, into
``oracle/_ref/FGMS_ref/backend*.so`` — a build product that is kept out of version control.  No reference source
is copied.  The module name is ``FGMS_ref.backend`` on disk; the extension's init symbol is ``PyInit_backend``, so it
is imported as the submodule ``backend`` of the package directory ``oracle/_ref/FGMS_ref``.

Used by the GPU tests and the benchmark to put the reference's kernels beside this library's on the shapes where
the reference is sound (fp16 128 -> 128 submanifold: fused forward ``_fgms_fusion_fp16_v2``, dgrad
``_fgms_fusion_fp16_W_transpose_v2``, wgrad ``_fgms_fusion_fp16_I_transpose_v4``).  It is never loaded by the
product package.

    python -m oracle.build_ref [--force]          (needs the reference checkout: FGMS_REFERENCE_DIR, or the default below)
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref", "FGMS_ref")
REF = os.environ.get("FGMS_REFERENCE_DIR", "/root/reference")


def so_path() -> str:
    return os.path.join(OUT_DIR, "backend" + sysconfig.get_config_var("EXT_SUFFIX"))


def available() -> bool:
    return os.path.exists(so_path())


def build(force: bool = False) -> str | None:
    """Returns the path of the built module, or None when there is no reference checkout to build from."""
    srcs = [os.path.join(REF, "backend", f) for f in ("pybind_cuda.cpp", "spconv.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return so_path() if available() else None
    out = so_path()
    if not force and os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in srcs):
        return out
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT_DIR, exist_ok=True)
    open(os.path.join(OUT_DIR, "__init__.py"), "w").close()
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-x", "cu", "-DTORCH_EXTENSION_NAME=backend", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "--expt-relaxed-constexpr", "-w",
           *inc, *srcs, f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-lcublas", f"-Xlinker", f"-rpath={tlib}", "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout[-4000:] + res.stderr[-4000:])
        raise RuntimeError("building the reference extension failed")
    return out


def load():
    """Import the built extension (``torch`` must be imported first: the module links its libraries)."""
    import importlib
    import torch  # noqa: F401
    if not available():
        raise ImportError("the reference extension has not been built (python -m oracle.build_ref)")
    parent = os.path.dirname(OUT_DIR)
    if parent not in sys.path:
        sys.path.insert(0, parent)
    return importlib.import_module("FGMS_ref.backend")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
