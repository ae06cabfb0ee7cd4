"""Drop-in proof: the reference's own check scripts, unmodified, run against this repository as ``FGMS.backend``.

``cpu-check.py`` and ``cpu-check-back.py`` (repository root of hkeee21/FGMS) load every file of
``./sample-data/tiny-samples`` (keys at ``cpu-check.py:83-94``), call ``fgms_fwd_cuda`` / ``fgms_fusion_fwd_cuda`` /
``fgms_bwd_cuda`` from ``FGMS.backend`` and compare with their pure-Python loops, printing ``all close: True/False``
per tensor.  The sample files are downloaded by the reference and are not available offline, so this test writes
fixture files with the same keys from seeded synthetic clouds into a temporary directory, runs the scripts there
with ``runpy`` (as ``__main__``, with their own ``argparse``), and asserts that every line says ``all close: True``.

Two variants:

* GPU (marked ``gpu``): the real ``FGMS.backend`` of this repository, fixtures on the CUDA device.
* CPU: the same harness with a stand-in ``FGMS.backend`` that answers with the CPU oracle on CPU tensors.  It
  proves the harness and pins the oracle once more against the reference's own loops, without a GPU.

Both need a checkout of the reference (``FGMS_REFERENCE_DIR``, or the default of ``REF`` below) and are skipped without
one: its scripts are not copied into this repository.
"""
import contextlib
import io
import os
import runpy
import sys
import types

import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps
from oracle import spconv_oracle as orc

REF = os.environ.get("FGMS_REFERENCE_DIR", "/root/reference")
needs_reference = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "cpu-check.py")),
                                     reason="no checkout of the reference's scripts")


def _write_fixtures(directory, device):
    """Three layers in the reference's file format.  File names carry the kernel size at [8:11] and the stride
    at [13:16] (``cpu-check.py:136-137``).  Submanifold layers omit the centre offset, as the reference's files
    do (the scripts set ``separate_mid = in_nnz == out_nnz``, ``cpu-check.py:96``)."""
    os.makedirs(directory, exist_ok=True)
    rng = np.random.default_rng(3)
    coords = clouds.uniform_cloud(90, 7, 11)
    cases = {
        "sample--333--111-subm.pth": maps.drop_centre(maps.build_submanifold_map(coords)),
        "sample--222--222-down.pth": maps.build_strided_map(coords, 2, 2),
    }
    for name, km in cases.items():
        t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        torch.save({
            "in_feats": t(rng.standard_normal((km.n_in, 16)).astype(np.float32)),
            "kernel": t(rng.uniform(-0.2, 0.2, size=(km.k_vol, 16, 16)).astype(np.float32)),
            "sum_nnz": int(km.pairs), "out_nnz": int(km.n_out),
            "knnz": t(km.knnz), "kpos": t(km.kpos), "imap": t(km.imap), "omap": t(km.omap),
        }, os.path.join(directory, name))
    return len(cases)


def _run(script, argv, cwd):
    old_argv, old_cwd = sys.argv, os.getcwd()
    buf = io.StringIO()
    try:
        sys.argv = [script] + argv
        os.chdir(cwd)
        with contextlib.redirect_stdout(buf):
            runpy.run_path(os.path.join(REF, script), run_name="__main__")
    finally:
        sys.argv = old_argv
        os.chdir(old_cwd)
    lines = [l for l in buf.getvalue().splitlines() if "all close" in l]
    return lines


def _oracle_backend():
    """``FGMS.backend`` answered by the CPU oracle (in-place accumulation into the caller's tensors, the centre
    term when ``separate_mid``, gradients for the backward)."""
    mod = types.ModuleType("FGMS.backend")

    def fwd(feats, w, n_out, kpos, imap, omap, separate_mid):
        return torch.from_numpy(orc.fwd(feats.numpy(), w.numpy(), n_out, kpos.numpy(), imap.numpy(), omap.numpy(),
                                        precompute=separate_mid, acc=torch.float32))

    def fgms_fusion_fwd_cuda(in_feats, kernel, sum_nnz, out_feats, kpos, qkpos, in_map, out_map, separate_mid, arch80):
        res = fwd(in_feats, kernel, out_feats.size(0), kpos, in_map, out_map, separate_mid)
        if separate_mid:
            out_feats.zero_()  # the fused entry overwrites (beta = 0, backend/spconv.cu:55-56)
        out_feats += res

    def fgms_fwd_cuda(in_feats, kernel, sum_nnz, out_feats, kernel_nnz, kernel_pos, in_map, out_map, separate_mid, arch80):
        out_feats += fwd(in_feats, kernel, out_feats.size(0), kernel_pos, in_map, out_map, separate_mid)

    def fgms_bwd_cuda(out_grad, in_feats, kernel, sum_nnz, in_grad, kernel_grad, kpos, qkpos, in_map, out_map, separate_mid, arch80):
        in_grad += torch.from_numpy(orc.dgrad(out_grad.numpy(), kernel.numpy(), in_grad.size(0), kpos.numpy(), in_map.numpy(),
                                              out_map.numpy(), acc=torch.float32))
        kernel_grad += torch.from_numpy(orc.wgrad(in_feats.numpy(), out_grad.numpy(), kernel.size(0), kpos.numpy(),
                                                  in_map.numpy(), out_map.numpy(), acc=torch.float32))

    mod.fgms_fusion_fwd_cuda, mod.fgms_fwd_cuda, mod.fgms_bwd_cuda = fgms_fusion_fwd_cuda, fgms_fwd_cuda, fgms_bwd_cuda
    return mod


def _check_scripts(tmp_path, device, n_expected_files):
    for script, argv, per_file in (("cpu-check.py", [], 1), ("cpu-check.py", ["--fusion"], 1), ("cpu-check-back.py", [], 2)):
        lines = _run(script, argv + ["--in-channel", "16", "--out-channel", "16"], str(tmp_path))
        assert len(lines) == per_file * n_expected_files, (script, argv, lines)
        assert all(l.rstrip().endswith("all close: True") for l in lines), (script, argv, lines)


@needs_reference
def test_reference_scripts_accept_the_oracle_as_backend(tmp_path, monkeypatch):
    n = _write_fixtures(tmp_path / "sample-data" / "tiny-samples", "cpu")
    monkeypatch.setitem(sys.modules, "FGMS.backend", _oracle_backend())
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda *a: (10, 0))  # cpu-check.py:75 asks before anything else
    _check_scripts(tmp_path, "cpu", n)


@needs_reference
@pytest.mark.gpu
def test_reference_scripts_accept_this_repository_as_backend(tmp_path):
    import FGMS.backend  # noqa: F401  (the repository's drop-in module, not a stand-in)
    assert FGMS.backend.fgms_bwd_cuda.__module__ == "fgms_b200.backend"
    n = _write_fixtures(tmp_path / "sample-data" / "tiny-samples", "cuda")
    _check_scripts(tmp_path, "cuda", n)
