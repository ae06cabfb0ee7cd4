"""Generate the golden fixtures in this directory from the UNMODIFIED reference scripts.

Run once, in a container that has the reference checkout (it is not needed at test time):

    python tests/golden/make_golden.py /path/to/FGMS

It imports ``cpu_compute`` / ``kpos_quantized`` from the reference's ``cpu-check.py`` and
``cpu-check-back.py`` and ``remove_mid`` from ``spconv-test.py`` (their only import that
needs CUDA, ``FGMS.backend``, is replaced by an empty stand-in module because only the
CPU functions are called), feeds them small seeded cases built with this repo's map
builder, and stores inputs and the reference's outputs as ``.npz``.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from fgms_b200 import clouds, maps  # noqa: E402


def _load_reference(ref_root: str):
    stub = types.ModuleType("FGMS.backend")
    for name in ("fgms_fwd_cuda", "fgms_fusion_fwd_cuda", "fgms_bwd_cuda"):
        setattr(stub, name, None)
    pkg = types.ModuleType("FGMS")
    pkg.backend = stub
    sys.modules["FGMS"] = pkg
    sys.modules["FGMS.backend"] = stub
    mods = {}
    for key, fname in (("fwd", "cpu-check.py"), ("bwd", "cpu-check-back.py"), ("bench", "spconv-test.py")):
        spec = importlib.util.spec_from_file_location(f"_ref_{key}", os.path.join(ref_root, fname))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[key] = mod
    return mods


CASES = [
    # name, n voxels, grid, kind, c_in, c_out, seed
    ("sub3_c4x6", 60, 6, "sub", 4, 6, 11),
    ("sub3_c5x3_nocentre", 48, 5, "sub_nocentre", 5, 3, 12),
    ("down2_c3x8", 70, 8, "down", 3, 8, 13),
    ("up2_c8x3", 70, 8, "up", 8, 3, 14),
    ("sub3_c16x16", 40, 5, "sub", 16, 16, 15),
]


def main(ref_root: str) -> None:
    ref = _load_reference(ref_root)
    for name, n, grid, kind, c_in, c_out, seed in CASES:
        coords = clouds.uniform_cloud(n, grid, seed)
        if kind.startswith("sub"):
            km = maps.build_submanifold_map(coords, 3)
            if kind == "sub_nocentre":
                km = maps.drop_centre(km)
        else:
            km = maps.build_strided_map(coords, 2, 2)
            if kind == "up":
                km = maps.transpose_map(km)
        feats, weights, grad_out = clouds.make_tensors(km.n_in, km.n_out, c_in, c_out, km.k_vol, seed)
        precompute = kind == "sub_nocentre"
        t = torch.from_numpy
        knnz_t = t(km.knnz)
        out = ref["fwd"].cpu_compute(t(feats), t(weights), km.n_out, knnz_t, t(km.imap), t(km.omap), precompute)
        in_grad, w_grad = ref["bwd"].cpu_compute(t(grad_out), t(weights), t(feats), km.n_in, knnz_t,
                                                 t(km.imap), t(km.omap))
        qkpos, qsum = ref["fwd"].kpos_quantized(knnz_t, t(km.kpos), km.k_vol, 256)
        extra = {}
        if kind == "sub_nocentre":
            rq, rs, rkpos, rimap, romap = ref["bench"].remove_mid(
                km.n_in, knnz_t.clone(), t(km.kpos), km.k_vol, 256, t(km.imap), t(km.omap))
            extra = dict(rm_qkpos=rq.numpy(), rm_qsum=np.int64(rs), rm_kpos=rkpos.numpy(),
                         rm_imap=rimap.numpy(), rm_omap=romap.numpy())
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            coords=coords, n_in=np.int64(km.n_in), n_out=np.int64(km.n_out), knnz=km.knnz, kpos=km.kpos,
            imap=km.imap, omap=km.omap, feats=feats, weights=weights, grad_out=grad_out,
            precompute=np.bool_(precompute), out=out.numpy(), in_grad=in_grad.numpy(), w_grad=w_grad.numpy(),
            qkpos=qkpos.numpy(), qsum=np.int64(qsum), **extra)
        print(f"{name}: n_in={km.n_in} n_out={km.n_out} pairs={km.pairs} |out|max={np.abs(out.numpy()).max():.4f}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of hkeee21/FGMS>")
    main(sys.argv[1])
