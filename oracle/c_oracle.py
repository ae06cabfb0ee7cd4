"""Build recipe and ctypes loader for the C restatement (``spconv_oracle.c``).

TEST INFRASTRUCTURE ONLY — see the header of ``spconv_oracle.py``.  ``build()`` compiles
``oracle/_build/liboracle.so`` with gcc (``-ffp-contract=off`` so the fp32 functions keep
the reference's one-rounding-per-operation arithmetic).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "spconv_oracle.c")
_OUT = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    if not force and os.path.exists(_OUT) and os.path.getmtime(_OUT) >= os.path.getmtime(_SRC):
        return _OUT
    os.makedirs(os.path.dirname(_OUT), exist_ok=True)
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c99", _SRC, "-o", _OUT]
    subprocess.run(cmd, check=True)
    return _OUT


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _prep(x, dt):
    return np.ascontiguousarray(np.asarray(x), dtype=dt)


def fwd(feats, weights, n_out, knnz, imap, omap, precompute=False, acc="f64"):
    lib = _load()
    f, w = _prep(feats, np.float32), _prep(weights, np.float32)
    kn, im, om = _prep(knnz, np.int32), _prep(imap, np.int32), _prep(omap, np.int32)
    k_vol, c_in, c_out = w.shape
    out = np.empty((n_out, c_out), dtype=np.float64 if acc == "f64" else np.float32)
    getattr(lib, f"fgms_oracle_fwd_{acc}")(
        _p(f), _p(w), _p(out), ctypes.c_int(n_out), ctypes.c_int(c_in), ctypes.c_int(c_out),
        ctypes.c_int(k_vol), _p(kn), _p(im), _p(om), ctypes.c_int(int(bool(precompute))))
    return out


def bwd(out_grad, weights, feats, n_in, knnz, imap, omap, acc="f64"):
    lib = _load()
    g, w, f = _prep(out_grad, np.float32), _prep(weights, np.float32), _prep(feats, np.float32)
    kn, im, om = _prep(knnz, np.int32), _prep(imap, np.int32), _prep(omap, np.int32)
    k_vol, c_in, c_out = w.shape
    dt = np.float64 if acc == "f64" else np.float32
    in_grad = np.empty((n_in, c_in), dtype=dt)
    w_grad = np.empty((k_vol, c_in, c_out), dtype=dt)
    getattr(lib, f"fgms_oracle_bwd_{acc}")(
        _p(g), _p(w), _p(f), _p(in_grad), _p(w_grad), ctypes.c_int(n_in), ctypes.c_int(c_in),
        ctypes.c_int(c_out), ctypes.c_int(k_vol), _p(kn), _p(im), _p(om))
    return in_grad, w_grad
