"""CPU oracle for a stack of sparse-convolution layers.  TEST INFRASTRUCTURE ONLY.

Chains the per-layer oracle of ``oracle/spconv_oracle.py`` (the reference's CPU definition,
``cpu-check.py:16-44`` / ``cpu-check-back.py:16-44``) over a layer list the way the reference's benchmark
driver walks one (``spconv-test.py:51-126``): every layer's output is the next layer's input; a layer with a
skip connection adds another layer's output to its own.  Only ``tests/`` and the benchmark's CPU leg may
import this file; the product package never does.

Two uses:

* ``forward`` / ``backward`` — the whole stack in fp64 from the stack's inputs (end-to-end check);
* ``check_layer`` inputs — the caller can also feed each layer the *stored* (fp16) input the CUDA path saw
  and compare that layer alone, which keeps the per-layer tolerance independent of depth.
"""
from __future__ import annotations

import numpy as np
import torch

from . import spconv_oracle as orc

__all__ = ["forward", "backward"]


def _np(x):
    return np.asarray(x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x)


def forward(spec, umaps, weights, feats, acc=torch.float64):
    """Returns ``{value name: array}`` for every value of the stack (``"input"`` included)."""
    val = {"input": _np(feats).astype(np.float64)}
    for layer, w in zip(spec, weights):
        km = umaps.of(layer)
        y = orc.fwd(val[layer.src], _np(w), km.n_out, km.kpos, km.imap, km.omap, acc=acc)
        if layer.skip is not None:
            y = y + val[layer.skip]
        val[layer.dst] = y
    return val


def backward(spec, umaps, weights, val, grad_out, acc=torch.float64):
    """Gradients of ``sum(output * grad_out)``: returns ``(grads by value name, weight gradients by layer)``.
    The first layer's input gradient is not formed (the stack's input needs none)."""
    grad = {spec[-1].dst: _np(grad_out).astype(np.float64)}
    w_grads = [None] * len(spec)
    for i in range(len(spec) - 1, -1, -1):
        layer, w = spec[i], weights[i]
        km = umaps.of(layer)
        g = grad[layer.dst]
        if layer.skip is not None:
            grad[layer.skip] = grad.get(layer.skip, 0) + g
        w_grads[i] = orc.wgrad(val[layer.src], g, layer.k_vol, km.kpos, km.imap, km.omap, acc=acc)
        if i > 0:
            gi = orc.dgrad(g, _np(w), km.n_in, km.kpos, km.imap, km.omap, acc=acc)
            grad[layer.src] = grad.get(layer.src, 0) + gi
    return grad, w_grads
