"""Autograd wrapper around the operator: what dgSPARSE-Lib (the caller named by the reference's README)
puts on top of ``FGMS.backend``.

``sparse_conv(feats, weight, kmap)`` is differentiable in ``feats`` and ``weight``; forward is
``fgms_fusion_fwd_cuda``, backward is ``fgms_bwd_cuda`` (dgrad + wgrad).  ``SparseConv3d`` is the
``nn.Module`` that owns the ``[k_vol, c_in, c_out]`` weight.  Kernel maps are passed in (a
:class:`fgms_b200.gpu_maps.DeviceKernelMap`, or anything with ``kpos / imap / omap / n_in / n_out``
device tensors): layers at one resolution share one map, which is the map caching the reference's driver
does by loading one file per layer shape (``spconv-test.py:63-73``).
"""
from __future__ import annotations

import math

import torch

from . import backend

__all__ = ["sparse_conv", "sparse_conv_inference", "SparseConv3d", "SparseUNet"]


class _SparseConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, feats, weight, kpos, imap, omap, n_out, arch80):
        feats = feats.contiguous()
        weight = weight.contiguous()
        out = torch.zeros((n_out, weight.size(2)), dtype=feats.dtype, device=feats.device)
        backend.fgms_fusion_fwd_cuda(feats, weight, 0, out, kpos, None, imap, omap, False, arch80)
        ctx.save_for_backward(feats, weight, kpos, imap, omap)
        ctx.arch80 = arch80
        return out

    @staticmethod
    def backward(ctx, grad_out):
        feats, weight, kpos, imap, omap = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        in_grad = torch.zeros_like(feats)
        w_grad = torch.zeros_like(weight)
        backend.fgms_bwd_cuda(grad_out, feats, weight, 0, in_grad, w_grad, kpos, None, imap, omap, False, ctx.arch80)
        return in_grad, w_grad, None, None, None, None, None


def sparse_conv(feats: torch.Tensor, weight: torch.Tensor, kmap, arch80: bool = True) -> torch.Tensor:
    """``out[omap[j]] += feats[imap[j]] @ weight[k(j)]`` over the pairs of ``kmap``; differentiable."""
    if feats.size(0) != kmap.n_in:
        raise ValueError(f"feats has {feats.size(0)} rows, the kernel map expects {kmap.n_in}")
    if weight.size(0) != kmap.kpos.numel() - 1:
        raise ValueError("weight and kernel map disagree on the number of offsets")
    return _SparseConvFunction.apply(feats, weight, kmap.kpos, kmap.imap, kmap.omap, kmap.n_out, arch80)


def sparse_conv_inference(feats: torch.Tensor, weight: torch.Tensor, kmap, bias: torch.Tensor | None = None,
                          relu: bool = False, arch80: bool = True) -> torch.Tensor:
    """Forward only, through the output-stationary kernel (``backend.fgms_fwd_os_cuda``): every output row is
    written once — the same bits on every run — with ``bias`` and ReLU applied in the kernel's epilogue (a
    batch-norm layer in inference form is a scaled weight and a bias).  No autograd.  The neighbour table the
    kernel reads is built on first use and kept on ``kmap``.  Tensor-core shapes only (fp16, or fp32 storage
    with tf32 arithmetic; channel counts multiples of 16 up to 256)."""
    if feats.size(0) != kmap.n_in:
        raise ValueError(f"feats has {feats.size(0)} rows, the kernel map expects {kmap.n_in}")
    nbr = getattr(kmap, "_neighbor_table", None)
    if nbr is None:
        nbr = backend.build_neighbor_table(kmap.kpos, kmap.imap, kmap.omap, kmap.n_in, kmap.n_out)
        try:
            kmap._neighbor_table = nbr
        except AttributeError:  # a map type without room for it: rebuilt on every call
            pass
    out = torch.empty((kmap.n_out, weight.size(2)), dtype=feats.dtype, device=feats.device)
    with torch.no_grad():
        backend.fgms_fwd_os_cuda(feats.contiguous(), weight.detach().contiguous(), out, nbr, arch80, bias=bias, relu=relu)
    return out


class SparseConv3d(torch.nn.Module):
    """Sparse 3-D convolution layer with a ``[k_vol, c_in, c_out]`` weight (no bias, like the reference's
    operator); initialised like ``torch.nn.Conv3d`` (kaiming uniform, a = sqrt(5), fan_in = c_in * k_vol)."""

    def __init__(self, c_in: int, c_out: int, k_vol: int = 27, dtype=torch.float16, device="cuda", arch80: bool = True):
        super().__init__()
        self.c_in, self.c_out, self.k_vol, self.arch80 = c_in, c_out, k_vol, arch80
        bound = 1.0 / math.sqrt(c_in * k_vol)
        w = (torch.rand((k_vol, c_in, c_out), device=device, dtype=torch.float32) * 2 - 1) * bound
        self.weight = torch.nn.Parameter(w.to(dtype))

    def forward(self, feats: torch.Tensor, kmap) -> torch.Tensor:
        return sparse_conv(feats, self.weight, kmap, self.arch80)


class SparseUNet(torch.nn.Module):
    """The encoder-decoder stack of :mod:`fgms_b200.unet` as an ``nn.Module`` over the autograd operator: one
    :class:`SparseConv3d` per layer of the specification, decoder skips added to the transposed convolutions'
    outputs.  ``forward(feats, umaps)`` takes the kernel maps of all resolutions (``unet.build_unet_maps``)."""

    def __init__(self, spec, dtype=torch.float16, device="cuda", arch80: bool = True):
        super().__init__()
        self.spec = list(spec)
        self.layers = torch.nn.ModuleList(
            SparseConv3d(l.c_in, l.c_out, l.k_vol, dtype=dtype, device=device, arch80=arch80) for l in self.spec)

    def load_weights(self, weights):
        with torch.no_grad():
            for layer, w in zip(self.layers, weights):
                layer.weight.copy_(torch.as_tensor(w).to(layer.weight.device, layer.weight.dtype))

    def forward(self, feats: torch.Tensor, umaps) -> torch.Tensor:
        val = {"input": feats}
        for spec, layer in zip(self.spec, self.layers):
            y = layer(val[spec.src], umaps.of(spec))
            if spec.skip is not None:
                y = y + val[spec.skip]
            val[spec.dst] = y
        return val[self.spec[-1].dst]
