"""Helpers shared by the GPU parity tests: build a seeded problem, run the CUDA operator through
the public binding, and get the fp64 oracle answer for the same inputs."""
from __future__ import annotations

import numpy as np
import torch

from fgms_b200 import clouds, maps
from fgms_b200.workloads import LayerTensors
from oracle import spconv_oracle as orc

# parity bounds of the task: max-abs error over the tensor, normalised by max |reference|
TOL = {"fp32": 1e-5, "tf32": 5e-3, "fp16": 1e-2}


def mode_dtype(mode):
    return torch.float16 if mode == "fp16" else torch.float32


def mode_arch80(mode):
    return mode != "fp32"


class Problem(LayerTensors):
    """A layer's device tensors plus the oracle answers for them."""

    # --- oracle (fp64 on the stored, i.e. already rounded, inputs) ---
    def ref_fwd(self, precompute=False):
        return orc.fwd(self.f_np, self.w_np, self.km.n_out, self.km.kpos, self.km.imap, self.km.omap, precompute)

    def ref_dgrad(self):
        return orc.dgrad(self.g_np, self.w_np, self.km.n_in, self.km.kpos, self.km.imap, self.km.omap)

    def ref_wgrad(self):
        return orc.wgrad(self.f_np, self.g_np, self.km.k_vol, self.km.kpos, self.km.imap, self.km.omap)

    # --- CUDA path ---
    def run_fwd(self, separate_mid=False, fused=True, out=None):
        from fgms_b200 import backend
        if out is None:
            out = torch.zeros((self.km.n_out, self.c_out), dtype=self.dtype, device=self.feats.device)
        if fused:
            backend.fgms_fusion_fwd_cuda(self.feats, self.weights, self.qsum, out, self.kpos, self.qkpos,
                                         self.imap, self.omap, separate_mid, self.arch80)
        else:
            backend.fgms_fwd_cuda(self.feats, self.weights, self.km.pairs, out, torch.from_numpy(self.km.knnz),
                                  self.kpos, self.imap, self.omap, separate_mid, self.arch80)
        return out

    def run_bwd(self):
        from fgms_b200 import backend
        in_grad = torch.zeros((self.km.n_in, self.c_in), dtype=self.dtype, device=self.feats.device)
        w_grad = torch.zeros_like(self.weights)
        backend.fgms_bwd_cuda(self.grad_out, self.feats, self.weights, self.qsum, in_grad, w_grad, self.kpos,
                              self.qkpos, self.imap, self.omap, False, self.arch80)
        return in_grad, w_grad


def err(got: torch.Tensor, ref: np.ndarray) -> float:
    return orc.rel_err(got.detach().float().cpu().numpy().astype(np.float64), ref)
