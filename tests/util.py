"""Helpers shared by the GPU parity tests: build a seeded problem, run the CUDA operator through
the public binding, and get the fp64 oracle answer for the same inputs."""
from __future__ import annotations

import numpy as np
import torch

from fgms_b200 import clouds, maps
from oracle import spconv_oracle as orc

# parity bounds of the task: max-abs error over the tensor, normalised by max |reference|
TOL = {"fp32": 1e-5, "tf32": 5e-3, "fp16": 1e-2}


def mode_dtype(mode):
    return torch.float16 if mode == "fp16" else torch.float32


def mode_arch80(mode):
    return mode != "fp32"


class Problem:
    def __init__(self, km: maps.KernelMap, c_in: int, c_out: int, seed: int, mode: str, device="cuda"):
        self.km, self.c_in, self.c_out, self.mode = km, c_in, c_out, mode
        npdt = np.float16 if mode == "fp16" else np.float32
        f, w, g = clouds.make_tensors(km.n_in, km.n_out, c_in, c_out, km.k_vol, seed, npdt)
        self.f_np, self.w_np, self.g_np = f, w, g
        dev = torch.device(device)
        self.feats = torch.from_numpy(f).to(dev)
        self.weights = torch.from_numpy(w).to(dev)
        self.grad_out = torch.from_numpy(g).to(dev)
        self.kpos = torch.from_numpy(km.kpos).to(dev)
        self.imap = torch.from_numpy(km.imap).to(dev)
        self.omap = torch.from_numpy(km.omap).to(dev)
        self.qkpos_np, self.qsum = maps.kpos_quantized(km.knnz, km.kpos, km.k_vol, 256)
        self.qkpos = torch.from_numpy(self.qkpos_np).to(dev)
        self.dtype = mode_dtype(mode)
        self.arch80 = mode_arch80(mode)

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
