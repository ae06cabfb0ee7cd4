"""Kernel maps built on the GPU (``csrc/map_builder.cuh`` through the C ABI).

Same canonical form, bit for bit, as the host builders in :mod:`fgms_b200.maps`; the results stay on
the device as int32 tensors, ready for ``fgms_fusion_fwd_cuda`` / ``fgms_bwd_cuda``.  The reference has
no map builder (it loads maps from files, ``spconv-test.py:63-73``).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib

_L = _lib.lib

__all__ = ["DeviceKernelMap", "build_submanifold_map", "build_strided_map", "transpose_map"]


@dataclass
class DeviceKernelMap:
    """Flat offset-major kernel map on the device (all int32)."""

    n_in: int
    n_out: int
    k_vol: int
    kpos: torch.Tensor   # [k_vol + 1]
    imap: torch.Tensor   # [pairs]
    omap: torch.Tensor   # [pairs]
    out_coords: torch.Tensor | None = None  # [n_out, 3]

    @property
    def pairs(self) -> int:
        return int(self.imap.numel())


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


def _check_coords(coords: torch.Tensor) -> torch.Tensor:
    if not (coords.is_cuda and coords.dtype == torch.int32 and coords.dim() == 2 and coords.size(1) == 3):
        raise ValueError("coords must be a CUDA int32 tensor of shape [n, 3]")
    return coords.contiguous()


def _workspace(n: int, n_cols: int, k_vol: int, device) -> torch.Tensor:
    nbytes = _L.fgms_b200_map_workspace_bytes(n, n_cols, k_vol)
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


def build_submanifold_map(coords: torch.Tensor, kernel_size: int = 3) -> DeviceKernelMap:
    """Stride-1 map: pair ``(i, o)`` in offset ``d`` iff ``coords[i] == coords[o] + d``."""
    coords = _check_coords(coords)
    n, k_vol, dev = coords.size(0), kernel_size ** 3, coords.device
    kpos = torch.empty(k_vol + 1, dtype=torch.int32, device=dev)
    imap = torch.empty(n * k_vol, dtype=torch.int32, device=dev)
    omap = torch.empty(n * k_vol, dtype=torch.int32, device=dev)
    ws = _workspace(n, n, k_vol, dev)
    pairs = ctypes.c_int64(0)
    with torch.cuda.device(dev):
        _lib.check(_L.fgms_b200_build_submanifold_map(_ptr(coords), n, kernel_size, kpos.data_ptr(), _ptr(imap), _ptr(omap),
                                                       ws.data_ptr(), ws.numel(), ctypes.addressof(pairs), _stream()))
    p = int(pairs.value)
    return DeviceKernelMap(n, n, k_vol, kpos, imap[:p], omap[:p], coords)


def build_strided_map(coords: torch.Tensor, stride: int = 2) -> DeviceKernelMap:
    """Downsampling map with ``kernel_size == stride``; output voxels are the distinct ``coords // stride``."""
    coords = _check_coords(coords)
    n, k_vol, dev = coords.size(0), stride ** 3, coords.device
    kpos = torch.empty(k_vol + 1, dtype=torch.int32, device=dev)
    imap = torch.empty(n, dtype=torch.int32, device=dev)
    omap = torch.empty(n, dtype=torch.int32, device=dev)
    out_coords = torch.empty((n, 3), dtype=torch.int32, device=dev)
    ws = _workspace(n, n, k_vol, dev)
    n_out = ctypes.c_int(0)
    with torch.cuda.device(dev):
        _lib.check(_L.fgms_b200_build_strided_map(_ptr(coords), n, stride, _ptr(out_coords), kpos.data_ptr(), _ptr(imap),
                                                   _ptr(omap), ws.data_ptr(), ws.numel(), ctypes.addressof(n_out), _stream()))
    return DeviceKernelMap(n, int(n_out.value), k_vol, kpos, imap, omap, out_coords[: int(n_out.value)])


def transpose_map(km: DeviceKernelMap, out_coords: torch.Tensor | None = None) -> DeviceKernelMap:
    """Map of the transposed convolution: the same pairs with input and output swapped."""
    dev = km.kpos.device
    kpos = torch.empty_like(km.kpos)
    imap = torch.empty_like(km.imap)
    omap = torch.empty_like(km.omap)
    ws = _workspace(0, km.n_in, km.k_vol, dev)
    with torch.cuda.device(dev):
        _lib.check(_L.fgms_b200_transpose_map(km.kpos.data_ptr(), _ptr(km.imap), _ptr(km.omap), km.n_in, km.k_vol, km.pairs,
                                              kpos.data_ptr(), _ptr(imap), _ptr(omap), ws.data_ptr(), ws.numel(), _stream()))
    return DeviceKernelMap(km.n_out, km.n_in, km.k_vol, kpos, imap, omap, out_coords)
