"""Named benchmark workloads: the synthetic stand-ins for the reference's sample layers.

Each workload is one sparse-convolution layer (cloud → kernel map, channel counts, arithmetic
mode).  The clouds are seeded, so the exact voxel and pair counts are reproducible; they are
recorded with every result.

================  =====================================================================
``cfg1``          8 000 voxels uniform in 64^3, 3x3x3 submanifold, fp32 16→16
``cfg2``          ~100 k-voxel indoor-surface cloud in 256^3, 3x3x3 submanifold, fp16 64→64
``cfg3a``         ~200 k-voxel surface cloud in 512^3, 2x2x2 stride-2 downsample, tf32 32→64
``cfg3b``         the transposed 2x2x2 convolution back to the fine voxels, tf32 64→32
``cfg4``          two overlaid 64-beam LiDAR sweeps voxelised at 5 cm (~145 k voxels),
                  3x3x3 submanifold, fp16 128→128
``cfg5l0``        the finest-resolution layer of the cfg5 stack on its own: ~120 k-voxel surface
                  cloud, 3x3x3 submanifold, fp16 32→32 (small channels: gather-bound)
================  =====================================================================

``cfg5`` is not one layer but a stack (``unet_workload``): the MinkUNet-style encoder-decoder of
:mod:`fgms_b200.unet` over a batch of ~120 k-voxel surface scenes, fp16.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

from . import clouds, maps

__all__ = ["Workload", "LayerTensors", "get", "NAMES", "flops", "algorithmic_bytes", "UNetWorkload", "unet_workload",
           "layer_bytes"]

NAMES = ("cfg1", "cfg2", "cfg3a", "cfg3b", "cfg4", "cfg5l0")


@dataclass(frozen=True)
class Workload:
    name: str
    description: str
    kmap: maps.KernelMap
    c_in: int
    c_out: int
    mode: str  # "fp32" | "tf32" | "fp16"
    seed: int

    @property
    def elem_bytes(self) -> int:
        return 2 if self.mode == "fp16" else 4


@lru_cache(maxsize=None)
def get(name: str, seed_offset: int = 0) -> Workload:
    """Build (and cache) a workload.  ``seed_offset`` gives an independent scene of the same
    kind — one per rank in multi-GPU runs."""
    s = seed_offset
    if name == "cfg1":
        km = maps.build_submanifold_map(clouds.uniform_cloud(8000, 64, 101 + s))
        return Workload(name, "uniform 8k voxels in 64^3, subm 3x3x3, fp32 16->16", km, 16, 16, "fp32", 101 + s)
    if name == "cfg2":
        km = maps.build_submanifold_map(clouds.surface_cloud(100_000, 256, 102 + s))
        return Workload(name, "indoor-surface ~100k voxels in 256^3, subm 3x3x3, fp16 64->64", km, 64, 64, "fp16", 102 + s)
    if name in ("cfg3a", "cfg3b"):
        coords = clouds.surface_cloud(200_000, 512, 103 + s)
        down = maps.build_strided_map(coords, 2, 2)
        if name == "cfg3a":
            return Workload(name, "surface ~200k voxels in 512^3, 2x2x2 stride 2, tf32 32->64", down, 32, 64, "tf32", 103 + s)
        up = maps.transpose_map(down, coords)
        return Workload(name, "transposed 2x2x2 back to ~200k voxels, tf32 64->32", up, 64, 32, "tf32", 103 + s)
    if name == "cfg4":
        km = maps.build_submanifold_map(clouds.lidar_cloud(104 + s, sweeps=2))
        return Workload(name, "64-beam LiDAR, 2 sweeps, 5 cm voxels (~145k), subm 3x3x3, fp16 128->128", km, 128, 128, "fp16", 104 + s)
    if name == "cfg5l0":
        # one layer of the cfg5 stack on its own: the finest-resolution 32 -> 32 submanifold convolution (the small-channel,
        # gather-bound shape that dominates the stack's step), on the first scene of the stack's batch
        km = maps.build_submanifold_map(clouds.surface_cloud(120_000, 256, 105 + 17 * (s // 1000)))
        return Workload(name, "cfg5 finest level: surface ~120k voxels in 256^3, subm 3x3x3, fp16 32->32", km, 32, 32, "fp16", 105 + s)
    raise KeyError(name)


def flops(wl: Workload, passes: int = 3) -> float:
    """Effective flops: 2 * pairs * c_in * c_out per pass (forward, dgrad, wgrad)."""
    return 2.0 * wl.kmap.pairs * wl.c_in * wl.c_out * passes


def algorithmic_bytes(wl: Workload, which: str) -> float:
    """Algorithmic bytes of one pass under the gathered-bytes model: every pair reads one
    gathered row and updates one scattered row, both maps are read once, weights once.
    ``which``: "fwd" | "dgrad" | "wgrad" | "all"."""
    p, s = wl.kmap.pairs, wl.elem_bytes
    w_elems = wl.kmap.k_vol * wl.c_in * wl.c_out
    gms = p * (wl.c_in + wl.c_out) * s + 8 * p + w_elems * s
    wg = p * (wl.c_in + wl.c_out) * s + 8 * p + w_elems * 4
    return {"fwd": gms, "dgrad": gms, "wgrad": wg, "all": 2 * gms + wg}[which]


class LayerTensors:
    """Seeded device tensors of one layer: features, weights, output gradient and the kernel map,
    laid out as the operator expects them (``mode``: "fp32" | "tf32" | "fp16")."""

    def __init__(self, km: maps.KernelMap, c_in: int, c_out: int, seed: int, mode: str, device="cuda"):
        import numpy as np
        import torch
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
        self.dtype = torch.float16 if mode == "fp16" else torch.float32
        self.arch80 = mode != "fp32"  # the reference's flag: tensor cores for fp32 storage


# ---------------------------------------------------------------------------------------------
# cfg5: the encoder-decoder stack
# ---------------------------------------------------------------------------------------------
SCENE_PITCH = 4096  # scenes of a batch are placed this far apart along x: no kernel offset or parent voxel is shared


@dataclass(frozen=True)
class UNetWorkload:
    """Inputs of one step of the stack: batched voxel coordinates, input features ``[n, c_in]`` and the gradient
    of the output ``[n, widths[0]]`` (both fp16, seeded).  Weights come from ``unet.unet_weights`` once the maps exist."""

    name: str
    description: str
    coords: object     # int32 [n, 3], unique, sorted lexicographically
    feats: object      # float16 [n, c_in]
    grad_out: object   # float16 [n, widths[0]]
    scenes: int
    seed: int
    c_in: int = 4
    widths: tuple = (32, 32, 64, 128, 256)


@lru_cache(maxsize=None)
def unet_workload(scenes: int = 1, first_scene: int = 0, voxels: int = 120_000, grid: int = 256, seed: int = 105) -> UNetWorkload:
    """``scenes`` surface scenes of about ``voxels`` voxels each (the cfg2 generator, one seed per scene) batched
    into one cloud; ``first_scene`` selects which scenes of the global batch (one per rank in multi-GPU runs)."""
    import numpy as np
    parts = []
    for s in range(first_scene, first_scene + scenes):
        c = clouds.surface_cloud(voxels, grid, seed + 17 * s).copy()
        c[:, 0] += SCENE_PITCH * (s - first_scene)
        parts.append(c)
    coords = maps.unique_coords(np.concatenate(parts))
    rng = np.random.default_rng(seed + 1000 * first_scene + scenes)
    n = coords.shape[0]
    feats = rng.standard_normal((n, 4), dtype=np.float32).astype(np.float16)
    grad_out = (0.25 * rng.standard_normal((n, 32), dtype=np.float32)).astype(np.float16)
    return UNetWorkload("cfg5", f"MinkUNet-style stack (stem 4->32, stages 32/64/128/256, mirrored decoder, 25 layers), "
                        f"{scenes} surface scene(s) of ~{voxels // 1000}k voxels in {grid}^3, fp16",
                        coords, feats, grad_out, scenes, seed)


def layer_bytes(pairs: int, c_in: int, c_out: int, k_vol: int, elem: int, which: str) -> float:
    """Algorithmic bytes of one pass of a layer (same model as ``algorithmic_bytes``)."""
    w = k_vol * c_in * c_out
    return pairs * (c_in + c_out) * elem + 8 * pairs + w * (4 if which == "wgrad" else elem)
