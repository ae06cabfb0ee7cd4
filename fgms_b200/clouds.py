"""Seeded synthetic voxel clouds that stand in for the reference's downloaded sample maps.

The reference benchmarks on kernel maps extracted from public point-cloud
datasets (``spconv-test.py:42,51-52``; fetched by ``download_data.sh``), which are
not redistributable here.  These generators produce clouds with the same
character — thin surfaces in a large empty grid, and a rotating-LiDAR sweep —
from a seed alone, so every number is reproducible without any dataset.

Every generator returns unique int32 voxel coordinates ``[N, 3]`` sorted
lexicographically; features, weights and gradients come from ``make_tensors``.
"""
from __future__ import annotations

import math

import numpy as np

from .maps import unique_coords

__all__ = ["uniform_cloud", "surface_cloud", "lidar_cloud", "make_tensors", "kaiming_uniform_bound"]


def uniform_cloud(n: int, grid: int, seed: int) -> np.ndarray:
    """``n`` unique coordinates drawn uniformly in ``[0, grid)^3``."""
    rng = np.random.default_rng(seed)
    assert n <= grid ** 3
    got = np.zeros((0, 3), dtype=np.int32)
    while got.shape[0] < n:
        extra = rng.integers(0, grid, size=(int((n - got.shape[0]) * 1.2) + 16, 3), dtype=np.int64)
        got = unique_coords(np.concatenate([got, extra.astype(np.int32)]))
    if got.shape[0] > n:
        keep = np.sort(rng.choice(got.shape[0], size=n, replace=False))
        got = got[keep]
    return np.ascontiguousarray(got)


def surface_cloud(target: int, grid: int, seed: int, n_planes: int = 12, n_boxes: int = 20) -> np.ndarray:
    """Indoor-surface-like cloud: points on random planes and on the faces of random
    axis-aligned boxes inside ``[0, grid)^3`` at unit voxel size, deduplicated.

    The shapes are drawn once from the seed; their common scale is then grown until the
    densely sampled surfaces hold at least ``target`` voxels, and the surplus (a few per
    cent) is thinned at random, so surfaces stay nearly filled and each voxel keeps the
    many in-plane neighbours real scans have."""
    rng = np.random.default_rng(seed)
    planes = []
    for _ in range(n_planes):
        nrm = rng.normal(size=3)
        nrm /= np.linalg.norm(nrm)
        u = np.cross(nrm, [1.0, 0.0, 0.0] if abs(nrm[0]) < 0.9 else [0.0, 1.0, 0.0])
        u /= np.linalg.norm(u)
        v = np.cross(nrm, u)
        centre = rng.uniform(0.3, 0.7, size=3)
        planes.append((centre, u, v, rng.uniform(0.5, 1.0)))
    boxes = []
    for _ in range(n_boxes):
        size = rng.uniform(0.3, 1.0, size=3)
        centre = rng.uniform(0.2, 0.8, size=3)
        boxes.append((centre, size))
    plane_area = sum((2 * e) ** 2 for *_, e in planes)
    box_area = sum(2 * (s[0] * s[1] + s[1] * s[2] + s[0] * s[2]) for _, s in boxes)
    # unit-scale area -> scale (in voxels) at which the total area is ~1.1x the target
    scale = math.sqrt(1.1 * target / (plane_area + box_area))

    def sample(scale: float) -> np.ndarray:
        pts = []
        for centre, u, v, ext in planes:
            e = ext * scale
            m = int(6 * (2 * e) ** 2) + 8
            a = rng.uniform(-e, e, size=(m, 1))
            b = rng.uniform(-e, e, size=(m, 1))
            pts.append(centre * grid + a * u + b * v)
        for centre, size in boxes:
            sz = size * scale
            lo = centre * grid - sz / 2
            m = int(6 * 2 * (sz[0] * sz[1] + sz[1] * sz[2] + sz[0] * sz[2])) + 8
            p = lo + rng.uniform(0, 1, size=(m, 3)) * sz
            face = rng.integers(0, 6, size=m)
            ax = face % 3
            p[np.arange(m), ax] = lo[ax] + (face // 3) * sz[ax]
            pts.append(p)
        p = np.concatenate(pts)
        p = p[((p >= 0) & (p < grid)).all(axis=1)]
        return unique_coords(np.floor(p).astype(np.int32))

    got = sample(scale)
    tries = 0
    while got.shape[0] < target and tries < 40:
        scale *= 1.05
        got = sample(scale)
        tries += 1
    if got.shape[0] > target:
        keep = np.sort(rng.choice(got.shape[0], size=target, replace=False))
        got = got[keep]
    return np.ascontiguousarray(got)


def lidar_cloud(seed: int, beams: int = 64, azimuths: int = 2048, voxel: float = 0.05,
                elev_deg=(-25.0, 3.0), range_median: float = 15.0, range_sigma: float = 0.6,
                range_clip=(1.0, 80.0), ground_z: float = -1.7,
                bounds=((-50.0, 50.0), (-50.0, 50.0), (-3.0, 1.0)), sweeps: int = 1) -> np.ndarray:
    """Rotating-scanner cloud: ``beams`` elevations uniform over ``elev_deg``, ``azimuths``
    steps per sweep, log-normal ranges clipped to ``range_clip``, rays stopped by a ground
    plane at ``ground_z``; voxelised at ``voxel`` metres inside ``bounds``.  ``sweeps`` > 1
    overlays jittered sweeps (denser cloud of the same geometry)."""
    rng = np.random.default_rng(seed)
    elev = np.deg2rad(np.linspace(elev_deg[0], elev_deg[1], beams))
    pts = []
    for s in range(sweeps):
        az = (np.arange(azimuths) + rng.uniform(0, 1)) * (2 * math.pi / azimuths)
        e, a = np.meshgrid(elev, az, indexing="ij")
        rr = np.exp(rng.normal(math.log(range_median), range_sigma, size=e.shape))
        rr = np.clip(rr, range_clip[0], range_clip[1])
        dz = np.sin(e)
        with np.errstate(divide="ignore", invalid="ignore"):
            r_ground = np.where(dz < 0, ground_z / dz, np.inf)
        rr = np.minimum(rr, r_ground)
        x = rr * np.cos(e) * np.cos(a)
        y = rr * np.cos(e) * np.sin(a)
        z = rr * dz
        pts.append(np.stack([x.ravel(), y.ravel(), z.ravel()], axis=1))
    p = np.concatenate(pts)
    b = np.asarray(bounds)
    inside = ((p >= b[:, 0]) & (p < b[:, 1])).all(axis=1)
    p = p[inside]
    vox = np.floor((p - b[:, 0]) / voxel).astype(np.int32)
    return np.ascontiguousarray(unique_coords(vox))


def kaiming_uniform_bound(c_in: int, k_vol: int) -> float:
    """Bound of the kaiming-uniform weight initialisation with ``a = sqrt(5)`` and the
    convolution convention ``fan_in = c_in * k_vol``: ``U(-1/sqrt(fan_in), 1/sqrt(fan_in))``."""
    return 1.0 / math.sqrt(c_in * k_vol)


def make_tensors(n_in: int, n_out: int, c_in: int, c_out: int, k_vol: int, seed: int,
                 dtype=np.float32):
    """Features ``N(0,1) [n_in, c_in]``, weights kaiming-uniform ``[k_vol, c_in, c_out]`` and an
    output gradient ``N(0,1) [n_out, c_out]``, all from one seed, cast to ``dtype``."""
    rng = np.random.default_rng(seed)
    feats = rng.standard_normal((n_in, c_in), dtype=np.float32)
    bound = kaiming_uniform_bound(c_in, k_vol)
    weights = rng.uniform(-bound, bound, size=(k_vol, c_in, c_out)).astype(np.float32)
    grad_out = rng.standard_normal((n_out, c_out), dtype=np.float32)
    return feats.astype(dtype), weights.astype(dtype), grad_out.astype(dtype)
