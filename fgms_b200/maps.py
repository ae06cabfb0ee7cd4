"""Host-side kernel-map construction and the index plumbing of the FGMS operator.

The FGMS operator consumes *kernel maps*: for every kernel offset ``k`` a list of
``(input row, output row)`` pairs, stored flat and offset-major in two int32
arrays ``imap`` / ``omap`` with ``kpos`` (exclusive prefix sum of the per-offset
pair counts ``knnz``) giving the start of each offset's slice.  The reference
loads these arrays from files (``spconv-test.py:63-73``) and never builds them;
this module builds them exactly on the host so that tests and the benchmark have
a canonical, bit-reproducible input for the CUDA path.

Canonical order produced here: offset-major; inside one offset, ascending output
row.  Offsets are enumerated lexicographically over ``(dx, dy, dz)`` so that for
an odd kernel volume the centre offset has index ``k_vol // 2`` — the index the
reference dispatch treats as the "mid" weight (``backend/spconv.cu:52``).

Also here: ``kpos_quantized`` and ``remove_mid``, re-statements of the two index
helpers every reference driver script carries (``cpu-check.py:6-14``,
``spconv-test.py:17-38``).
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import product

import numpy as np

__all__ = [
    "KernelMap",
    "build_submanifold_map",
    "build_strided_map",
    "transpose_map",
    "kpos_quantized",
    "remove_mid",
    "drop_centre",
    "unique_coords",
]

_COORD_BITS = 21  # coordinates are shifted to be non-negative and packed 21 bits each


@dataclass
class KernelMap:
    """Flat offset-major kernel map (all int32, C-contiguous)."""

    n_in: int
    n_out: int
    k_vol: int
    knnz: np.ndarray  # [k_vol]
    kpos: np.ndarray  # [k_vol + 1]
    imap: np.ndarray  # [P]
    omap: np.ndarray  # [P]
    out_coords: np.ndarray | None = None  # [n_out, 3]

    @property
    def pairs(self) -> int:
        return int(self.kpos[-1])

    def validate(self) -> None:
        assert self.knnz.dtype == np.int32 and self.kpos.dtype == np.int32
        assert self.imap.dtype == np.int32 and self.omap.dtype == np.int32
        assert self.kpos.shape == (self.k_vol + 1,) and self.kpos[0] == 0
        assert np.array_equal(np.diff(self.kpos), self.knnz)
        assert self.imap.shape == self.omap.shape == (self.pairs,)
        if self.pairs:
            assert 0 <= self.imap.min() and self.imap.max() < self.n_in
            assert 0 <= self.omap.min() and self.omap.max() < self.n_out


def _pack(coords: np.ndarray, lo: np.ndarray) -> np.ndarray:
    c = coords.astype(np.int64) - lo.astype(np.int64)
    assert (c >= 0).all() and (c < (1 << _COORD_BITS)).all(), "coordinate range too large"
    return (c[:, 0] << (2 * _COORD_BITS)) | (c[:, 1] << _COORD_BITS) | c[:, 2]


def unique_coords(coords: np.ndarray) -> np.ndarray:
    """Deduplicate integer voxel coordinates; result sorted lexicographically (x, y, z)."""
    coords = np.ascontiguousarray(coords, dtype=np.int32)
    if coords.shape[0] == 0:
        return coords.reshape(0, 3)
    return np.unique(coords, axis=0).astype(np.int32)


class _CoordTable:
    """Exact coordinate → row lookup (sorted packed keys + binary search)."""

    def __init__(self, coords: np.ndarray, lo: np.ndarray):
        self.lo = lo
        keys = _pack(coords, lo)
        self.order = np.argsort(keys, kind="stable")
        self.keys = keys[self.order]
        assert self.keys.size < 2 or (np.diff(self.keys) > 0).all(), "duplicate coordinates"

    def lookup(self, query: np.ndarray) -> np.ndarray:
        """Row index of each query coordinate, or -1 when absent."""
        if self.keys.size == 0 or query.shape[0] == 0:
            return np.full(query.shape[0], -1, dtype=np.int64)
        q = query.astype(np.int64) - self.lo.astype(np.int64)
        ok = ((q >= 0) & (q < (1 << _COORD_BITS))).all(axis=1)
        qk = (q[:, 0] << (2 * _COORD_BITS)) | (q[:, 1] << _COORD_BITS) | q[:, 2]
        pos = np.searchsorted(self.keys, qk)
        pos = np.minimum(pos, self.keys.size - 1)
        hit = ok & (self.keys[pos] == qk)
        return np.where(hit, self.order[pos], -1)


def _assemble(n_in, n_out, per_offset, out_coords) -> KernelMap:
    k_vol = len(per_offset)
    knnz = np.array([len(i) for i, _ in per_offset], dtype=np.int32)
    kpos = np.zeros(k_vol + 1, dtype=np.int32)
    np.cumsum(knnz, out=kpos[1:])
    if kpos[-1]:
        imap = np.concatenate([i for i, _ in per_offset]).astype(np.int32)
        omap = np.concatenate([o for _, o in per_offset]).astype(np.int32)
    else:
        imap = np.zeros(0, dtype=np.int32)
        omap = np.zeros(0, dtype=np.int32)
    km = KernelMap(int(n_in), int(n_out), k_vol, knnz, kpos,
                   np.ascontiguousarray(imap), np.ascontiguousarray(omap), out_coords)
    km.validate()
    return km


def build_submanifold_map(coords: np.ndarray, kernel_size: int = 3) -> KernelMap:
    """Stride-1 submanifold map: output coordinates are the input coordinates.

    Pair ``(i, o)`` belongs to offset ``d`` iff ``coords[i] == coords[o] + d``.
    ``d`` runs lexicographically over ``{-(ks//2) .. ks//2}^3``.
    """
    coords = np.ascontiguousarray(coords, dtype=np.int32)
    n = coords.shape[0]
    r = kernel_size // 2
    lo = (coords.min(axis=0) - r) if n else np.zeros(3, dtype=np.int32)
    table = _CoordTable(coords, lo)
    out_rows = np.arange(n, dtype=np.int64)
    per_offset = []
    for d in product(range(-r, kernel_size - r), repeat=3):
        src = table.lookup(coords + np.asarray(d, dtype=np.int32))
        hit = src >= 0
        per_offset.append((src[hit], out_rows[hit]))  # already ascending in output row
    return _assemble(n, n, per_offset, coords)


def build_strided_map(coords: np.ndarray, kernel_size: int = 2, stride: int = 2) -> KernelMap:
    """Downsampling map with ``kernel_size == stride``: every input has exactly one parent.

    Output coordinates are ``unique(coords // stride)`` (lexicographic order); the
    offset of a pair is ``coords[i] - stride * out[o]`` in ``[0, kernel_size)^3``,
    enumerated lexicographically.
    """
    assert kernel_size == stride, "only the non-overlapping downsample is needed by the path"
    coords = np.ascontiguousarray(coords, dtype=np.int32)
    n = coords.shape[0]
    parent = np.floor_divide(coords, stride).astype(np.int32)
    out_coords = unique_coords(parent)
    lo = out_coords.min(axis=0) if n else np.zeros(3, dtype=np.int32)
    out_row = _CoordTable(out_coords, lo).lookup(parent)
    assert (out_row >= 0).all()
    off = coords - parent * stride
    off_id = (off[:, 0].astype(np.int64) * kernel_size + off[:, 1]) * kernel_size + off[:, 2]
    in_rows = np.arange(n, dtype=np.int64)
    per_offset = []
    for k in range(kernel_size ** 3):
        sel = np.nonzero(off_id == k)[0]
        sel = sel[np.argsort(out_row[sel], kind="stable")]
        per_offset.append((in_rows[sel], out_row[sel]))
    return _assemble(n, out_coords.shape[0], per_offset, out_coords)


def transpose_map(km: KernelMap, out_coords: np.ndarray | None = None) -> KernelMap:
    """Map of the transposed convolution: the same pairs with input and output swapped,
    re-sorted inside each offset so the canonical order (ascending output row) holds."""
    per_offset = []
    for k in range(km.k_vol):
        a, b = int(km.kpos[k]), int(km.kpos[k + 1])
        new_in, new_out = km.omap[a:b].astype(np.int64), km.imap[a:b].astype(np.int64)
        order = np.argsort(new_out, kind="stable")
        per_offset.append((new_in[order], new_out[order]))
    return _assemble(km.n_out, km.n_in, per_offset, out_coords)


def drop_centre(km: KernelMap) -> KernelMap:
    """Remove the centre offset's pairs (the form the reference's data files use for
    submanifold layers, to be combined with ``separate_mid=True``: ``cpu-check.py:96,39-43``)."""
    mid = km.k_vol // 2 if km.k_vol % 2 == 1 else 0
    per_offset = []
    for k in range(km.k_vol):
        a, b = int(km.kpos[k]), int(km.kpos[k + 1])
        if k == mid:
            a = b
        per_offset.append((km.imap[a:b].astype(np.int64), km.omap[a:b].astype(np.int64)))
    return _assemble(km.n_in, km.n_out, per_offset, km.out_coords)


def kpos_quantized(knnz, kpos, k_vol: int, q: int = 256):
    """Prefix sums of ``knnz`` rounded up to multiples of ``q`` per offset.

    Same arithmetic as ``kpos_quantized`` in ``cpu-check.py:6-14``: a tile of ``q``
    (or a divisor of ``q``) padded rows never straddles two offsets.  Returns
    ``(qkpos int32[k_vol+1], qsum_nnz)``.
    """
    knnz = np.asarray(knnz, dtype=np.int64)
    qk = np.zeros(k_vol + 1, dtype=np.int64)
    qk[1:] = np.cumsum((knnz[:k_vol] + q - 1) // q * q)
    assert qk[-1] < 2 ** 31
    return qk.astype(np.int32), int(qk[-1])


def remove_mid(nnz: int, km: KernelMap, q: int = 256):
    """Re-insert an identity map for the centre offset of a map that omits it.

    Mirrors ``remove_mid`` in ``spconv-test.py:17-38``: the benchmark turns
    ``separate_mid=True`` layers into plain fused layers by giving the centre
    offset the pairs ``(i, i)`` for all ``nnz`` rows.  Returns
    ``(qkpos, qsum_nnz, KernelMap)``.  The reference replaces the centre count only
    when it was zero; a map that already holds centre pairs is returned unchanged
    here (the reference would leave its arrays inconsistent in that case).
    """
    mid = km.k_vol // 2 if km.k_vol % 2 == 1 else 0
    change = int(km.kpos[mid])
    knnz = km.knnz.copy()
    imap, omap = km.imap, km.omap
    if knnz[mid] == 0:
        ident = np.arange(nnz, dtype=np.int32)
        imap = np.concatenate([km.imap[:change], ident, km.imap[change:]]).astype(np.int32)
        omap = np.concatenate([km.omap[:change], ident, km.omap[change:]]).astype(np.int32)
        knnz[mid] = nnz
    kpos = np.zeros(km.k_vol + 1, dtype=np.int32)
    np.cumsum(knnz, out=kpos[1:])
    qkpos, qsum = kpos_quantized(knnz, kpos, km.k_vol, q)
    new = KernelMap(km.n_in, km.n_out, km.k_vol, knnz, kpos, imap, omap, km.out_coords)
    return qkpos, qsum, new
