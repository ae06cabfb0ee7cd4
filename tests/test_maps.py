"""Kernel-map builder against a brute-force dictionary lookup, and the index helpers
against the reference's own outputs stored in the golden fixtures."""
from itertools import product

import numpy as np
import pytest

from fgms_b200 import clouds, maps


def _brute_submanifold(coords, ks=3):
    table = {tuple(c): i for i, c in enumerate(coords.tolist())}
    r = ks // 2
    imap, omap, knnz = [], [], []
    for d in product(range(-r, ks - r), repeat=3):
        cnt = 0
        for o, c in enumerate(coords.tolist()):
            i = table.get((c[0] + d[0], c[1] + d[1], c[2] + d[2]))
            if i is not None:
                imap.append(i)
                omap.append(o)
                cnt += 1
        knnz.append(cnt)
    return np.array(knnz, np.int32), np.array(imap, np.int32), np.array(omap, np.int32)


@pytest.mark.parametrize("n,grid,seed", [(1, 4, 0), (50, 4, 1), (400, 9, 2), (64, 4, 3)])
def test_submanifold_map_is_exact(n, grid, seed):
    coords = clouds.uniform_cloud(n, grid, seed)
    km = maps.build_submanifold_map(coords)
    knnz, imap, omap = _brute_submanifold(coords)
    assert np.array_equal(km.knnz, knnz)
    assert np.array_equal(km.imap, imap)
    assert np.array_equal(km.omap, omap)
    assert km.knnz[13] == n  # the centre offset is the identity
    a, b = km.kpos[13], km.kpos[14]
    assert np.array_equal(km.imap[a:b], np.arange(n)) and np.array_equal(km.omap[a:b], np.arange(n))


def test_negative_coordinates_and_empty_cloud():
    coords = maps.unique_coords(np.array([[-3, 0, 5], [-2, 0, 5], [-3, 1, 5], [7, -9, -1]], np.int32))
    km = maps.build_submanifold_map(coords)
    knnz, imap, omap = _brute_submanifold(coords)
    assert np.array_equal(km.imap, imap) and np.array_equal(km.omap, omap) and np.array_equal(km.knnz, knnz)
    empty = maps.build_submanifold_map(np.zeros((0, 3), np.int32))
    assert empty.pairs == 0 and empty.k_vol == 27 and empty.kpos.shape == (28,)
    assert maps.build_strided_map(np.zeros((0, 3), np.int32)).n_out == 0


def test_strided_and_transposed_maps():
    coords = clouds.uniform_cloud(300, 10, 5)
    km = maps.build_strided_map(coords)
    assert km.pairs == 300 and km.k_vol == 8
    parents = {tuple(c): i for i, c in enumerate(km.out_coords.tolist())}
    seen = np.zeros(300, bool)
    for k in range(8):
        d = np.array([(k >> 2) & 1, (k >> 1) & 1, k & 1])
        sl = slice(km.kpos[k], km.kpos[k + 1])
        for i, o in zip(km.imap[sl], km.omap[sl]):
            assert np.array_equal(coords[i] - 2 * km.out_coords[o], d)
            assert parents[tuple((coords[i] // 2).tolist())] == o
            seen[i] = True
        assert (np.diff(km.omap[sl]) > 0).all()  # canonical order, unique output per offset
    assert seen.all()
    kt = maps.transpose_map(km, coords)
    assert kt.n_in == km.n_out and kt.n_out == km.n_in and np.array_equal(kt.knnz, km.knnz)
    for k in range(8):
        sl = slice(km.kpos[k], km.kpos[k + 1])
        assert set(zip(kt.imap[sl].tolist(), kt.omap[sl].tolist())) == set(zip(km.omap[sl].tolist(), km.imap[sl].tolist()))
        assert (np.diff(kt.omap[sl]) > 0).all()


def test_kpos_quantized_matches_reference(golden):
    qkpos, qsum = maps.kpos_quantized(golden["knnz"], golden["kpos"], golden["knnz"].shape[0], 256)
    assert np.array_equal(qkpos, golden["qkpos"]) and qsum == int(golden["qsum"])


def test_remove_mid_matches_reference(golden):
    if "rm_imap" not in golden:
        pytest.skip("fixture has a centre offset")
    g = golden
    k_vol = g["knnz"].shape[0]
    km = maps.KernelMap(int(g["n_in"]), int(g["n_out"]), k_vol, g["knnz"], g["kpos"], g["imap"], g["omap"])
    qkpos, qsum, new = maps.remove_mid(int(g["n_in"]), km, 256)
    assert np.array_equal(qkpos, g["rm_qkpos"]) and qsum == int(g["rm_qsum"])
    assert np.array_equal(new.kpos, g["rm_kpos"])
    assert np.array_equal(new.imap, g["rm_imap"]) and np.array_equal(new.omap, g["rm_omap"])
    new.validate()
    # and it equals the full submanifold map built directly
    full = maps.build_submanifold_map(g["coords"])
    assert np.array_equal(new.imap, full.imap) and np.array_equal(new.omap, full.omap)


def test_generators_are_seeded_and_unique():
    a = clouds.surface_cloud(5000, 64, 3)
    b = clouds.surface_cloud(5000, 64, 3)
    assert np.array_equal(a, b) and a.shape == (5000, 3)
    assert np.unique(a, axis=0).shape[0] == 5000
    lid = clouds.lidar_cloud(1, beams=8, azimuths=128)
    assert lid.dtype == np.int32 and np.unique(lid, axis=0).shape[0] == lid.shape[0]
    km = maps.build_submanifold_map(a)
    assert km.pairs / km.n_in > 4  # surfaces keep their in-plane neighbours
