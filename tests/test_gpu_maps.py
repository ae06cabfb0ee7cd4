"""The GPU kernel-map builders against the host builders of fgms_b200/maps.py: bit-exact."""
import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps

pytestmark = pytest.mark.gpu


def _same(dk, hk):
    assert (dk.n_in, dk.n_out, dk.k_vol) == (hk.n_in, hk.n_out, hk.k_vol)
    assert np.array_equal(dk.kpos.cpu().numpy(), hk.kpos)
    assert np.array_equal(dk.imap.cpu().numpy(), hk.imap)
    assert np.array_equal(dk.omap.cpu().numpy(), hk.omap)


def _dev(coords):
    return torch.from_numpy(np.ascontiguousarray(coords, dtype=np.int32)).cuda()


CLOUDS = {
    "uniform": lambda: clouds.uniform_cloud(5000, 40, 3),
    "uniform_dense": lambda: clouds.uniform_cloud(6000, 20, 4),
    "surface": lambda: clouds.surface_cloud(20000, 128, 5),
    "lidar": lambda: clouds.lidar_cloud(6, sweeps=1),
    "negative": lambda: clouds.uniform_cloud(3000, 30, 7) - np.array([17, 900, 5], dtype=np.int32),
    "single": lambda: np.array([[3, -2, 7]], dtype=np.int32),
    "empty": lambda: np.zeros((0, 3), dtype=np.int32),
}


@pytest.mark.parametrize("name", list(CLOUDS))
@pytest.mark.parametrize("ks", [3, 5])
def test_submanifold(name, ks):
    from fgms_b200 import backend, gpu_maps
    coords = CLOUDS[name]()
    if ks == 5 and coords.shape[0] > 8000:
        coords = coords[:8000]
    backend.device_status(reset=True)
    dk = gpu_maps.build_submanifold_map(_dev(coords), ks)
    assert backend.device_status() == 0
    _same(dk, maps.build_submanifold_map(coords, ks))


@pytest.mark.parametrize("name", list(CLOUDS))
@pytest.mark.parametrize("stride", [2, 3])
def test_strided_and_transposed(name, stride):
    from fgms_b200 import backend, gpu_maps
    coords = CLOUDS[name]()
    backend.device_status(reset=True)
    dk = gpu_maps.build_strided_map(_dev(coords), stride)
    hk = maps.build_strided_map(coords, stride, stride)
    _same(dk, hk)
    assert np.array_equal(dk.out_coords.cpu().numpy(), hk.out_coords.reshape(-1, 3))
    dt = gpu_maps.transpose_map(dk, _dev(coords))
    _same(dt, maps.transpose_map(hk, coords))
    assert backend.device_status() == 0


def test_transpose_of_a_submanifold_map():
    from fgms_b200 import gpu_maps
    coords = clouds.uniform_cloud(4000, 24, 11)
    dk = gpu_maps.build_submanifold_map(_dev(coords), 3)
    _same(gpu_maps.transpose_map(dk), maps.transpose_map(maps.build_submanifold_map(coords, 3)))


def test_bad_coordinates_are_counted_not_used():
    from fgms_b200 import backend, gpu_maps
    coords = clouds.uniform_cloud(1000, 20, 2)
    bad = np.concatenate([coords, coords[:3], np.array([[1 << 22, 0, 0]], dtype=np.int32)])  # 3 duplicates, 1 out of range
    backend.device_status(reset=True)
    dk = gpu_maps.build_submanifold_map(_dev(bad), 3)
    assert backend.device_status() == 4
    hk = maps.build_submanifold_map(coords, 3)
    # the first 1000 voxels keep their rows; the skipped voxels take part in no pair except their own centre lookups
    keep = (dk.imap.cpu().numpy() < 1000) & (dk.omap.cpu().numpy() < 1000)
    assert int(keep.sum()) == hk.pairs


def test_maps_feed_the_operator():
    """A map built on the device drives the convolution to the same result as the host-built map."""
    from fgms_b200 import backend, gpu_maps
    from tests.util import Problem, err, TOL
    coords = clouds.uniform_cloud(3000, 20, 13)
    hk = maps.build_submanifold_map(coords, 3)
    p = Problem(hk, 64, 64, seed=5, mode="fp16")
    dk = gpu_maps.build_submanifold_map(_dev(coords), 3)
    out = torch.zeros((hk.n_out, 64), dtype=p.dtype, device="cuda")
    backend.fgms_fusion_fwd_cuda(p.feats, p.weights, p.qsum, out, dk.kpos, None, dk.imap, dk.omap, False, True)
    assert err(out, p.ref_fwd()) <= TOL["fp16"]
