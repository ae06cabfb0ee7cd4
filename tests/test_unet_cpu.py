"""The stack's layer list, map plumbing and CPU oracle (no GPU): shapes chain, skips mirror, and the oracle's
backward is the gradient of its forward."""
import numpy as np

from fgms_b200 import clouds, unet
from oracle import unet_oracle


def test_spec_chains_and_mirrors():
    spec = unet.minkunet_spec()
    assert len(spec) == 25 and spec[0].c_in == 4 and spec[0].c_out == 32
    width = {"input": 4}
    level = {"input": 0}
    for l in spec:
        assert width[l.src] == l.c_in and level[l.src] == l.res_in
        if l.skip is not None:
            assert l.kind == "up" and width[l.skip] == l.c_out and level[l.skip] == l.res_out
        width[l.dst], level[l.dst] = l.c_out, l.res_out
    assert [l.c_out for l in spec if l.kind == "down"] == [32, 64, 128, 256]
    assert [l.c_out for l in spec if l.kind == "up"] == [128, 64, 32, 32]
    assert spec[-1].res_out == 0 and spec[-1].c_out == 32


def test_maps_of_all_levels_are_consistent():
    coords = clouds.surface_cloud(3000, 64, 3)
    um = unet.build_unet_maps_host(coords, levels=3)
    assert len(um.subm) == 4 and len(um.down) == 3 and len(um.up) == 3
    for r in range(3):
        assert um.down[r].n_in == um.subm[r].n_in and um.down[r].n_out == um.subm[r + 1].n_in
        assert um.up[r].n_in == um.down[r].n_out and um.up[r].n_out == um.down[r].n_in
        assert um.down[r].pairs == um.down[r].n_in  # every voxel has exactly one parent


def test_oracle_backward_is_the_gradient_of_its_forward():
    coords = clouds.surface_cloud(600, 32, 4)
    spec = unet.minkunet_spec(4, (16, 16, 32))
    um = unet.build_unet_maps_host(coords, levels=2)
    w = unet.unet_weights(spec, um, 1, dtype=np.float64)
    rng = np.random.default_rng(0)
    f = rng.standard_normal((um.voxels[0], 4))
    g = rng.standard_normal((um.voxels[0], 16))
    val = unet_oracle.forward(spec, um, w, f)
    grad, wg = unet_oracle.backward(spec, um, w, val, g)
    loss = lambda ws: float((unet_oracle.forward(spec, um, ws, f)[spec[-1].dst] * g).sum())
    base = loss(w)
    for li, idx in ((0, (13, 2, 5)), (4, (3, 7, 1)), (len(spec) - 1, (20, 0, 9)), (7, (5, 10, 3))):
        w2 = [x.copy() for x in w]
        eps = 1e-6
        w2[li][idx] += eps
        num = (loss(w2) - base) / eps
        assert abs(num - wg[li][idx]) <= 1e-4 * max(1.0, abs(num)), (li, num, wg[li][idx])
