"""The bound (validated-once) layer step gives the results of the checked entry points."""
import pytest
import torch

from fgms_b200 import clouds, maps
from tests.util import TOL, Problem, err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,c_in,c_out", [("fp16", 128, 128), ("fp16", 32, 32), ("tf32", 32, 64), ("fp32", 16, 16)])
def test_bound_layer_matches_oracle(mode, c_in, c_out):
    from fgms_b200.dist import BoundSceneLayer
    km = maps.build_submanifold_map(clouds.uniform_cloud(2500, 18, 3))
    p = Problem(km, c_in, c_out, seed=6, mode=mode)
    out = torch.zeros((km.n_out, c_out), dtype=p.dtype, device="cuda")
    in_grad = torch.zeros((km.n_in, c_in), dtype=p.dtype, device="cuda")
    w_grad = torch.zeros_like(p.weights)
    layer = BoundSceneLayer(p.feats, p.weights, p.grad_out, out, in_grad, w_grad, p.kpos, p.imap, p.omap, p.arch80)
    layer.forward()
    layer.backward()
    assert err(out, p.ref_fwd()) <= TOL[mode]
    assert err(in_grad, p.ref_dgrad()) <= TOL[mode]
    assert err(w_grad, p.ref_wgrad()) <= TOL[mode]
    with pytest.raises(ValueError):
        BoundSceneLayer(p.feats, p.weights, p.grad_out, out[:-1], in_grad, w_grad, p.kpos, p.imap, p.omap, p.arch80)
