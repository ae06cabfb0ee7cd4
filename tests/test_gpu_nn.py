"""The autograd wrapper: gradients through ``sparse_conv`` equal the oracle's dgrad / wgrad."""
import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps
from tests.util import TOL, Problem, err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,c_in,c_out", [("fp16", 64, 128), ("tf32", 32, 64), ("fp32", 16, 16)])
def test_autograd_matches_oracle(mode, c_in, c_out):
    from fgms_b200 import gpu_maps, nn
    coords = clouds.uniform_cloud(2500, 18, 21)
    hk = maps.build_submanifold_map(coords, 3)
    p = Problem(hk, c_in, c_out, seed=4, mode=mode)
    dk = gpu_maps.build_submanifold_map(torch.from_numpy(coords).cuda(), 3)
    feats = p.feats.clone().requires_grad_(True)
    weight = p.weights.clone().requires_grad_(True)
    out = nn.sparse_conv(feats, weight, dk, arch80=p.arch80)
    assert err(out, p.ref_fwd()) <= TOL[mode]
    out.backward(p.grad_out)
    assert err(feats.grad, p.ref_dgrad()) <= TOL[mode]
    assert err(weight.grad, p.ref_wgrad()) <= TOL[mode]


def test_two_layers_share_a_map_and_train():
    """conv -> ReLU -> conv on one cached map: one SGD step lowers a quadratic loss."""
    from fgms_b200 import gpu_maps, nn
    torch.manual_seed(0)
    coords = clouds.uniform_cloud(4000, 22, 8)
    dk = gpu_maps.build_submanifold_map(torch.from_numpy(coords).cuda(), 3)
    l1 = nn.SparseConv3d(32, 64, dtype=torch.float32)
    l2 = nn.SparseConv3d(64, 32, dtype=torch.float32)
    x = torch.randn((dk.n_in, 32), device="cuda")
    target = torch.randn((dk.n_out, 32), device="cuda")
    params = list(l1.parameters()) + list(l2.parameters())
    losses = []
    for _ in range(3):
        y = l2(torch.relu(l1(x, dk)), dk)
        loss = ((y - target) ** 2).mean()
        losses.append(float(loss.detach()))
        for q in params:
            q.grad = None
        loss.backward()
        with torch.no_grad():
            for q in params:
                q -= 0.5 * q.grad
    assert losses[2] < losses[1] < losses[0]


def test_inference_form_matches_the_autograd_form_with_bias_and_relu():
    """conv + bias + ReLU in one kernel (output-stationary forward) against the same three steps with the scatter
    form; the table is built once and kept on the map; two calls give identical bits."""
    from fgms_b200 import gpu_maps, nn
    torch.manual_seed(1)
    coords = clouds.uniform_cloud(3000, 20, 5)
    dk = gpu_maps.build_submanifold_map(torch.from_numpy(coords).cuda(), 3)
    layer = nn.SparseConv3d(64, 32, dtype=torch.float16)
    x = torch.randn((dk.n_in, 64), device="cuda").half()
    bias = (torch.randn(32, device="cuda") * 0.3).half()
    ref = torch.relu(layer(x, dk).detach().float() + bias.float())
    got = nn.sparse_conv_inference(x, layer.weight, dk, bias=bias, relu=True)
    assert hasattr(dk, "_neighbor_table")
    assert float((got.float() - ref).abs().max()) <= 1e-2 * max(float(ref.abs().max()), 1e-6)
    assert torch.equal(got, nn.sparse_conv_inference(x, layer.weight, dk, bias=bias, relu=True))
