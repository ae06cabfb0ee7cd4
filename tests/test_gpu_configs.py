"""The benchmark configurations at full size: parity with the vectorised fp64 oracle plus
size-independent properties (linearity in the features, pair-order invariance)."""
import numpy as np
import pytest
import torch

from fgms_b200 import workloads
from tests.util import TOL, Problem, err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg3a", "cfg3b", "cfg4", "cfg5l0"])
def test_config_parity(name):
    wl = workloads.get(name)
    p = Problem(wl.kmap, wl.c_in, wl.c_out, seed=wl.seed, mode=wl.mode)
    from fgms_b200 import backend
    backend.device_status(reset=True)
    out = p.run_fwd()
    in_grad, w_grad = p.run_bwd()
    assert backend.device_status() == 0
    tol = TOL[wl.mode]
    assert err(out, p.ref_fwd()) <= tol
    assert err(in_grad, p.ref_dgrad()) <= tol
    assert err(w_grad, p.ref_wgrad()) <= tol


def test_cfg1_literal_reference_definition():
    """cfg1 is the case the reference's own CPU loops can check: the C restatement of those loops
    (bit-exact with the reference on the golden fixtures) is the comparison here."""
    from oracle import c_oracle
    wl = workloads.get("cfg1")
    p = Problem(wl.kmap, wl.c_in, wl.c_out, seed=wl.seed, mode="fp32")
    out = p.run_fwd()
    in_grad, w_grad = p.run_bwd()
    km = wl.kmap
    ref = c_oracle.fwd(p.f_np, p.w_np, km.n_out, km.knnz, km.imap, km.omap, acc="f32")
    ig, wg = c_oracle.bwd(p.g_np, p.w_np, p.f_np, km.n_in, km.knnz, km.imap, km.omap, acc="f32")
    # the reference's tolerance: allclose(rtol=1e-2, atol=1e-4), cpu-check.py:127
    assert np.allclose(out.cpu().numpy(), ref, rtol=1e-2, atol=1e-4)
    assert np.allclose(in_grad.cpu().numpy(), ig, rtol=1e-2, atol=1e-4)
    assert np.allclose(w_grad.cpu().numpy(), wg, rtol=1e-2, atol=1e-4)
    assert err(out, ref) <= 1e-5 and err(in_grad, ig) <= 1e-5 and err(w_grad, wg) <= 1e-5


@pytest.mark.parametrize("name", ["cfg2", "cfg4"])
def test_linearity_and_pair_order_invariance(name):
    wl = workloads.get(name)
    p = Problem(wl.kmap, wl.c_in, wl.c_out, seed=wl.seed, mode=wl.mode)
    base = p.run_fwd().float()
    # f -> 2 f doubles the output exactly (scaling by two is exact in fp16/fp32)
    p2 = Problem(wl.kmap, wl.c_in, wl.c_out, seed=wl.seed, mode=wl.mode)
    p2.feats = p.feats * 2
    twice = p2.run_fwd().float()
    assert float((twice - 2 * base).abs().max()) <= 2e-2 * float(base.abs().max())
    # shuffling the pairs inside every offset must not change the result beyond rounding
    rng = np.random.default_rng(0)
    perm = np.concatenate([a + rng.permutation(b - a) for a, b in zip(wl.kmap.kpos[:-1], wl.kmap.kpos[1:])])
    p3 = Problem(wl.kmap, wl.c_in, wl.c_out, seed=wl.seed, mode=wl.mode)
    p3.imap = torch.from_numpy(wl.kmap.imap[perm]).cuda()
    p3.omap = torch.from_numpy(wl.kmap.omap[perm]).cuda()
    shuffled = p3.run_fwd().float()
    assert float((shuffled - base).abs().max()) <= 1e-2 * float(base.abs().max())
