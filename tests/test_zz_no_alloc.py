"""The allocation-free weight-gradient entry point (``fgms_b200_wgrad_f16_noalloc``).

Some callers of this library cannot allocate device memory at call time — a serving thread that
must never hit ``cudaMalloc``, a process whose pool is already handed out in full, a binding that
owns no allocator — so the library offers one weight-gradient entry point whose fp32 scratch is a
fixed array inside the library itself.  This file checks, through the C ABI, that it returns what
the ordinary entry point returns, twice in a row (the shared scratch keeps the previous call's
contents and has to be cleared by the call itself), and that it refuses shapes beyond its limit.
It is named to be collected last."""
import pytest
import torch

from fgms_b200 import clouds, maps
from tests.util import TOL, Problem, err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("c_in,c_out", [(128, 128), (64, 64), (48, 24)])
def test_noalloc_wgrad_matches_the_workspace_entry_point_twice(c_in, c_out):
    from fgms_b200 import backend
    km = maps.build_submanifold_map(clouds.surface_cloud(4000, 48, 77))
    p = Problem(km, c_in, c_out, seed=5, mode="fp16")
    ref = torch.zeros_like(p.weights)
    backend.fgms_wgrad_cuda(p.feats, p.grad_out, ref, p.kpos, p.imap, p.omap, True)
    oracle = p.ref_wgrad()
    assert err(ref, oracle) <= TOL["fp16"]
    for call in range(2):
        got = torch.zeros_like(p.weights)
        backend.fgms_wgrad_noalloc_cuda(p.feats, p.grad_out, got, p.kpos, p.imap, p.omap, True)
        torch.cuda.synchronize()
        scale = float(ref.float().abs().max())
        diff = float((got.float() - ref.float()).abs().max())
        assert diff <= TOL["fp16"] * scale, f"call {call}: differs from the workspace entry point by {diff}"
        assert err(got, oracle) <= TOL["fp16"]
    # a different gradient next: nothing of the previous call may leak through the shared scratch
    p.grad_out = -2 * p.grad_out
    got = torch.zeros_like(p.weights)
    backend.fgms_wgrad_noalloc_cuda(p.feats, p.grad_out, got, p.kpos, p.imap, p.omap, True)
    assert err(got, -2 * oracle) <= TOL["fp16"]


def test_noalloc_wgrad_refuses_shapes_beyond_its_scratch():
    from fgms_b200 import backend
    km = maps.build_submanifold_map(clouds.uniform_cloud(200, 8, 3))
    p = Problem(km, 256, 128, seed=1, mode="fp16")  # 27 * 256 * 128 > 512 Ki values
    assert km.k_vol * 256 * 128 > backend.NOALLOC_MAX_ELEMS
    with pytest.raises(ValueError, match="built-in scratch"):
        backend.fgms_wgrad_noalloc_cuda(p.feats, p.grad_out, torch.zeros_like(p.weights), p.kpos, p.imap, p.omap, True)
