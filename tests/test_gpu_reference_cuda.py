"""This library beside the reference's own CUDA kernels, on identical seeded inputs.

The reference's extension (``backend/pybind_cuda.cpp`` + ``backend/spconv.cu``) is compiled from a checkout of the
reference by ``oracle/build_ref.py`` into a build product that is not under version control; without it these tests
are skipped.  Only shapes on which the reference's kernels are sound are launched: fp16, channel counts that are
multiples of 32 and not 64 on the output side — fused forward ``_fgms_fusion_fp16_v2``
(``backend/fwd_kernels.cuh:17-144``), dgrad ``_fgms_fusion_fp16_W_transpose_v2`` (``backend/bwd_kernels.cuh:281-408``),
wgrad ``_fgms_fusion_fp16_I_transpose_v4`` (``:876-980``).  The kernel it takes for 64 output channels, the tf32 dgrad
for more than 32 input channels and the weight gradients for channel counts that are no multiple of 32 access memory
out of range or misaligned and are never run here.

The reference accumulates in fp16 (``wmma`` accumulators of type ``half``, fp16 atomics), so its own error against
the fp64 oracle is the larger one; both are asserted against the oracle and against each other."""
import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps, workloads
from oracle import build_ref
from tests.util import TOL, Problem, err

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not build_ref.available(), reason="reference extension not built")]


def _reference_run(p: Problem):
    try:
        ref = build_ref.load()
    except Exception as exc:  # built for another interpreter or torch: nothing to compare with here
        pytest.skip(f"the reference extension does not load: {exc!r}")
    torch.cuda.synchronize()
    out = torch.zeros((p.km.n_out, p.c_out), dtype=p.dtype, device="cuda")
    in_grad = torch.zeros((p.km.n_in, p.c_in), dtype=p.dtype, device="cuda")
    w_grad = torch.zeros_like(p.weights)
    # the reference launches on the legacy default stream, which is PyTorch's default stream
    ref.fgms_fusion_fwd_cuda(p.feats, p.weights, p.qsum, out, p.kpos, p.qkpos, p.imap, p.omap, False, True)
    ref.fgms_bwd_cuda(p.grad_out, p.feats, p.weights, p.qsum, in_grad, w_grad, p.kpos, p.qkpos, p.imap, p.omap, False, True)
    torch.cuda.synchronize()
    return out, in_grad, w_grad


@pytest.mark.parametrize("case", ["small 128->128", "small 96->32", "cfg4"])
def test_matches_the_reference_cuda_path(case):
    if case == "cfg4":
        wl = workloads.get("cfg4")
        p = Problem(wl.kmap, wl.c_in, wl.c_out, seed=wl.seed, mode="fp16")
    else:
        c_in, c_out = (128, 128) if "128" in case else (96, 32)
        p = Problem(maps.build_submanifold_map(clouds.surface_cloud(5000, 48, 9)), c_in, c_out, seed=3, mode="fp16")
    assert p.c_in % 32 == 0 and p.c_out % 32 == 0 and p.c_out != 64 and p.c_in > 16 and p.c_out > 16
    r_out, r_in, r_w = _reference_run(p)
    out = p.run_fwd()
    in_grad, w_grad = p.run_bwd()
    o_out, o_in, o_w = p.ref_fwd(), p.ref_dgrad(), p.ref_wgrad()
    ours = (err(out, o_out), err(in_grad, o_in), err(w_grad, o_w))
    theirs = (err(r_out, o_out), err(r_in, o_in), err(r_w, o_w))
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    between = (err(out, f64(r_out)), err(in_grad, f64(r_in)), err(w_grad, f64(r_w)))
    print(f"{case}: error vs fp64 oracle ours {ours}, reference CUDA {theirs}; ours vs reference CUDA {between}")
    assert max(ours) <= TOL["fp16"]
    assert max(theirs) <= 3 * TOL["fp16"]   # fp16 accumulation: the reference's own error
    assert max(between) <= 3 * TOL["fp16"]
    # fp32 accumulation is at least as close to the exact result, up to what the order of the fp16 atomics (both
    # libraries scatter with them) moves either error from run to run
    assert max(ours) <= max(theirs) + 1e-3
