"""cfg5 — the MinkUNet-style encoder-decoder stack (``fgms_b200.unet``): every layer's output, input gradient and
weight gradient against the fp64 oracle, the device-built maps against the host builders, and the bound step
against the autograd module.

Per-layer comparisons feed the oracle the *stored* (fp16) tensors the CUDA path read, so a layer's bound does not
depend on its depth; the end-to-end comparison runs the whole stack in fp64 from the inputs."""
import numpy as np
import pytest
import torch

from fgms_b200 import unet, workloads
from oracle import spconv_oracle as orc
from oracle import unet_oracle
from tests.util import TOL, err

pytestmark = pytest.mark.gpu


def _setup(voxels, grid, scenes=1):
    wl = workloads.unet_workload(scenes=scenes, voxels=voxels, grid=grid)
    spec = unet.minkunet_spec(wl.c_in, wl.widths)
    host = unet.build_unet_maps_host(wl.coords)
    dev = unet.build_unet_maps(torch.from_numpy(wl.coords).cuda())
    weights = unet.unet_weights(spec, host, wl.seed)
    return wl, spec, host, dev, weights


def _same_maps(host, dev):
    for hs, ds in ((host.subm, dev.subm), (host.down, dev.down), (host.up, dev.up)):
        for h, d in zip(hs, ds):
            assert (h.n_in, h.n_out, h.pairs) == (d.n_in, d.n_out, d.pairs)
            assert np.array_equal(d.kpos.cpu().numpy(), h.kpos)
            assert np.array_equal(d.imap.cpu().numpy(), h.imap) and np.array_equal(d.omap.cpu().numpy(), h.omap)


def _f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("scenes", [1, 2])
def test_cfg5_parity(scenes):
    """Reduced scenes (~20 k voxels each), the whole stack."""
    from fgms_b200 import backend
    wl, spec, host, dev, weights = _setup(20_000, 128, scenes)
    _same_maps(host, dev)
    step = unet.UNetStep(spec, dev, weights, torch.from_numpy(wl.feats).cuda(), torch.from_numpy(wl.grad_out).cuda())
    fallbacks = backend.fallback_count()
    backend.device_status(reset=True)
    step.run()
    assert backend.device_status() == 0 and backend.fallback_count() == fallbacks
    tol = TOL["fp16"]
    # ---- per layer, on the tensors the CUDA path stored
    expect_grad = {}
    for i, l in enumerate(spec):
        km = host.of(l)
        x, w, g = _f64(step.val[l.src])[:, : l.c_in], _f64(step.weights[i]), _f64(step.grad[l.dst])
        ref = orc.fwd(x, w, km.n_out, km.kpos, km.imap, km.omap)
        if l.skip is not None:
            ref = ref + _f64(step.val[l.skip])
            expect_grad[l.skip] = expect_grad.get(l.skip, 0) + g
        assert err(step.val[l.dst], ref) <= tol, f"{l.name}: forward"
        assert err(step.w_grads[i], orc.wgrad(x, g, l.k_vol, km.kpos, km.imap, km.omap)) <= tol, f"{l.name}: wgrad"
        if i > 0:
            expect_grad[l.src] = expect_grad.get(l.src, 0) + orc.dgrad(g, w, km.n_in, km.kpos, km.imap, km.omap)
    for name, ref in expect_grad.items():
        assert err(step.grad[name], ref) <= tol, f"gradient of {name}"
    # ---- end to end: the whole stack in fp64 from the inputs (error accumulates over 25 fp16 layers)
    val = unet_oracle.forward(spec, host, weights, wl.feats)
    grad, w_grads = unet_oracle.backward(spec, host, weights, val, wl.grad_out)
    assert err(step.val[spec[-1].dst], val[spec[-1].dst]) <= 3 * tol
    assert err(step.grad["e0"], grad["e0"]) <= 3 * tol
    assert err(step.w_grads[0], w_grads[0]) <= 3 * tol and err(step.w_grads[12], w_grads[12]) <= 3 * tol


def test_cfg5_full_size_layers():
    """One full-size scene (~120 k voxels): the device-built maps and the two heaviest fine-resolution layer shapes
    (stem 4 -> 32 and a 32 -> 32 submanifold layer) against the oracle."""
    wl, spec, host, dev, weights = _setup(120_000, 256, 1)
    _same_maps(host, dev)
    step = unet.UNetStep(spec, dev, weights, torch.from_numpy(wl.feats).cuda(), torch.from_numpy(wl.grad_out).cuda())
    step.run()
    for i in (0, len(spec) - 1):
        l, km = spec[i], host.of(spec[i])
        x, w, g = _f64(step.val[l.src])[:, : l.c_in], _f64(step.weights[i]), _f64(step.grad[l.dst])
        assert err(step.val[l.dst], orc.fwd(x, w, km.n_out, km.kpos, km.imap, km.omap)) <= TOL["fp16"]
        assert err(step.w_grads[i], orc.wgrad(x, g, l.k_vol, km.kpos, km.imap, km.omap)) <= TOL["fp16"]
        if i > 0:
            assert err(step.grad[l.src], orc.dgrad(g, w, km.n_in, km.kpos, km.imap, km.omap)) <= TOL["fp16"]


def test_data_parallel_form_on_one_rank():
    """The form several ranks run (fp32 sums of all layers in one flat buffer cut into buckets, added to the fp16
    gradients at the end) gives the single-rank gradients; with one rank the collective is skipped."""
    wl, spec, host, dev, weights = _setup(8_000, 96, 1)
    feats, grad_out = torch.from_numpy(wl.feats).cuda(), torch.from_numpy(wl.grad_out).cuda()
    one = unet.UNetStep(spec, dev, weights, feats, grad_out)
    dp = unet.UNetStep(spec, dev, weights, feats, grad_out, exchange=True, bucket_bytes=1 << 20)
    assert len(dp.buckets) >= 3 and dp.buckets[0][0] == 0 and dp.buckets[-1][1] == dp.w_grad.numel()
    assert all(a[1] == b[0] for a, b in zip(dp.buckets, dp.buckets[1:]))
    one.run(); dp.run()
    for i, l in enumerate(spec):
        ref = one.w_grads[i].float()
        assert float((dp.w_grads[i].float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max()), l.name
    assert torch.equal(one.val[spec[-1].dst], dp.val[spec[-1].dst]) or \
        float((one.val[spec[-1].dst].float() - dp.val[spec[-1].dst].float()).abs().max()) <= 1e-2 * float(one.val[spec[-1].dst].float().abs().max())


def test_bound_step_equals_the_autograd_module():
    from fgms_b200 import nn
    wl, spec, host, dev, weights = _setup(8_000, 96, 1)
    feats, grad_out = torch.from_numpy(wl.feats).cuda(), torch.from_numpy(wl.grad_out).cuda()
    step = unet.UNetStep(spec, dev, weights, feats, grad_out)
    step.run()
    net = nn.SparseUNet(spec)
    net.load_weights(weights)
    out = net(feats, dev)
    out.backward(grad_out)
    scale = float(step.val[spec[-1].dst].float().abs().max())
    assert float((out.detach().float() - step.val[spec[-1].dst].float()).abs().max()) <= 1e-2 * scale
    for i, layer in enumerate(net.layers):
        ref = step.w_grads[i].float()
        assert float((layer.weight.grad.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max()), spec[i].name
