"""Output-stationary forward (``fgms_b200_fwd_output_stationary``) against the oracle of the reference's forward
(``cpu-check.py:16-44``), through the binding and the C ABI: parity on submanifold, strided and transposed maps,
run-to-run identical bits, the fused bias + ReLU epilogue, the accumulate form, refusals."""
import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps
from tests.util import TOL, Problem, err

pytestmark = pytest.mark.gpu


def _table_ref(km):
    """The neighbour table restated on the host."""
    stride = (km.n_out + 127) // 128 * 128
    nbr = np.full((km.k_vol, stride), -1, np.int32)
    for k in range(km.k_vol):
        a, b = km.kpos[k], km.kpos[k + 1]
        nbr[k, km.omap[a:b]] = km.imap[a:b]
    return nbr


def _run(p, **kw):
    from fgms_b200 import backend
    nbr = backend.build_neighbor_table(p.kpos, p.imap, p.omap, p.km.n_in, p.km.n_out)
    out = kw.pop("out", None)
    if out is None:
        out = torch.full((p.km.n_out, p.c_out), 7.0, dtype=p.dtype, device="cuda")  # overwritten, not added to
    backend.fgms_fwd_os_cuda(p.feats, p.weights, out, nbr, p.arch80, **kw)
    return out, nbr


@pytest.mark.parametrize("mode", ["fp16", "tf32"])
@pytest.mark.parametrize("c_in,c_out", [(16, 16), (32, 32), (64, 64), (48, 80), (128, 128), (16, 256), (256, 128), (160, 96)])
def test_parity_submanifold(mode, c_in, c_out):
    from fgms_b200 import backend
    km = maps.build_submanifold_map(clouds.uniform_cloud(1500, 14, c_in * 7 + c_out))
    p = Problem(km, c_in, c_out, seed=c_in + 3 * c_out, mode=mode)
    backend.device_status(reset=True)
    out, nbr = _run(p)
    assert backend.device_status() == 0
    assert np.array_equal(nbr.cpu().numpy(), _table_ref(km))
    assert err(out, p.ref_fwd()) <= TOL[mode]


def test_parity_fp16_256_channels():
    km = maps.build_submanifold_map(clouds.uniform_cloud(900, 12, 5))
    p = Problem(km, 256, 256, seed=9, mode="fp16")
    out, _ = _run(p)
    assert err(out, p.ref_fwd()) <= TOL["fp16"]


@pytest.mark.parametrize("mode", ["fp16", "tf32"])
def test_strided_and_transposed(mode):
    coords = clouds.surface_cloud(4000, 64, 21)
    down = maps.build_strided_map(coords)
    p = Problem(down, 32, 64, seed=3, mode=mode)
    out, _ = _run(p)
    assert err(out, p.ref_fwd()) <= TOL[mode]
    up = maps.transpose_map(down, coords)
    p = Problem(up, 64, 32, seed=4, mode=mode)
    out, _ = _run(p)
    assert err(out, p.ref_fwd()) <= TOL[mode]


def test_same_bits_every_run_and_close_to_the_scatter_form():
    km = maps.build_submanifold_map(clouds.surface_cloud(6000, 64, 2))
    p = Problem(km, 64, 64, seed=1, mode="fp16")
    a, _ = _run(p)
    b, _ = _run(p)
    assert torch.equal(a, b)
    scatter = p.run_fwd()
    assert err(scatter, a.float().cpu().numpy().astype(np.float64)) <= 2 * TOL["fp16"]


@pytest.mark.parametrize("mode", ["fp16", "tf32"])
def test_bias_relu_epilogue(mode):
    km = maps.build_submanifold_map(clouds.uniform_cloud(1200, 13, 8))
    p = Problem(km, 32, 48, seed=2, mode=mode)
    bias = (torch.randn(48, device="cuda") * 0.5).to(p.dtype)
    out, _ = _run(p, bias=bias, relu=True)
    ref = np.maximum(p.ref_fwd() + bias.float().cpu().numpy().astype(np.float64)[None, :], 0.0)
    assert err(out, ref) <= TOL[mode]
    assert float(out.min()) >= 0.0
    out_b, _ = _run(p, bias=bias)
    assert err(out_b, p.ref_fwd() + bias.float().cpu().numpy().astype(np.float64)[None, :]) <= TOL[mode]


def test_accumulate_adds_like_the_reference_forward():
    km = maps.build_submanifold_map(clouds.uniform_cloud(700, 11, 4))
    p = Problem(km, 64, 32, seed=6, mode="fp16")
    out = torch.ones((km.n_out, 32), dtype=torch.float16, device="cuda")
    out, _ = _run(p, out=out, accumulate=True)
    assert err(out, p.ref_fwd() + 1.0) <= TOL["fp16"]


def test_refusals_and_empty():
    from fgms_b200 import backend
    km = maps.build_submanifold_map(clouds.uniform_cloud(300, 9, 1))
    p = Problem(km, 32, 32, seed=1, mode="fp16")
    nbr = backend.build_neighbor_table(p.kpos, p.imap, p.omap, km.n_in, km.n_out)
    out = torch.zeros((km.n_out, 32), dtype=torch.float16, device="cuda")
    bias = torch.zeros(32, dtype=torch.float16, device="cuda")
    with pytest.raises((ValueError, RuntimeError)):
        backend.fgms_fwd_os_cuda(p.feats, p.weights, out, nbr, p.arch80, bias=bias, accumulate=True)
    with pytest.raises((ValueError, RuntimeError)):
        backend.fgms_fwd_os_cuda(p.feats, p.weights, out, nbr[:, :-1].contiguous(), p.arch80)
    q = Problem(km, 32, 32, seed=1, mode="fp32")  # exact fp32 arithmetic has no tensor-core form
    out32 = torch.zeros((km.n_out, 32), device="cuda")
    with pytest.raises((ValueError, RuntimeError)):
        backend.fgms_fwd_os_cuda(q.feats, q.weights, out32, nbr, q.arch80)
    r = Problem(km, 24, 32, seed=1, mode="fp16")  # 24 channels: no multiple of 16
    with pytest.raises((ValueError, RuntimeError)):
        backend.fgms_fwd_os_cuda(r.feats, r.weights, out, nbr, r.arch80)
    empty = maps.build_submanifold_map(np.zeros((0, 3), np.int32))
    e = Problem(empty, 32, 32, seed=1, mode="fp16")
    nbr0 = backend.build_neighbor_table(e.kpos, e.imap, e.omap, 0, 0)
    out0 = torch.zeros((0, 32), dtype=torch.float16, device="cuda")
    backend.fgms_fwd_os_cuda(e.feats, e.weights, out0, nbr0, e.arch80)
    assert nbr0.numel() == 0
