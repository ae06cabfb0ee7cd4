"""Parity of the CUDA path (through the public binding, hence through the C ABI) with the oracle.

Bounds (max-abs error / max |reference|): 1e-5 for fp32, 5e-3 for tf32, 1e-2 for fp16; the
reference's own script uses allclose(rtol=1e-2, atol=1e-4) (cpu-check.py:127)."""
import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps
from tests.util import TOL, Problem, err

pytestmark = pytest.mark.gpu

MODES = ["fp32", "tf32", "fp16"]


def _sub_map(n, grid, seed):
    return maps.build_submanifold_map(clouds.uniform_cloud(n, grid, seed))


def expected_family(mode, c_in, c_out, pass_="fwd"):
    """The dispatch rule, restated: tensor cores for tf32 / fp16 arithmetic when both channel counts are
    multiples of 16 and at most 256 (and the operands fit shared memory, which only tf32 256 x 256 forward and
    dgrad do not)."""
    if mode == "fp32" or c_in % 16 or c_out % 16 or max(c_in, c_out) > 256:
        return "simt"
    if mode == "tf32" and c_in == 256 and c_out == 256 and pass_ != "wgrad":
        return "simt"
    return "tcgen05"


def _check_all(p: Problem, tol=None):
    from fgms_b200 import backend
    tol = TOL[p.mode] if tol is None else tol
    # a parity case must not pass on a slower kernel family than the shape is meant to run on
    for pass_ in ("fwd", "dgrad", "wgrad"):
        assert backend.kernel_family(pass_, p.c_in, p.c_out, p.dtype, p.arch80, p.km.k_vol) == \
            expected_family(p.mode, p.c_in, p.c_out, pass_), (pass_, p.mode, p.c_in, p.c_out)
    fallbacks = backend.fallback_count()
    backend.device_status(reset=True)
    out = p.run_fwd()
    in_grad, w_grad = p.run_bwd()
    assert backend.device_status() == 0
    assert backend.fallback_count() == fallbacks, "a launch fell back to the CUDA-core kernels"
    e = (err(out, p.ref_fwd()), err(in_grad, p.ref_dgrad()), err(w_grad, p.ref_wgrad()))
    assert max(e) <= tol, f"fwd/dgrad/wgrad errors {e} exceed {tol} ({p.mode}, {p.c_in}->{p.c_out})"
    return e


def test_golden_fixtures_fp32(golden):
    """The reference's own CPU outputs, reproduced by the fp32 FFMA path."""
    g = golden
    from fgms_b200 import backend
    dev = "cuda"
    t = lambda a: torch.from_numpy(a).to(dev)
    n_in, n_out = int(g["n_in"]), int(g["n_out"])
    k_vol, c_in, c_out = g["weights"].shape
    qkpos, qsum = maps.kpos_quantized(g["knnz"], g["kpos"], k_vol, 256)
    out = torch.zeros((n_out, c_out), device=dev)
    backend.fgms_fusion_fwd_cuda(t(g["feats"]), t(g["weights"]), qsum, out, t(g["kpos"]), t(qkpos), t(g["imap"]),
                                 t(g["omap"]), bool(g["precompute"]), False)
    assert err(out, g["out"]) <= 1e-5
    in_grad = torch.zeros((n_in, c_in), device=dev)
    w_grad = torch.zeros((k_vol, c_in, c_out), device=dev)
    backend.fgms_bwd_cuda(t(g["grad_out"]), t(g["feats"]), t(g["weights"]), qsum, in_grad, w_grad, t(g["kpos"]),
                          t(qkpos), t(g["imap"]), t(g["omap"]), False, False)
    assert err(in_grad, g["in_grad"]) <= 1e-5
    assert err(w_grad, g["w_grad"]) <= 1e-5


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("c_in,c_out", [(1, 1), (3, 5), (4, 32), (16, 16), (16, 32), (32, 16), (16, 128), (64, 128), (17, 33), (32, 32), (32, 64), (64, 32), (64, 64),
                                        (48, 80), (128, 128), (96, 128), (128, 64), (256, 128), (128, 256), (192, 64),
                                        (160, 96), (224, 32), (16, 256), (256, 256)])
def test_channel_classes_submanifold(mode, c_in, c_out):
    p = Problem(_sub_map(1500, 14, c_in * 131 + c_out), c_in, c_out, seed=c_in + 7 * c_out, mode=mode)
    _check_all(p)


@pytest.mark.parametrize("mode", MODES)
def test_strided_and_transposed(mode):
    coords = clouds.surface_cloud(4000, 64, 21)
    down = maps.build_strided_map(coords)
    _check_all(Problem(down, 32, 64, seed=3, mode=mode))
    up = maps.transpose_map(down, coords)
    _check_all(Problem(up, 64, 32, seed=4, mode=mode))


@pytest.mark.parametrize("mode", MODES)
def test_k_vol_one_and_empty_offsets(mode):
    # k_vol = 1: a plain gathered GEMM
    n = 700
    ident = np.arange(n, dtype=np.int32)
    perm = np.random.default_rng(0).permutation(n).astype(np.int32)
    km = maps.KernelMap(n, n, 1, np.array([n], np.int32), np.array([0, n], np.int32), perm, ident)
    _check_all(Problem(km, 64, 64, seed=5, mode=mode))
    # most offsets empty (isolated voxels: only the centre offset has pairs)
    coords = (clouds.uniform_cloud(300, 20, 9) * 3).astype(np.int32)
    km = maps.build_submanifold_map(coords)
    assert (km.knnz == 0).sum() == 26
    _check_all(Problem(km, 64, 128, seed=6, mode=mode))


@pytest.mark.parametrize("mode", ["fp16", "tf32"])
@pytest.mark.parametrize("c_in,c_out", [(16, 16), (16, 32), (32, 16), (32, 32)])
def test_short_rows_full_and_partial_stages(mode, c_in, c_out):
    # rows of at most 64 bytes: the weight-gradient kernel stages several pairs to one 128-byte row.  One offset
    # of 1000 pairs = three whole 256-pair stages and a partial one; then a map whose offsets hold 1 .. 5 pairs.
    n = 1000
    ident = np.arange(n, dtype=np.int32)
    perm = np.random.default_rng(1).permutation(n).astype(np.int32)
    km = maps.KernelMap(n, n, 1, np.array([n], np.int32), np.array([0, n], np.int32), perm, ident)
    _check_all(Problem(km, c_in, c_out, seed=11, mode=mode))
    knnz = np.array([1, 0, 5, 2, 0, 3, 1, 4], np.int32)
    kpos = np.concatenate([[0], np.cumsum(knnz)]).astype(np.int32)
    rng = np.random.default_rng(2)
    imap = np.concatenate([rng.permutation(40)[:c] for c in knnz]).astype(np.int32)
    omap = np.concatenate([rng.permutation(30)[:c] for c in knnz]).astype(np.int32)
    km = maps.KernelMap(40, 30, 8, knnz, kpos, imap, omap)
    _check_all(Problem(km, c_in, c_out, seed=12, mode=mode))


@pytest.mark.parametrize("mode", MODES)
def test_empty_cloud_and_no_pairs(mode):
    km = maps.build_submanifold_map(np.zeros((0, 3), np.int32))
    p = Problem(km, 64, 64, seed=1, mode=mode)
    out = p.run_fwd()
    in_grad, w_grad = p.run_bwd()
    assert out.shape == (0, 64) and in_grad.shape == (0, 64)
    assert float(w_grad.abs().max()) == 0.0


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("c", [16, 64])
def test_separate_mid_and_sequential_entry(mode, c):
    coords = clouds.surface_cloud(2500, 40, 17)
    full = maps.build_submanifold_map(coords)
    nomid = maps.drop_centre(full)
    p = Problem(nomid, c, c, seed=8, mode=mode)
    ref = p.ref_fwd(precompute=True)
    # fused entry: the centre term overwrites whatever out held (beta = 0 in the reference)
    dirty = torch.full((nomid.n_out, c), 3.0, dtype=p.dtype, device="cuda")
    assert err(p.run_fwd(separate_mid=True, fused=True, out=dirty), ref) <= TOL[mode]
    # sequential entry: accumulates (beta = 1)
    assert err(p.run_fwd(separate_mid=True, fused=False), ref) <= TOL[mode]
    # and both equal the plain fused call on the full map (what remove_mid builds)
    pf = Problem(full, c, c, seed=8, mode=mode)
    assert err(pf.run_fwd(), ref) <= TOL[mode]
    assert err(pf.run_fwd(fused=False), ref) <= TOL[mode]


@pytest.mark.parametrize("mode", MODES)
def test_accumulate_semantics(mode):
    """Outputs are accumulated into (the caller zeroes them): a second call doubles the result."""
    p = Problem(_sub_map(900, 12, 2), 64, 64, seed=2, mode=mode)
    out = p.run_fwd()
    once = out.clone()
    p.run_fwd(out=out)
    # fp16: every atomic of the second call rounds at twice the magnitude and in another order than the first
    assert err(out, 2.0 * once.float().cpu().numpy().astype(np.float64)) <= {"fp32": 1e-5, "tf32": 2e-3, "fp16": 1e-2}[mode]


def test_error_behaviour():
    from fgms_b200 import backend
    p = Problem(_sub_map(100, 6, 1), 16, 16, seed=1, mode="fp32")
    out = torch.zeros((p.km.n_out, 16), device="cuda")
    with pytest.raises(ValueError, match="Input feature size and kernel size mismatch"):
        backend.fgms_fusion_fwd_cuda(p.feats[:, :8].contiguous(), p.weights, p.qsum, out, p.kpos, p.qkpos, p.imap,
                                     p.omap, False, False)
    with pytest.raises(ValueError):
        backend.fgms_fusion_fwd_cuda(p.feats.cpu(), p.weights, p.qsum, out, p.kpos, p.qkpos, p.imap, p.omap, False, False)
    with pytest.raises(ValueError):
        backend.fgms_fusion_fwd_cuda(p.feats, p.weights, p.qsum, out, p.kpos, p.qkpos, p.imap.long(), p.omap, False, False)
    with pytest.raises(ValueError):
        backend.fgms_fusion_fwd_cuda(p.feats.double(), p.weights.double(), p.qsum, out.double(), p.kpos, p.qkpos,
                                     p.imap, p.omap, False, False)


@pytest.mark.parametrize("mode", MODES)
def test_out_of_range_map_entries_are_skipped_and_counted(mode):
    from fgms_b200 import backend
    p = Problem(_sub_map(600, 10, 4), 64, 64, seed=4, mode=mode)
    bad = p.km.imap.copy()
    bad_pos = [3, 77, p.km.pairs - 1]
    bad[bad_pos[0]] = -1
    bad[bad_pos[1]] = p.km.n_in
    bad[bad_pos[2]] = 2 ** 30
    p.imap = torch.from_numpy(bad).cuda()
    backend.device_status(reset=True)
    out = p.run_fwd()
    assert backend.device_status() == 3
    # reference result with those three pairs removed
    keep = np.ones(p.km.pairs, bool)
    keep[bad_pos] = False
    seg = np.repeat(np.arange(p.km.k_vol), p.km.knnz)
    knnz = np.bincount(seg[keep], minlength=p.km.k_vol).astype(np.int32)
    kpos = np.concatenate([[0], np.cumsum(knnz)]).astype(np.int32)
    from oracle import spconv_oracle as orc
    ref = orc.fwd(p.f_np, p.w_np, p.km.n_out, kpos, p.km.imap[keep], p.km.omap[keep])
    assert err(out, ref) <= TOL[mode]


@pytest.mark.parametrize("c_in,c_out", [(64, 64), (128, 128), (64, 128), (256, 128)])
def test_fp16_wgrad_both_forms(c_in, c_out):
    """fp16 weight gradient: the single-launch form (fp16 atomics across CTAs) and the fp32-workspace form
    agree with the oracle, accumulate into kernel_grad, and the workspace form leaves the fp32 sums behind."""
    from fgms_b200 import backend
    p = Problem(_sub_map(3000, 20, 31), c_in, c_out, seed=9, mode="fp16")
    assert backend.kernel_family("wgrad", c_in, c_out, torch.float16, True, p.km.k_vol) == "tcgen05"
    ref = p.ref_wgrad()
    prior = (torch.randn_like(p.weights) * 0.5)
    for fp32_sums in (False, True):
        w_grad = prior.clone()
        ws = backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, p.kpos, p.imap, p.omap, True, fp32_sums=fp32_sums)
        assert (ws is None) == (not fp32_sums)
        e = err(w_grad.float() - prior.float(), ref)
        assert e <= TOL["fp16"], f"fp32_sums={fp32_sums}: error {e}"
        if fp32_sums:
            sums = ws[: w_grad.numel()].view_as(w_grad)
            assert err(sums, ref) <= 1e-3
    # the reference-shaped entry point follows the module switch
    for flag in (False, True):
        backend.WGRAD_FP32_SUMS = flag
        try:
            _, w_grad = p.run_bwd()
        finally:
            backend.WGRAD_FP32_SUMS = False
        assert err(w_grad, ref) <= TOL["fp16"]


@pytest.mark.parametrize("mode", MODES)
def test_kpos_beyond_the_maps_is_clamped_and_counted(mode):
    """A stale kpos that points past the end of the maps must not move a read past them: the kernels clamp
    every entry to the maps' length, count the problem, and compute the pairs that do exist."""
    from fgms_b200 import backend
    from oracle import spconv_oracle as orc
    p = Problem(_sub_map(800, 11, 12), 64, 64, seed=3, mode=mode)
    k_vol, pairs = p.km.k_vol, p.km.pairs
    cut = int(p.km.kpos[k_vol - 2])             # the maps passed hold only the first `cut` pairs
    p.imap, p.omap = p.imap[:cut].contiguous(), p.omap[:cut].contiguous()
    assert cut < pairs
    backend.device_status(reset=True)
    out = p.run_fwd()
    in_grad, w_grad = p.run_bwd()
    assert backend.device_status() >= 3          # one report per launch at least
    kpos = np.minimum(p.km.kpos, cut).astype(np.int32)
    assert err(out, orc.fwd(p.f_np, p.w_np, p.km.n_out, kpos, p.km.imap[:cut], p.km.omap[:cut])) <= TOL[mode]
    assert err(in_grad, orc.dgrad(p.g_np, p.w_np, p.km.n_in, kpos, p.km.imap[:cut], p.km.omap[:cut])) <= TOL[mode]
    assert err(w_grad, orc.wgrad(p.f_np, p.g_np, k_vol, kpos, p.km.imap[:cut], p.km.omap[:cut])) <= TOL[mode]


def test_unaligned_tensors_fall_back_and_are_counted():
    """Tensors that are not 16-byte aligned cannot feed the tensor-core kernels: the CUDA-core kernels run
    instead, the result is still right, and the fallback counter says so."""
    from fgms_b200 import backend
    p = Problem(_sub_map(700, 10, 5), 64, 64, seed=6, mode="fp16")
    storage = torch.zeros(p.feats.numel() + 8, dtype=p.dtype, device="cuda")
    shifted = storage[1:1 + p.feats.numel()].view_as(p.feats)  # 2 bytes off a 16-byte boundary
    shifted.copy_(p.feats)
    assert shifted.data_ptr() % 16 != 0
    p.feats = shifted
    before = backend.fallback_count()
    out = p.run_fwd()
    assert backend.fallback_count() == before + 1
    assert err(out, p.ref_fwd()) <= TOL["fp16"]


def test_results_do_not_depend_on_the_number_of_sms_used():
    """The persistent kernels on fewer SMs (room left for a kernel of another stream) compute the same layer."""
    from fgms_b200 import _lib
    p = Problem(_sub_map(3000, 18, 8), 128, 64, seed=2, mode="fp16")
    try:
        assert _lib.lib.fgms_b200_set_reserved_sms(16) == 0
        _check_all(p)
    finally:
        _lib.lib.fgms_b200_set_reserved_sms(0)
    _check_all(p)
