"""The oracle (Python and C restatements) against the reference's own CPU outputs."""
import numpy as np
import pytest
import torch

from fgms_b200 import clouds, maps
from oracle import c_oracle, spconv_oracle as orc


def test_python_literal_is_bit_exact_with_reference(golden):
    g = golden
    if g["imap"].size * g["weights"].shape[1] * g["weights"].shape[2] > 40_000:
        pytest.skip("pure-Python loop kept to the small fixtures")
    out = orc.fwd_literal(g["feats"], g["weights"], int(g["n_out"]), g["knnz"], g["imap"], g["omap"],
                          bool(g["precompute"]))
    assert np.array_equal(out, g["out"])
    in_grad, w_grad = orc.bwd_literal(g["grad_out"], g["weights"], g["feats"], int(g["n_in"]), g["knnz"],
                                      g["imap"], g["omap"])
    assert np.array_equal(in_grad, g["in_grad"])
    assert np.array_equal(w_grad, g["w_grad"])


def test_c_f32_is_bit_exact_with_reference(golden):
    g = golden
    out = c_oracle.fwd(g["feats"], g["weights"], int(g["n_out"]), g["knnz"], g["imap"], g["omap"],
                       bool(g["precompute"]), acc="f32")
    assert np.array_equal(out, g["out"])
    in_grad, w_grad = c_oracle.bwd(g["grad_out"], g["weights"], g["feats"], int(g["n_in"]), g["knnz"],
                                   g["imap"], g["omap"], acc="f32")
    assert np.array_equal(in_grad, g["in_grad"])
    assert np.array_equal(w_grad, g["w_grad"])


@pytest.mark.parametrize("impl", ["c", "torch"])
def test_f64_ground_truth_matches_reference(golden, impl):
    g = golden
    n_in, n_out, k_vol = int(g["n_in"]), int(g["n_out"]), g["weights"].shape[0]
    if impl == "c":
        out = c_oracle.fwd(g["feats"], g["weights"], n_out, g["knnz"], g["imap"], g["omap"], bool(g["precompute"]))
        in_grad, w_grad = c_oracle.bwd(g["grad_out"], g["weights"], g["feats"], n_in, g["knnz"], g["imap"], g["omap"])
    else:
        out = orc.fwd(g["feats"], g["weights"], n_out, g["kpos"], g["imap"], g["omap"], bool(g["precompute"]))
        in_grad = orc.dgrad(g["grad_out"], g["weights"], n_in, g["kpos"], g["imap"], g["omap"])
        w_grad = orc.wgrad(g["feats"], g["grad_out"], k_vol, g["kpos"], g["imap"], g["omap"])
    # the reference accumulates in fp32; the fp64 ground truth differs by fp32 rounding only
    assert orc.rel_err(out, g["out"]) < 2e-6
    assert orc.rel_err(in_grad, g["in_grad"]) < 2e-6
    assert orc.rel_err(w_grad, g["w_grad"]) < 2e-6


def test_vectorised_f32_matches_f64_on_a_larger_case():
    coords = clouds.surface_cloud(3000, 48, 7)
    km = maps.build_submanifold_map(coords)
    f, w, g = clouds.make_tensors(km.n_in, km.n_out, 24, 40, km.k_vol, 7)
    ref = orc.fwd(f, w, km.n_out, km.kpos, km.imap, km.omap)
    got = orc.fwd(f, w, km.n_out, km.kpos, km.imap, km.omap, acc=torch.float32)
    assert orc.rel_err(got, ref) < 1e-5
    c = c_oracle.fwd(f, w, km.n_out, km.knnz, km.imap, km.omap)
    assert orc.rel_err(c, ref) < 1e-12
    ig_c, wg_c = c_oracle.bwd(g, w, f, km.n_in, km.knnz, km.imap, km.omap)
    assert orc.rel_err(ig_c, orc.dgrad(g, w, km.n_in, km.kpos, km.imap, km.omap)) < 1e-12
    assert orc.rel_err(wg_c, orc.wgrad(f, g, km.k_vol, km.kpos, km.imap, km.omap)) < 1e-12


def test_empty_inputs():
    w = np.zeros((27, 4, 4), np.float32)
    kpos = np.zeros(28, np.int32)
    e = np.zeros(0, np.int32)
    assert orc.fwd(np.zeros((0, 4), np.float32), w, 0, kpos, e, e).shape == (0, 4)
    assert orc.wgrad(np.zeros((0, 4), np.float32), np.zeros((0, 4), np.float32), 27, kpos, e, e).shape == (27, 4, 4)
    assert orc.rel_err(np.zeros((0, 4)), np.zeros((0, 4))) == 0.0
