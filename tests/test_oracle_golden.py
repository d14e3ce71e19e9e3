"""The oracle against (a) fixtures produced by the reference's own PyTorch functions,
(b) the reference's functions imported live when its tree is present, and
(c) torch.autograd through the oracle's forward in fp64."""
import os

import numpy as np
import pytest
import torch

from oracle import ttt_mlp as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden", "ttt_mlp_golden.npz")
FWD_KEYS = ["Out", "W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints",
            "W1_final", "b1_final", "W2_final", "b2_final"]
BWD_KEYS = ["grad_L_ttt_norm_weight", "grad_L_ttt_norm_bias", "grad_L_W1_init", "grad_L_b1_init",
            "grad_L_W2_init", "grad_L_b2_init", "grad_L_last_eta", "grad_L_XQ", "grad_L_XK", "grad_L_XV"]


def _case(blob, name):
    B, H, NC, cgs, seed = [int(x) for x in blob[f"{name}/cfg"]]
    es = float(blob[f"{name}/eta_scale"][0])
    d = orc.make_inputs(B, H, NC, seed=seed, eta_scale=es, backward=True)
    sums = np.array([float(v.double().sum()) for v in d.values()])
    np.testing.assert_allclose(sums, blob[f"{name}/input_sum"], rtol=1e-12,
                               err_msg="seeded input recipe drifted from the fixture's")
    return d, cgs


@pytest.mark.parametrize("name", ["ragged", "even"])
def test_oracle_matches_reference_fixture(name):
    blob = np.load(GOLD)
    d, cgs = _case(blob, name)
    fwd = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                          d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    for k in FWD_KEYS:
        # same fp32 arithmetic, same op order: only reduction-order noise is allowed
        assert orc.rel_l2(fwd[k], torch.from_numpy(blob[f"{name}/{k}"])) < 2e-6, k
    bwd = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                           d["ttt_norm_bias"], fwd["W1_checkpoints"], fwd["b1_checkpoints"],
                           fwd["W2_checkpoints"], fwd["b2_checkpoints"], d["grad_L_W1_last"],
                           d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                           d["grad_L_XQW_mini_batch"], cgs)
    for k in BWD_KEYS:
        assert orc.rel_l2(bwd[k], torch.from_numpy(blob[f"{name}/{k}"])) < 2e-5, k


@pytest.mark.parametrize("B,H,NC,cgs", [(1, 2, 3, 2), (2, 2, 4, 4), (1, 1, 1, 1)])
def test_hand_backward_equals_autograd_fp64(B, H, NC, cgs):
    d = orc.make_inputs(B, H, NC, seed=3, eta_scale=1.0, backward=True)
    f64 = torch.float64
    fwd = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                          d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], cgs, dtype=f64)
    hand = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                            d["ttt_norm_bias"], fwd["W1_checkpoints"], fwd["b1_checkpoints"],
                            fwd["W2_checkpoints"], fwd["b2_checkpoints"], d["grad_L_W1_last"],
                            d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                            d["grad_L_XQW_mini_batch"], cgs, dtype=f64)
    auto = orc.ttt_backward_autograd(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                     d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"],
                                     d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"],
                                     d["grad_L_b2_last"], d["grad_L_XQW_mini_batch"])
    for k in BWD_KEYS:
        # the hand VJP uses the reference's 8-digit GELU constants; autograd uses torch's
        assert orc.rel_l2(hand[k], auto[k]) < 1e-6, k


def test_gelu_family_against_autograd():
    x = torch.linspace(-6, 6, 4001, dtype=torch.float64, requires_grad=True)
    y = orc.gelu_tanh(x)
    (g1,) = torch.autograd.grad(y.sum(), x, create_graph=True)
    (g2,) = torch.autograd.grad(g1.sum(), x)
    assert (orc.gelu_bwd(x) - g1).abs().max() < 1e-7
    assert (orc.gelu_bwd_derivative(x) - g2).abs().max() < 1e-6


def test_checkpoint_rule_and_ragged_count():
    d = orc.make_inputs(1, 1, 5, seed=0)
    r = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                        d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], cgs=2)
    assert r["W1_checkpoints"].shape == (1, 1, 3, 64, 256)
    assert torch.equal(r["W1_checkpoints"][:, :, 0], d["W1"])
    # last_eta rank 4 and rank 5 are the same input
    r5 = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"].unsqueeze(-1), d["ttt_norm_weight"],
                         d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], cgs=2)
    assert torch.equal(r["Out"], r5["Out"])


REF = os.environ.get("TTT_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "kernels/ttt_backward/matching.py")),
                    reason="reference tree not present on this machine")
def test_oracle_matches_live_reference_functions():
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_golden
    ref_fwd, ref_bwd = make_golden.load_reference(REF)
    d = orc.make_inputs(1, 2, 5, seed=7, eta_scale=0.5, backward=True)
    cgs = 2
    with torch.no_grad():
        want = make_golden.run_reference(ref_fwd, ref_bwd, d, cgs)
    fwd = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                          d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    bwd = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                           d["ttt_norm_bias"], fwd["W1_checkpoints"], fwd["b1_checkpoints"],
                           fwd["W2_checkpoints"], fwd["b2_checkpoints"], d["grad_L_W1_last"],
                           d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                           d["grad_L_XQW_mini_batch"], cgs)
    for k in FWD_KEYS:
        assert orc.rel_l2(fwd[k], want[k]) < 2e-6, k
    for k in BWD_KEYS:
        assert orc.rel_l2(bwd[k], want[k]) < 2e-5, k
