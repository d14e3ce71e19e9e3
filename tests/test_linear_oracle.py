"""The TTT-Linear oracle has no reference statement to be pinned to (the reference ships the MLP
operator only), so its algebra is checked against first principles: the fused LayerNorm + L2 gradient
equals torch.autograd's gradient of the inner loss 0.5 * ||gamma * LN(K W + b) + beta - (V - K)||^2
with respect to Z = K W + b, the update equals one gradient step on (W, b) with per-token learning
rates, and the driver loop applies the checkpoint rule of the MLP oracle."""
import torch

from oracle import ttt_linear as lin
from oracle import ttt_mlp as orc


def test_update_is_a_gradient_step_on_the_inner_loss():
    torch.manual_seed(0)
    B, H = 1, 2
    dt = torch.float64
    xk, xv, xq = (torch.randn(B, H, 64, 64, dtype=dt) for _ in range(3))
    eta = 0.01 * torch.rand(B, H, 64, 1, dtype=dt)
    gamma = 1 + 0.1 * torch.randn(1, H, 1, 64, dtype=dt)
    beta = 0.1 * torch.randn(1, H, 1, 64, dtype=dt)
    W = (0.1 * torch.randn(B, H, 64, 64, dtype=dt)).requires_grad_()
    b = (0.1 * torch.randn(B, H, 1, 64, dtype=dt)).requires_grad_()
    # per-token losses, each token's gradient scaled by its own learning rate
    Z = xk @ W + b
    mu = Z.mean(-1, keepdim=True)
    xh = (Z - mu) / torch.sqrt(Z.var(-1, keepdim=True, unbiased=False) + orc.LN_EPS)
    per_token = 0.5 * ((gamma * xh + beta - (xv - xk)) ** 2).sum(-1, keepdim=True)
    (eta * per_token).sum().backward()
    out, Wn, bn = lin.mini_batch_forward(W.detach(), b.detach(), xq, xk, xv, eta, gamma, beta)
    assert orc.rel_l2(Wn, W.detach() - W.grad) < 1e-10
    assert orc.rel_l2(bn, b.detach() - b.grad) < 1e-10
    # the output uses the updated state
    Zb = xq @ Wn + bn
    xhb = (Zb - Zb.mean(-1, keepdim=True)) / torch.sqrt(Zb.var(-1, keepdim=True, unbiased=False) + orc.LN_EPS)
    assert orc.rel_l2(out, xq + gamma * xhb + beta) < 1e-12


def test_driver_loop_checkpoints_and_final_state():
    d = lin.make_inputs(1, 2, 5, seed=3)
    r = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                               d["W1"], d["b1"], 2)
    assert r["W1_checkpoints"].shape == (1, 2, 3, 64, 64) and r["b1_checkpoints"].shape == (1, 2, 3, 1, 64)
    assert torch.equal(r["W1_checkpoints"][:, :, 0], d["W1"]) and torch.equal(r["b1_checkpoints"][:, :, 0], d["b1"])
    # a sequence restarted from checkpoint 1 (the state before mini-batch 2) gives the same tail
    t = lin.ttt_linear_forward(d["XQ"][:, :, 2:], d["XK"][:, :, 2:], d["XV"][:, :, 2:], d["last_eta"][:, :, 2:],
                               d["ttt_norm_weight"], d["ttt_norm_bias"], r["W1_checkpoints"][:, :, 1],
                               r["b1_checkpoints"][:, :, 1], 2)
    assert torch.equal(t["Out"], r["Out"][:, :, 2:])
    assert torch.equal(t["W1_final"], r["W1_final"]) and torch.equal(t["b1_final"], r["b1_final"])
    assert torch.equal(t["W1_checkpoints"][:, :, 1], r["W1_checkpoints"][:, :, 2])


def test_hand_derived_backward_equals_autograd():
    """The reverse step the backward kernel follows, against torch.autograd through the forward, in fp64, with
    non-zero upstream state gradients and a ragged last checkpoint group."""
    torch.manual_seed(1)
    B, H, NC, cgs = 2, 2, 5, 2
    dt = torch.float64
    d = lin.make_inputs(B, H, NC, seed=9)
    d = {k: v.to(dt) for k, v in d.items()}
    go = torch.randn(B, H, NC, 64, 64, dtype=dt)
    gW = 1e-2 * torch.randn(B, H, 64, 64, dtype=dt)
    gb = 1e-2 * torch.randn(B, H, 1, 64, dtype=dt)
    f = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                               d["W1"], d["b1"], cgs, dtype=dt)
    a = lin.ttt_linear_backward_autograd(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                         d["ttt_norm_bias"], d["W1"], d["b1"], go, gW, gb, cgs, dtype=dt)
    h = lin.ttt_linear_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                                f["W1_checkpoints"], f["b1_checkpoints"], go, gW, gb, cgs, dtype=dt)
    for k in ("grad_L_XQ", "grad_L_XK", "grad_L_XV", "grad_L_W1_init", "grad_L_b1_init"):
        assert orc.rel_l2(h[k], a[k]) < 1e-9, k
    assert orc.rel_l2(h["grad_L_last_eta"].squeeze(-1), a["grad_L_last_eta"]) < 1e-9
    assert orc.rel_l2(h["grad_L_ttt_norm_weight"].sum(0, keepdim=True), a["grad_L_ttt_norm_weight"]) < 1e-9
    assert orc.rel_l2(h["grad_L_ttt_norm_bias"].sum(0, keepdim=True), a["grad_L_ttt_norm_bias"]) < 1e-9
