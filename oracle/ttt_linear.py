"""CPU oracle for the TTT-Linear forward (TEST INFRASTRUCTURE ONLY).

This file is a checker.  Only the tests and the CPU-baseline leg of the benchmark may
import it; the shipped operator never does.

PARITY UNPINNED: the reference ships the TTT-MLP operator only (README.md:18) and holds
no statement, test or fixture of the linear variant.  This file restates the reference's
mini-batch step (kernels/ttt/matching.py:30-125, driver loop :219-252, checkpoint rule
:223-228, LayerNorm eps :75) with the inner model reduced from the two-layer MLP to one
linear layer f(x) = x W1 + b1, i.e. with the hidden layer, W2 and b2 removed and nothing
else changed; it reuses the MLP oracle's LayerNorm helpers, which are pinned to the
reference.  What it is checked against instead (tests/test_linear_oracle.py): the fused
gradient equals torch.autograd's gradient of the inner loss, and the update equals one
plain gradient step with per-token learning rates.

Layouts: XQ, XK, XV, Out [B,H,NC,64,64]; last_eta [B,H,NC,64]; ttt_norm_weight / bias
[1,H,1,64]; W1 [B,H,64,64]; b1 [B,H,1,64]; checkpoints [B,H,ceil(NC/cgs),...].
"""
from __future__ import annotations

from typing import Dict

import torch

from .ttt_mlp import CS, F, _eta5, _ln_bwd, _ln_stats, num_checkpoints, rel_l2  # noqa: F401


def mini_batch_forward(W1, b1, xq, xk, xv, eta, gamma, beta):
    """One mini-batch: returns (Out tile, W1 after the update, b1 after the update).
    eta: [B,H,64,1] per-token learning rates (the reference's last row of its eta matrix)."""
    Z1 = xk @ W1 + b1
    x_hat, std = _ln_stats(Z1)
    grad_output = gamma * x_hat + beta - (xv - xk)          # d(0.5 ||LN(Z1) - (V - K)||^2) / d(LN output)
    grad_Z1 = _ln_bwd(grad_output * gamma, x_hat, std)
    W1n = W1 - (eta * xk).transpose(-1, -2) @ grad_Z1
    b1n = b1 - (eta * grad_Z1).sum(dim=-2, keepdim=True)
    Z1b = xq @ W1n + b1n
    x_hat_b, _ = _ln_stats(Z1b)
    return xq + gamma * x_hat_b + beta, W1n, b1n


def ttt_linear_forward(XQ, XK, XV, last_eta, gamma, beta, W1, b1, cgs: int,
                       dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Whole-sequence forward: Out, checkpoints (state before mini-batch i for i % cgs == 0), final state."""
    up = lambda t: t.to(dtype)
    XQ, XK, XV = up(XQ), up(XK), up(XV)
    eta = _eta5(up(last_eta))
    gamma, beta = up(gamma), up(beta)
    Wc, bc = up(W1), up(b1)
    B, H, NC = XQ.shape[:3]
    n = num_checkpoints(NC, cgs)
    out = torch.empty_like(XQ)
    ck = {"W1_checkpoints": torch.empty(B, H, n, F, F, dtype=dtype),
          "b1_checkpoints": torch.empty(B, H, n, 1, F, dtype=dtype)}
    for i in range(NC):
        if i % cgs == 0:
            ck["W1_checkpoints"][:, :, i // cgs] = Wc
            ck["b1_checkpoints"][:, :, i // cgs] = bc
        out[:, :, i], Wc, bc = mini_batch_forward(Wc, bc, XQ[:, :, i], XK[:, :, i], XV[:, :, i], eta[:, :, i],
                                                  gamma, beta)
    return {"Out": out, **ck, "W1_final": Wc, "b1_final": bc}


def make_inputs(B: int, H: int, NC: int, seed: int = 0, eta_scale: float = 0.1) -> Dict[str, torch.Tensor]:
    """Seeded synthetic inputs, distributions as for the MLP operator: XQ/XK/XV ~ N(0,1) (bf16), last_eta =
    eta_scale * sigmoid(N(0,1)) / 64 (bf16), norm weight 1 + 0.02 N(0,1), bias 0.02 N(0,1), W1 ~ 0.02 N(0,1),
    b1 ~ 0.02 N(0,1) (fp32)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)
    return {
        "XQ": rn(B, H, NC, CS, F).bfloat16(),
        "XK": rn(B, H, NC, CS, F).bfloat16(),
        "XV": rn(B, H, NC, CS, F).bfloat16(),
        "last_eta": (eta_scale * torch.sigmoid(rn(B, H, NC, CS)) / 64).bfloat16(),
        "ttt_norm_weight": 1 + 0.02 * rn(1, H, 1, F),
        "ttt_norm_bias": 0.02 * rn(1, H, 1, F),
        "W1": 0.02 * rn(B, H, F, F),
        "b1": 0.02 * rn(B, H, 1, F),
    }


# ---------------------------------------------------------------------------------------------- backward
def ttt_linear_backward_autograd(XQ, XK, XV, last_eta, gamma, beta, W1, b1, grad_out, grad_W1_last, grad_b1_last,
                                 cgs: int = 1, dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Gradients of sum(Out * grad_out) + sum(W1_final * grad_W1_last) + sum(b1_final * grad_b1_last) by
    torch.autograd through the forward above.  The norm gradients come out summed over the batch ([1,H,1,64])."""
    up = lambda t: t.detach().to(dtype).clone().requires_grad_(True)
    leaves = {"XQ": up(XQ), "XK": up(XK), "XV": up(XV), "last_eta": up(last_eta), "ttt_norm_weight": up(gamma),
              "ttt_norm_bias": up(beta), "W1": up(W1), "b1": up(b1)}
    r = ttt_linear_forward(leaves["XQ"], leaves["XK"], leaves["XV"], leaves["last_eta"], leaves["ttt_norm_weight"],
                           leaves["ttt_norm_bias"], leaves["W1"], leaves["b1"], cgs, dtype=dtype)
    loss = (r["Out"] * grad_out.to(dtype)).sum() + (r["W1_final"] * grad_W1_last.to(dtype)).sum() + \
        (r["b1_final"] * grad_b1_last.to(dtype)).sum()
    loss.backward()
    return {"grad_L_XQ": leaves["XQ"].grad, "grad_L_XK": leaves["XK"].grad, "grad_L_XV": leaves["XV"].grad,
            "grad_L_last_eta": leaves["last_eta"].grad, "grad_L_ttt_norm_weight": leaves["ttt_norm_weight"].grad,
            "grad_L_ttt_norm_bias": leaves["ttt_norm_bias"].grad, "grad_L_W1_init": leaves["W1"].grad,
            "grad_L_b1_init": leaves["b1"].grad}


def mini_batch_backward(W1, b1, xq, xk, xv, eta, gamma, beta, go, G_W, G_b):
    """Hand-derived reverse step of one mini-batch (the statement the backward kernel follows; the reference's
    step, kernels/ttt_backward/matching.py:173-342, with the hidden layer removed).  W1, b1: the state BEFORE
    the mini-batch; go = dL/dOut; G_W, G_b = dL/d(state after the mini-batch).  Returns the input gradients,
    the per-batch-element norm gradients and dL/d(state before)."""
    # forward quantities again
    Z1 = xk @ W1 + b1
    x_hat, std = _ln_stats(Z1)
    e = gamma * x_hat + beta - (xv - xk)
    g = e * gamma
    gZ1 = _ln_bwd(g, x_hat, std)
    W1n = W1 - (eta * xk).transpose(-1, -2) @ gZ1
    b1n = b1 - (eta * gZ1).sum(dim=-2, keepdim=True)
    Z1b = xq @ W1n + b1n
    x_hat_ln, std_ln = _ln_stats(Z1b)
    # output LayerNorm
    d_beta = go.sum(dim=-2, keepdim=True)
    d_gamma = (go * x_hat_ln).sum(dim=-2, keepdim=True)
    gZ1b = _ln_bwd(go * gamma, x_hat_ln, std_ln)
    G_b = G_b + gZ1b.sum(dim=-2, keepdim=True)
    G_W = G_W + xq.transpose(-1, -2) @ gZ1b
    d_xq = go + gZ1b @ W1n.transpose(-1, -2)
    # update rule
    A = -(eta * xk) @ G_W - eta * G_b                      # dL/d(gZ1)
    T1 = gZ1 @ G_W.transpose(-1, -2)
    d_xk = -eta * T1
    d_eta = -(T1 * xk).sum(dim=-1, keepdim=True) - (G_b * gZ1).sum(dim=-1, keepdim=True)
    # second order through the fused LayerNorm + L2 gradient
    s3 = (A * x_hat).sum(dim=-1, keepdim=True)
    Bt = (A - (A.sum(dim=-1, keepdim=True) + x_hat * s3) / F) / std
    gly = gamma * Bt
    d_beta = d_beta + gly.sum(dim=-2, keepdim=True)
    d_gamma = d_gamma + (e * Bt + gly * x_hat).sum(dim=-2, keepdim=True)
    d_xv = -gly
    d_xk = d_xk + gly
    gxh = gly * gamma - (g * s3 + A * (g * x_hat).sum(dim=-1, keepdim=True)) / (F * std)
    gstd = (-gxh * x_hat - A * gZ1) / std
    gZ1in = gxh / std + (x_hat * gstd.sum(dim=-1, keepdim=True) - gxh.sum(dim=-1, keepdim=True) / std) / F
    # inner forward Z1 = K W1 + b1
    d_xk = d_xk + gZ1in @ W1.transpose(-1, -2)
    G_W = G_W + xk.transpose(-1, -2) @ gZ1in
    G_b = G_b + gZ1in.sum(dim=-2, keepdim=True)
    return d_xq, d_xk, d_xv, d_eta, d_gamma, d_beta, G_W, G_b


def ttt_linear_backward(XQ, XK, XV, last_eta, gamma, beta, W1_checkpoints, b1_checkpoints, grad_out, grad_W1_last,
                        grad_b1_last, cgs: int, dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Whole-sequence backward from the forward's checkpoints: per group (last to first) recompute the states,
    then sweep the group in reverse.  Norm gradients per batch element ([B,H,1,64]) like the MLP operator."""
    up = lambda t: t.to(dtype)
    XQ, XK, XV, go = up(XQ), up(XK), up(XV), up(grad_out)
    eta = _eta5(up(last_eta))
    gamma, beta = up(gamma), up(beta)
    B, H, NC = XQ.shape[:3]
    G_W, G_b = up(grad_W1_last).clone(), up(grad_b1_last).clone()
    r = {k: torch.zeros_like(XQ) for k in ("grad_L_XQ", "grad_L_XK", "grad_L_XV")}
    r["grad_L_last_eta"] = torch.zeros(B, H, NC, CS, 1, dtype=dtype)
    d_gamma = torch.zeros(B, H, 1, F, dtype=dtype)
    d_beta = torch.zeros(B, H, 1, F, dtype=dtype)
    for c in reversed(range(num_checkpoints(NC, cgs))):
        i0, i1 = c * cgs, min(NC, (c + 1) * cgs)
        W, b = up(W1_checkpoints[:, :, c]), up(b1_checkpoints[:, :, c])
        states = []
        for i in range(i0, i1):
            states.append((W, b))
            _, W, b = mini_batch_forward(W, b, XQ[:, :, i], XK[:, :, i], XV[:, :, i], eta[:, :, i], gamma, beta)
        for i in reversed(range(i0, i1)):
            W, b = states[i - i0]
            dq, dk, dv, de, dg, db, G_W, G_b = mini_batch_backward(W, b, XQ[:, :, i], XK[:, :, i], XV[:, :, i],
                                                                   eta[:, :, i], gamma, beta, go[:, :, i], G_W, G_b)
            r["grad_L_XQ"][:, :, i], r["grad_L_XK"][:, :, i], r["grad_L_XV"][:, :, i] = dq, dk, dv
            r["grad_L_last_eta"][:, :, i] = de
            d_gamma += dg
            d_beta += db
    r.update({"grad_L_ttt_norm_weight": d_gamma, "grad_L_ttt_norm_bias": d_beta, "grad_L_W1_init": G_W,
              "grad_L_b1_init": G_b})
    return r
