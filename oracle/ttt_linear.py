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
