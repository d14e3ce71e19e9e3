"""CPU oracle for the TTT-MLP forward / backward path (TEST INFRASTRUCTURE ONLY).

This file is a checker.  Only the tests, the smoke entry and the CPU-baseline leg
of the benchmark may import it; the shipped operator never does.

It restates, in plain PyTorch eager arithmetic (fp32 by default, fp64 on request),
the algorithm of the reference's own PyTorch statement of the path:

  * forward mini-batch      kernels/ttt/matching.py:30-125
  * forward driver loop     kernels/ttt/matching.py:219-252   (checkpoint rule :223-228)
  * backward mini-batch     kernels/ttt_backward/matching.py:173-342
  * backward driver loop    kernels/ttt_backward/matching.py:539-663
                            (ragged last group: :355, :552, :598)
  * GELU' / GELU''          kernels/ttt_backward/matching.py:42-55
  * LayerNorm eps = 1e-8    kernels/ttt/matching.py:75

Parity pin: tests/test_oracle_golden.py imports the reference's two
`matching.py` files (when the reference tree is present) and checks every function
here against them; tests/golden/ holds outputs of the *reference's* functions on
seeded inputs, produced by tests/golden/make_golden.py, so the pin also holds on
machines without the reference tree.  The third-party arithmetic underneath is
PyTorch itself (the reference requires torch>=2.4, unpinned above): for PyTorch
version drift the parity is "unpinned" beyond those fixtures.

Layouts follow the operator API (kernels/ttt/ttt.cu:594-611):
  XQ, XK, XV, Out, grad_XQW : [B, H, NC, 64, 64]
  last_eta                  : [B, H, NC, 64] (or [..., 64, 1])
  ttt_norm_weight / bias    : [1, H, 1, 64]
  W1 [B,H,64,256]  b1 [B,H,1,256]  W2 [B,H,256,64]  b2 [B,H,1,64]
  checkpoints               : [B, H, ceil(NC/cgs), ...state shape...]
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

CS = 64      # tokens per mini-batch
F = 64       # head dimension
HID = 256    # MLP hidden width (4 * F)
LN_EPS = 1e-8

# Constants exactly as the reference writes them (matching.py:7-10, :42-55).
_K0 = 0.79788456
_K1 = 0.044715
_K2 = 0.1070322243


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """tanh-approximated GELU (kernels/ttt/matching.py:65)."""
    return torch.nn.functional.gelu(x, approximate="tanh")


def gelu_bwd(x: torch.Tensor) -> torch.Tensor:
    """d gelu_tanh / dx  (kernels/ttt/matching.py:7-10)."""
    t = torch.tanh(_K0 * x * (1 + _K1 * x * x))
    return 0.5 * x * ((1 - t * t) * (_K0 + _K2 * x * x)) + 0.5 * (1 + t)


def gelu_bwd_derivative(x: torch.Tensor) -> torch.Tensor:
    """d^2 gelu_tanh / dx^2  (kernels/ttt_backward/matching.py:47-55)."""
    t = torch.tanh(_K0 * x * (1 + _K1 * x * x))
    term1 = _K0
    term2 = 6 * _K0 * _K1 * x ** 2
    term3 = x * t * (_K0 + 3 * _K0 * _K1 * x ** 2) ** 2
    return (1 - t ** 2) * (term1 + term2 - term3)


def _ln_stats(z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    mu = z.mean(dim=-1, keepdim=True)
    var = z.var(dim=-1, keepdim=True, unbiased=False)
    std = torch.sqrt(var + LN_EPS)
    return (z - mu) / std, std


def _ln_bwd(gx_hat: torch.Tensor, x_hat: torch.Tensor, std: torch.Tensor) -> torch.Tensor:
    """Backward of x_hat = (z - mean) / std w.r.t. z (matching.py:85-94)."""
    return (
        (1.0 / F)
        * (
            F * gx_hat
            - gx_hat.sum(dim=-1, keepdim=True)
            - x_hat * (gx_hat * x_hat).sum(dim=-1, keepdim=True)
        )
        / std
    )


@dataclass
class MiniBatchSaved:
    """Everything the reverse sweep needs from one mini-batch of the forward."""
    W1: torch.Tensor
    b1: torch.Tensor
    W2: torch.Tensor
    b2: torch.Tensor
    Z1: torch.Tensor
    X2: torch.Tensor
    std_fused: torch.Tensor
    x_hat_fused: torch.Tensor
    grad_output_fused: torch.Tensor
    grad_x_hat_fused: torch.Tensor
    grad_l_wrt_Z2: torch.Tensor
    grad_l_wrt_Z1: torch.Tensor
    Z1_bar: torch.Tensor
    X2_bar: torch.Tensor
    std_ln: torch.Tensor
    x_hat_ln: torch.Tensor


def mini_batch_forward(W1, b1, W2, b2, xq, xk, xv, eta, gamma, beta, save: bool = False):
    """One mini-batch of the forward (kernels/ttt/matching.py:30-125).

    xq/xk/xv: [B,H,64,64]; eta: [B,H,64,1] (the reference's last row of eta_mb);
    gamma/beta: [1 or B, H, 1, 64].  Returns (out, W1', b1', W2', b2'[, saved]).
    """
    Z1 = xk @ W1 + b1
    X2 = gelu_tanh(Z1)
    Z2 = X2 @ W2 + b2
    target = xv - xk

    x_hat_fused, std_fused = _ln_stats(Z2)
    y = gamma * x_hat_fused + beta
    grad_output_fused = y - target
    grad_x_hat_fused = grad_output_fused * gamma
    gZ2 = _ln_bwd(grad_x_hat_fused, x_hat_fused, std_fused)
    gZ1 = gZ2 @ W2.transpose(-1, -2) * gelu_bwd(Z1)

    W1n = W1 - (eta * xk).transpose(-1, -2) @ gZ1
    b1n = b1 - (eta * gZ1).sum(dim=-2, keepdim=True)
    W2n = W2 - (eta * X2).transpose(-1, -2) @ gZ2
    b2n = b2 - (eta * gZ2).sum(dim=-2, keepdim=True)

    Z1_bar = xq @ W1n + b1n
    X2_bar = gelu_tanh(Z1_bar)
    Z2_bar = X2_bar @ W2n + b2n
    x_hat_ln, std_ln = _ln_stats(Z2_bar)
    out = xq + gamma * x_hat_ln + beta
    if not save:
        return out, W1n, b1n, W2n, b2n
    saved = MiniBatchSaved(W1, b1, W2, b2, Z1, X2, std_fused, x_hat_fused, grad_output_fused,
                           grad_x_hat_fused, gZ2, gZ1, Z1_bar, X2_bar, std_ln, x_hat_ln)
    return out, W1n, b1n, W2n, b2n, saved


def _eta5(last_eta: torch.Tensor) -> torch.Tensor:
    """Accept [B,H,NC,64] or [B,H,NC,64,1] (the two ranks the reference scripts use)."""
    return last_eta if last_eta.dim() == 5 else last_eta.unsqueeze(-1)


def num_checkpoints(NC: int, cgs: int) -> int:
    return math.ceil(NC / cgs)


def ttt_forward(XQ, XK, XV, last_eta, gamma, beta, W1, b1, W2, b2, cgs: int,
                dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Whole-sequence forward (driver loop kernels/ttt/matching.py:219-252).

    Inputs of any float dtype are upcast to `dtype` first (the reference script
    feeds the bf16-rounded tensors upcast to fp32).  Returns Out, the four
    checkpoint tensors (state *before* mini-batch i for i % cgs == 0) and the
    final state (which the reference computes but never stores).
    """
    up = lambda t: t.to(dtype)
    XQ, XK, XV = up(XQ), up(XK), up(XV)
    eta = _eta5(up(last_eta))
    gamma, beta = up(gamma), up(beta)
    W1c, b1c, W2c, b2c = up(W1), up(b1), up(W2), up(b2)
    B, H, NC = XQ.shape[:3]
    n = num_checkpoints(NC, cgs)
    out = torch.empty_like(XQ)
    ck = {
        "W1_checkpoints": torch.empty(B, H, n, F, HID, dtype=dtype),
        "b1_checkpoints": torch.empty(B, H, n, 1, HID, dtype=dtype),
        "W2_checkpoints": torch.empty(B, H, n, HID, F, dtype=dtype),
        "b2_checkpoints": torch.empty(B, H, n, 1, F, dtype=dtype),
    }
    for i in range(NC):
        if i % cgs == 0:
            c = i // cgs
            ck["W1_checkpoints"][:, :, c] = W1c
            ck["b1_checkpoints"][:, :, c] = b1c
            ck["W2_checkpoints"][:, :, c] = W2c
            ck["b2_checkpoints"][:, :, c] = b2c
        out[:, :, i], W1c, b1c, W2c, b2c = mini_batch_forward(
            W1c, b1c, W2c, b2c, XQ[:, :, i], XK[:, :, i], XV[:, :, i], eta[:, :, i], gamma, beta)
    res = {"Out": out, "W1_final": W1c, "b1_final": b1c, "W2_final": W2c, "b2_final": b2c}
    res.update(ck)
    return res


def mini_batch_backward(s: MiniBatchSaved, W1_post, W2_post, xq, xk, eta, gamma,
                        G_W1, G_b1, G_W2, G_b2, go):
    """Hand-derived VJP of one mini-batch (kernels/ttt_backward/matching.py:173-342).

    G_* are dL/d(post-update state); go = dL/dOut for this mini-batch.  The
    norm-parameter gradients are returned per batch element ([B,H,1,64]), the
    layout the operator writes (kernels/ttt_backward/ttt.cu:1437-1438); the
    reference function sums them over the batch (`.sum(dim=0)`), which the caller
    of the operator does afterwards (matching.py:522-523).
    Returns (d_gamma, d_beta, G_W1', G_b1', G_W2', G_b2', dXQ, dXV, dXK, d_eta).
    """
    # Stage 4: output LayerNorm
    d_beta_ln = go.sum(dim=-2, keepdim=True)
    d_gamma_ln = (go * s.x_hat_ln).sum(dim=-2, keepdim=True)
    gZ2_bar = _ln_bwd(go * gamma, s.x_hat_ln, s.std_ln)

    # Stage 3: post-update forward and the update rule
    gX2_bar = gZ2_bar @ W2_post.transpose(-2, -1)
    gZ1_bar = gX2_bar * gelu_bwd(s.Z1_bar)
    G_b2 = G_b2 + gZ2_bar.sum(dim=-2, keepdim=True)
    G_W2 = G_W2 + s.X2_bar.transpose(-2, -1) @ gZ2_bar
    G_b1 = G_b1 + gZ1_bar.sum(dim=-2, keepdim=True)
    G_W1 = G_W1 + xq.transpose(-2, -1) @ gZ1_bar

    gp1 = gelu_bwd(s.Z1)
    A1 = -(eta * xk) @ G_W1 - eta * G_b1                         # dL/d grad_l_wrt_Z1
    A2 = -(eta * s.X2) @ G_W2 - eta * G_b2 + (A1 * gp1) @ s.W2   # dL/d grad_l_wrt_Z2
    dXQ_mm = gZ1_bar @ W1_post.transpose(-2, -1)
    T1 = s.grad_l_wrt_Z1 @ G_W1.transpose(-2, -1)
    T2 = s.grad_l_wrt_Z2 @ G_W2.transpose(-2, -1)
    dXK_upd = -T1 * eta
    d_eta = (
        -(T2 * s.X2).sum(dim=-1, keepdim=True)
        - (G_b2 * s.grad_l_wrt_Z2).sum(dim=-1, keepdim=True)
        - (T1 * xk).sum(dim=-1, keepdim=True)
        - (G_b1 * s.grad_l_wrt_Z1).sum(dim=-1, keepdim=True)
    )

    # Stage 2: second order through the fused LayerNorm + L2 gradient
    dW2_pre = (A1 * gp1).transpose(-2, -1) @ s.grad_l_wrt_Z2
    xh, sd = s.x_hat_fused, s.std_fused
    Bt = (1.0 / sd) * (A2 + (-1.0 / F) * (A2.sum(dim=-1, keepdim=True)
                                           + xh * (A2 * xh).sum(dim=-1, keepdim=True)))
    gLy = gamma * Bt
    d_gamma_f = (s.grad_output_fused * Bt + gLy * xh).sum(dim=-2, keepdim=True)
    d_beta_f = gLy.sum(dim=-2, keepdim=True)
    gxh = gLy * gamma + (-1.0 / (F * sd)) * (
        s.grad_x_hat_fused * (A2 * xh).sum(dim=-1, keepdim=True)
        + A2 * (s.grad_x_hat_fused * xh).sum(dim=-1, keepdim=True))
    gstd = (-gxh * xh - A2 * s.grad_l_wrt_Z2) / sd
    gZ2 = gxh * (1.0 / sd) + (1.0 / F) * (gstd.sum(dim=-1, keepdim=True) * xh
                                          - gxh.sum(dim=-1, keepdim=True) * (1.0 / sd))
    g_target = -gamma * Bt

    # Stage 1: inner forward
    gX2 = gZ2 @ s.W2.transpose(-2, -1) - T2 * eta
    gZ1 = gX2 * gp1 + (s.grad_l_wrt_Z2 @ s.W2.transpose(-2, -1)) * A1 * gelu_bwd_derivative(s.Z1)

    dXQ = go + dXQ_mm
    dXK = -g_target + dXK_upd + gZ1 @ s.W1.transpose(-2, -1)
    dXV = g_target
    G_W2n = G_W2 + dW2_pre + s.X2.transpose(-2, -1) @ gZ2
    G_b2n = G_b2 + gZ2.sum(-2, keepdim=True)
    G_W1n = G_W1 + xk.transpose(-2, -1) @ gZ1
    G_b1n = G_b1 + gZ1.sum(-2, keepdim=True)
    return (d_gamma_ln + d_gamma_f, d_beta_ln + d_beta_f, G_W1n, G_b1n, G_W2n, G_b2n,
            dXQ, dXV, dXK, d_eta)


def ttt_backward(XQ, XK, XV, last_eta, gamma, beta,
                 W1_checkpoints, b1_checkpoints, W2_checkpoints, b2_checkpoints,
                 grad_W1_last, grad_b1_last, grad_W2_last, grad_b2_last, grad_XQW,
                 cgs: int, dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Whole-sequence backward: per checkpoint group (last to first) recompute the
    forward from that group's checkpoint, then sweep it in reverse
    (driver kernels/ttt_backward/matching.py:539-663).

    Each group starts from *its own* checkpoint, exactly as the operator does, so
    arbitrary (even inconsistent) checkpoints give a well-defined answer.
    """
    up = lambda t: t.to(dtype)
    XQ, XK, XV, go_all = up(XQ), up(XK), up(XV), up(grad_XQW)
    eta = _eta5(up(last_eta))
    gamma, beta = up(gamma), up(beta)
    W1k, b1k, W2k, b2k = up(W1_checkpoints), up(b1_checkpoints), up(W2_checkpoints), up(b2_checkpoints)
    B, H, NC = XQ.shape[:3]
    n = num_checkpoints(NC, cgs)
    assert W1k.shape[2] == n, "checkpoint count must be ceil(NC / cgs)"
    G_W1, G_b1, G_W2, G_b2 = (up(grad_W1_last).clone(), up(grad_b1_last).clone(),
                              up(grad_W2_last).clone(), up(grad_b2_last).clone())
    dXQ, dXK, dXV = torch.empty_like(XQ), torch.empty_like(XQ), torch.empty_like(XQ)
    d_eta = torch.empty(B, H, NC, CS, 1, dtype=dtype)
    d_gamma = torch.zeros(B, H, 1, F, dtype=dtype)
    d_beta = torch.zeros(B, H, 1, F, dtype=dtype)
    for c in range(n - 1, -1, -1):
        W1c, b1c, W2c, b2c = W1k[:, :, c], b1k[:, :, c], W2k[:, :, c], b2k[:, :, c]
        saved = []
        idx = [i for i in range(c * cgs, min((c + 1) * cgs, NC))]
        for i in idx:
            _, W1c, b1c, W2c, b2c, s = mini_batch_forward(
                W1c, b1c, W2c, b2c, XQ[:, :, i], XK[:, :, i], XV[:, :, i], eta[:, :, i],
                gamma, beta, save=True)
            saved.append(s)
        W1p, W2p = W1c, W2c
        for j in range(len(idx) - 1, -1, -1):
            i, s = idx[j], saved[j]
            (dg, db, G_W1, G_b1, G_W2, G_b2, dXQ[:, :, i], dXV[:, :, i], dXK[:, :, i],
             d_eta[:, :, i]) = mini_batch_backward(
                s, W1p, W2p, XQ[:, :, i], XK[:, :, i], eta[:, :, i], gamma,
                G_W1, G_b1, G_W2, G_b2, go_all[:, :, i])
            W1p, W2p = s.W1, s.W2
            d_gamma += dg
            d_beta += db
    return {
        "grad_L_ttt_norm_weight": d_gamma, "grad_L_ttt_norm_bias": d_beta,
        "grad_L_W1_init": G_W1, "grad_L_b1_init": G_b1,
        "grad_L_W2_init": G_W2, "grad_L_b2_init": G_b2,
        "grad_L_last_eta": d_eta, "grad_L_XQ": dXQ, "grad_L_XK": dXK, "grad_L_XV": dXV,
    }


def ttt_backward_autograd(XQ, XK, XV, last_eta, gamma, beta, W1, b1, W2, b2,
                          grad_W1_last, grad_b1_last, grad_W2_last, grad_b2_last, grad_XQW,
                          dtype: torch.dtype = torch.float64) -> Dict[str, torch.Tensor]:
    """Independent cross-check: torch.autograd through the forward from the initial
    state.  Equals `ttt_backward` whenever the checkpoints came from the forward.
    Norm-parameter gradients are per batch element, like the operator's.
    """
    up = lambda t: t.detach().to(dtype)
    B, H, NC = XQ.shape[:3]
    leaves = {
        "XQ": up(XQ), "XK": up(XK), "XV": up(XV), "eta": _eta5(up(last_eta)),
        "gamma": up(gamma).expand(B, H, 1, F).clone(), "beta": up(beta).expand(B, H, 1, F).clone(),
        "W1": up(W1), "b1": up(b1), "W2": up(W2), "b2": up(b2),
    }
    for v in leaves.values():
        v.requires_grad_(True)
    W1c, b1c, W2c, b2c = leaves["W1"], leaves["b1"], leaves["W2"], leaves["b2"]
    loss = 0.0
    go = up(grad_XQW)
    for i in range(NC):
        out, W1c, b1c, W2c, b2c = mini_batch_forward(
            W1c, b1c, W2c, b2c, leaves["XQ"][:, :, i], leaves["XK"][:, :, i], leaves["XV"][:, :, i],
            leaves["eta"][:, :, i], leaves["gamma"], leaves["beta"])
        loss = loss + (out * go[:, :, i]).sum()
    loss = loss + (W1c * up(grad_W1_last)).sum() + (b1c * up(grad_b1_last)).sum() \
        + (W2c * up(grad_W2_last)).sum() + (b2c * up(grad_b2_last)).sum()
    loss.backward()
    g = {k: v.grad for k, v in leaves.items()}
    return {
        "grad_L_ttt_norm_weight": g["gamma"], "grad_L_ttt_norm_bias": g["beta"],
        "grad_L_W1_init": g["W1"], "grad_L_b1_init": g["b1"],
        "grad_L_W2_init": g["W2"], "grad_L_b2_init": g["b2"],
        "grad_L_last_eta": g["eta"], "grad_L_XQ": g["XQ"], "grad_L_XK": g["XK"], "grad_L_XV": g["XV"],
    }


def make_inputs(B: int, H: int, NC: int, seed: int = 0, eta_scale: float = 0.1,
                backward: bool = False) -> Dict[str, torch.Tensor]:
    """Seeded synthetic inputs with the benchmark configurations' shapes and
    distributions: XQ/XK/XV ~ N(0,1) rounded to bf16; last_eta =
    eta_scale * sigmoid(N(0,1)) / 64 (bf16); norm weight 1 + 0.02 N(0,1), bias
    0.02 N(0,1); W1, W2 ~ 0.02 N(0,1), b1 = b2 = 0 (fp32).  With `backward`:
    grad_XQW ~ N(0,1) bf16 and upstream state grads ~ 1e-3 N(0,1) fp32.
    Drawn on the CPU generator in a fixed order so every machine sees the same data.
    """
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)
    d = {
        "XQ": rn(B, H, NC, CS, F).bfloat16(),
        "XK": rn(B, H, NC, CS, F).bfloat16(),
        "XV": rn(B, H, NC, CS, F).bfloat16(),
        "last_eta": (eta_scale * torch.sigmoid(rn(B, H, NC, CS)) / 64).bfloat16(),
        "ttt_norm_weight": 1 + 0.02 * rn(1, H, 1, F),
        "ttt_norm_bias": 0.02 * rn(1, H, 1, F),
        "W1": 0.02 * rn(B, H, F, HID),
        "b1": torch.zeros(B, H, 1, HID),
        "W2": 0.02 * rn(B, H, HID, F),
        "b2": torch.zeros(B, H, 1, F),
    }
    if backward:
        d["grad_L_XQW_mini_batch"] = rn(B, H, NC, CS, F).bfloat16()
        d["grad_L_W1_last"] = 1e-3 * rn(B, H, F, HID)
        d["grad_L_b1_last"] = 1e-3 * rn(B, H, 1, HID)
        d["grad_L_W2_last"] = 1e-3 * rn(B, H, HID, F)
        d["grad_L_b2_last"] = 1e-3 * rn(B, H, 1, F)
    return d


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    """||x - ref||_2 / ||ref||_2, the parity measure of every gate."""
    x = x.detach().double().reshape(-1)
    ref = ref.detach().double().reshape(-1)
    den = ref.norm().item()
    return (x - ref).norm().item() / (den if den > 0 else 1.0)
