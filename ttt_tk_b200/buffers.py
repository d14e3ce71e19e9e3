"""Allocation helpers for the caller-owned tensors of the operator API.

The operator allocates nothing: checkpoints, backward scratch and gradient outputs are the
caller's, with the shapes the reference's scripts use
(kernels/ttt/matching.py:170-173, kernels/ttt_backward/matching.py:406-435).
"""
import math

import torch

GRAD_NAMES = ["grad_L_ttt_norm_weight", "grad_L_ttt_norm_bias", "grad_L_W1_init", "grad_L_b1_init",
              "grad_L_W2_init", "grad_L_b2_init", "grad_L_last_eta", "grad_L_XQ", "grad_L_XK", "grad_L_XV"]
CHECKPOINT_NAMES = ["W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints"]


def alloc_checkpoints(B, H, NC, cgs, device="cuda"):
    """[W1, b1, W2, b2]_checkpoints for ceil(NC / cgs) states, fp32."""
    n = math.ceil(NC / cgs)
    return [torch.empty(B, H, n, *s, dtype=torch.float32, device=device)
            for s in ((64, 256), (1, 256), (256, 64), (1, 64))]


def alloc_backward_buffers(B, H, NC, cgs, device="cuda", fill=0.0):
    """(scratch, outputs): the sixteen `*_group` scratch tensors in the positional order of
    ttt_backward, and a dict of the ten gradient outputs (filled with `fill`; the kernel
    overwrites them)."""
    bf, f32 = torch.bfloat16, torch.float32
    z = lambda *s, dt=f32: torch.zeros(*s, dtype=dt, device=device)
    o = lambda *s, dt=f32: torch.full(s, fill, dtype=dt, device=device)
    g = cgs
    scratch = [z(B, H, g, 64, 256), z(B, H, g, 1, 256), z(B, H, g, 256, 64), z(B, H, g, 1, 64),
               z(B, H, g, 64, 64, dt=bf), z(B, H, g, 64, 1),
               z(B, H, g, 64, 256, dt=bf), z(B, H, g, 64, 256, dt=bf), z(B, H, g, 64, 256, dt=bf),
               z(B, H, g, 64, 256, dt=bf),
               z(B, H, g, 64, 64, dt=bf), z(B, H, g, 64, 256, dt=bf), z(B, H, g, 64, 64, dt=bf),
               z(B, H, g, 64, 64, dt=bf), z(B, H, g, 64, 64, dt=bf), z(B, H, g, 64, 1)]
    outs = {
        "grad_L_ttt_norm_weight": o(B, H, 1, 64), "grad_L_ttt_norm_bias": o(B, H, 1, 64),
        "grad_L_W1_init": o(B, H, 64, 256), "grad_L_b1_init": o(B, H, 1, 256),
        "grad_L_W2_init": o(B, H, 256, 64), "grad_L_b2_init": o(B, H, 1, 64),
        "grad_L_last_eta": o(B, H, NC, 64, 1, dt=bf),
        "grad_L_XQ": o(B, H, NC, 64, 64, dt=bf), "grad_L_XK": o(B, H, NC, 64, 64, dt=bf),
        "grad_L_XV": o(B, H, NC, 64, 64, dt=bf),
    }
    return scratch, outs
