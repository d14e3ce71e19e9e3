"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset is involved in this path: the reference measures on random
tensors too, kernels/ttt_backward/matching.py:366-404).

XQ/XK/XV ~ N(0,1) rounded to bf16; last_eta = eta_scale * sigmoid(N(0,1)) / 64 (bf16);
norm weight 1 + 0.02 N(0,1), bias 0.02 N(0,1); W1, W2 ~ 0.02 N(0,1), b1 = b2 = 0 (fp32);
with `backward`: grad_L_XQW ~ N(0,1) bf16, upstream state gradients ~ 1e-3 N(0,1) fp32.
Drawn on the CPU generator in a fixed order, so every machine and every rank sees the same
data for the same seed.
"""
import torch


def make_inputs(B, H, NC, seed=0, eta_scale=0.1, backward=False):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)
    d = {
        "XQ": rn(B, H, NC, 64, 64).bfloat16(),
        "XK": rn(B, H, NC, 64, 64).bfloat16(),
        "XV": rn(B, H, NC, 64, 64).bfloat16(),
        "last_eta": (eta_scale * torch.sigmoid(rn(B, H, NC, 64)) / 64).bfloat16(),
        "ttt_norm_weight": 1 + 0.02 * rn(1, H, 1, 64),
        "ttt_norm_bias": 0.02 * rn(1, H, 1, 64),
        "W1": 0.02 * rn(B, H, 64, 256),
        "b1": torch.zeros(B, H, 1, 256),
        "W2": 0.02 * rn(B, H, 256, 64),
        "b2": torch.zeros(B, H, 1, 64),
    }
    if backward:
        d["grad_L_XQW_mini_batch"] = rn(B, H, NC, 64, 64).bfloat16()
        d["grad_L_W1_last"] = 1e-3 * rn(B, H, 64, 256)
        d["grad_L_b1_last"] = 1e-3 * rn(B, H, 1, 256)
        d["grad_L_W2_last"] = 1e-3 * rn(B, H, 256, 64)
        d["grad_L_b2_last"] = 1e-3 * rn(B, H, 1, 64)
    return d
