"""CPU statements (test infrastructure: only tests, the smoke check and bench.py's checker may import
this) of the layer-side kernels around the operator.  The reference contains no code for them: its
callers pass `last_eta` and post-process `XQW_batch` themselves (README.md:22-98 of the reference), and
its scripts draw `last_eta` directly (kernels/ttt/matching.py:158).  What is stated here is therefore
the definition the CUDA kernels are held to, in plain torch:

  eta gate      last_eta = scale * sigmoid(logits), moved from token-major [B, T, H] to the operator's
                head-major [B, H, T // 64, 64]; computed in fp32 from the bf16 logits, rounded to bf16
  output norm   torch.nn.functional.layer_norm over the H * 64 features of a token (biased variance, eps
                inside the square root, fp32 statistics), on the operator's Out moved to [B, T, H * 64]
"""
import torch
import torch.nn.functional as F


def eta_gate(logits, scale):
    B, T, H = logits.shape
    e = scale * torch.sigmoid(logits.float())
    return e.permute(0, 2, 1).reshape(B, H, T // 64, 64).contiguous().bfloat16()


def eta_gate_backward(logits, grad_last_eta, scale):
    B, T, H = logits.shape
    s = torch.sigmoid(logits.float())
    g = grad_last_eta.float().reshape(B, H, T).permute(0, 2, 1)
    return (g * scale * s * (1 - s)).contiguous().bfloat16()


def unpack_layernorm(out, gamma, beta, eps=1e-6):
    B, H, NC = out.shape[:3]
    x = out.float().reshape(B, H, NC * 64, 64).permute(0, 2, 1, 3).reshape(B, NC * 64, H * 64)
    return F.layer_norm(x, (H * 64,), gamma.float().reshape(-1), beta.float().reshape(-1), eps).bfloat16()


def pack_layernorm_backward(grad_y, out, gamma, beta, eps=1e-6):
    """(grad_out [B, H, NC, 64, 64] bf16, grad_gamma, grad_beta fp32 [H * 64]) by autograd through the statement
    above (in fp32, without the final bf16 rounding of y)."""
    B, H, NC = out.shape[:3]
    x = out.float().clone().requires_grad_(True)
    g = gamma.float().reshape(-1).clone().requires_grad_(True)
    bb = beta.float().reshape(-1).clone().requires_grad_(True)
    xt = x.reshape(B, H, NC * 64, 64).permute(0, 2, 1, 3).reshape(B, NC * 64, H * 64)
    y = F.layer_norm(xt, (H * 64,), g, bb, eps)
    y.backward(grad_y.float())
    return x.grad.bfloat16(), g.grad, bb.grad
