"""`torch.autograd.Function` around the operator pair, with the buffer handling the raw API leaves
to its callers (the reference ships only the two functions, README.md:22-96): checkpoints and
scratch are allocated once per shape and reused, the per-batch norm-gradient rows are summed, and
the state after the last mini-batch is returned so that sequences can be processed in chunks.
"""
import math

import torch

from .buffers import GRAD_NAMES, alloc_backward_buffers, alloc_checkpoints
from .ops import ttt_backward, ttt_forward

# One scratch set per (shape, device, CUDA stream): backward passes on the same stream are ordered and may
# share it (its contents mean nothing between calls); passes on different streams could overlap on the
# GPU and get their own.
_scratch_cache = {}


def _scratch(B, H, NC, cgs, device):
    key = (B, H, cgs, str(device), torch.cuda.current_stream(device).cuda_stream)
    if key not in _scratch_cache:
        _scratch_cache[key] = alloc_backward_buffers(B, H, 1, cgs, device)[0]
    return _scratch_cache[key]


class TTTMLPFunction(torch.autograd.Function):
    """(XQW, W1_last, b1_last, W2_last, b2_last) = f(XQ, XK, XV, last_eta, norm_weight, norm_bias,
    W1, b1, W2, b2, checkpoint_group_size).  Tensors as in `ttt_forward`."""

    @staticmethod
    def forward(ctx, XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W2, b2, checkpoint_group_size):
        B, H, NC = XQ.shape[:3]
        cgs = int(checkpoint_group_size)
        dev = XQ.device
        args = [t.contiguous() for t in (XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W2, b2)]
        ck = alloc_checkpoints(B, H, NC, cgs, dev)
        out = torch.empty_like(args[0])
        final = tuple(torch.empty_like(t) for t in args[6:10])
        ttt_forward(*args, *ck, out, cgs, final_state=final)
        ctx.save_for_backward(*args[:6], *ck, out)
        ctx.cgs = cgs
        ctx.eta_shape = last_eta.shape
        return (out,) + final

    @staticmethod
    def backward(ctx, g_out, g_W1, g_b1, g_W2, g_b2):
        saved = ctx.saved_tensors
        XQ, XK, XV, last_eta, gamma, beta = saved[:6]
        ck, out = saved[6:10], saved[10]
        B, H, NC = XQ.shape[:3]
        cgs, dev = ctx.cgs, XQ.device
        zeros = lambda ref, g: torch.zeros_like(ref) if g is None else g.contiguous().to(torch.float32)
        g_W1 = zeros(ck[0][:, :, 0], g_W1)
        g_b1 = zeros(ck[1][:, :, 0], g_b1)
        g_W2 = zeros(ck[2][:, :, 0], g_W2)
        g_b2 = zeros(ck[3][:, :, 0], g_b2)
        g_out = torch.zeros_like(XQ) if g_out is None else g_out.contiguous().to(torch.bfloat16)
        scratch = _scratch(B, H, NC, cgs, dev)
        bf, f32 = torch.bfloat16, torch.float32
        o = {
            "grad_L_ttt_norm_weight": torch.empty(B, H, 1, 64, dtype=f32, device=dev),
            "grad_L_ttt_norm_bias": torch.empty(B, H, 1, 64, dtype=f32, device=dev),
            "grad_L_W1_init": torch.empty(B, H, 64, 256, dtype=f32, device=dev),
            "grad_L_b1_init": torch.empty(B, H, 1, 256, dtype=f32, device=dev),
            "grad_L_W2_init": torch.empty(B, H, 256, 64, dtype=f32, device=dev),
            "grad_L_b2_init": torch.empty(B, H, 1, 64, dtype=f32, device=dev),
            "grad_L_last_eta": torch.empty(B, H, NC, 64, 1, dtype=bf, device=dev),
            "grad_L_XQ": torch.empty_like(XQ), "grad_L_XK": torch.empty_like(XQ), "grad_L_XV": torch.empty_like(XQ),
        }
        eta5 = last_eta if last_eta.dim() == 5 else last_eta.unsqueeze(-1)
        ttt_backward(XQ, XK, XV, eta5.contiguous(), gamma, beta, *ck, out, *scratch,
                     g_W1, g_b1, g_W2, g_b2, g_out, *[o[k] for k in GRAD_NAMES], cgs)
        d_gamma = o["grad_L_ttt_norm_weight"].sum(dim=0, keepdim=True)
        d_beta = o["grad_L_ttt_norm_bias"].sum(dim=0, keepdim=True)
        d_eta = o["grad_L_last_eta"].reshape(ctx.eta_shape)
        return (o["grad_L_XQ"], o["grad_L_XK"], o["grad_L_XV"], d_eta, d_gamma, d_beta,
                o["grad_L_W1_init"], o["grad_L_b1_init"], o["grad_L_W2_init"], o["grad_L_b2_init"], None)


def ttt_mlp(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W2, b2, checkpoint_group_size=None):
    """Differentiable TTT-MLP layer core.  Returns (XQW, (W1, b1, W2, b2) after the last mini-batch)."""
    NC = XQ.shape[2]
    if checkpoint_group_size is None:
        checkpoint_group_size = max(1, int(math.sqrt(NC)))
    r = TTTMLPFunction.apply(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W2, b2,
                             checkpoint_group_size)
    return r[0], tuple(r[1:])


_linear_scratch_cache = {}


def _linear_scratch(B, H, cgs, device):
    from .ops import linear_backward_scratch_bytes
    key = (B, H, cgs, str(device), torch.cuda.current_stream(device).cuda_stream)
    if key not in _linear_scratch_cache:
        _linear_scratch_cache[key] = torch.empty(linear_backward_scratch_bytes(B, H, cgs), dtype=torch.uint8,
                                                 device=device)
    return _linear_scratch_cache[key]


class TTTLinearFunction(torch.autograd.Function):
    """(XQW, W1_last, b1_last) = f(XQ, XK, XV, last_eta, norm_weight, norm_bias, W1, b1, checkpoint_group_size):
    the TTT-Linear operator pair (`ttt_linear_forward` / `ttt_linear_backward`)."""

    @staticmethod
    def forward(ctx, XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, checkpoint_group_size):
        from .ops import ttt_linear_forward
        B, H, NC = XQ.shape[:3]
        cgs = int(checkpoint_group_size)
        dev = XQ.device
        args = [t.contiguous() for t in (XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1)]
        n = math.ceil(NC / cgs)
        ck = (torch.empty(B, H, n, 64, 64, dtype=torch.float32, device=dev),
              torch.empty(B, H, n, 1, 64, dtype=torch.float32, device=dev))
        out = torch.empty_like(args[0])
        final = (torch.empty_like(args[6]), torch.empty_like(args[7]))
        ttt_linear_forward(*args, *ck, out, cgs, final_state=final)
        ctx.save_for_backward(*args[:6], *ck)
        ctx.cgs = cgs
        ctx.eta_shape = last_eta.shape
        return (out,) + final

    @staticmethod
    def backward(ctx, g_out, g_W1, g_b1):
        from .ops import ttt_linear_backward
        XQ, XK, XV, last_eta, gamma, beta, Wc, bc = ctx.saved_tensors
        B, H, NC = XQ.shape[:3]
        cgs, dev = ctx.cgs, XQ.device
        f32 = torch.float32
        g_W1 = torch.zeros(B, H, 64, 64, dtype=f32, device=dev) if g_W1 is None else g_W1.contiguous().to(f32)
        g_b1 = torch.zeros(B, H, 1, 64, dtype=f32, device=dev) if g_b1 is None else g_b1.contiguous().to(f32)
        g_out = torch.zeros_like(XQ) if g_out is None else g_out.contiguous().to(torch.bfloat16)
        d_gamma = torch.empty(B, H, 1, 64, dtype=f32, device=dev)
        d_beta = torch.empty(B, H, 1, 64, dtype=f32, device=dev)
        d_W1 = torch.empty(B, H, 64, 64, dtype=f32, device=dev)
        d_b1 = torch.empty(B, H, 1, 64, dtype=f32, device=dev)
        d_eta = torch.empty(B, H, NC, 64, dtype=torch.bfloat16, device=dev)
        dq, dk, dv = torch.empty_like(XQ), torch.empty_like(XQ), torch.empty_like(XQ)
        eta4 = last_eta.reshape(B, H, NC, 64)
        ttt_linear_backward(XQ, XK, XV, eta4, gamma, beta, Wc, bc, g_W1, g_b1, g_out, d_gamma, d_beta, d_W1, d_b1, d_eta,
                            dq, dk, dv, cgs, scratch=_linear_scratch(B, H, cgs, dev))
        return (dq, dk, dv, d_eta.reshape(ctx.eta_shape), d_gamma.sum(dim=0, keepdim=True),
                d_beta.sum(dim=0, keepdim=True), d_W1, d_b1, None)


def ttt_linear(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, checkpoint_group_size=None):
    """Differentiable TTT-Linear layer core.  Returns (XQW, (W1, b1) after the last mini-batch)."""
    NC = XQ.shape[2]
    if checkpoint_group_size is None:
        checkpoint_group_size = max(1, int(math.sqrt(NC)))
    r = TTTLinearFunction.apply(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, checkpoint_group_size)
    return r[0], tuple(r[1:])
