"""Layer-side kernels around the operator (CUDA, `csrc/ttt_glue.cu`): the learning-rate gate that
produces `last_eta` and the LayerNorm that follows the operator's output, each fused with the change
between a model's token-major activations and the operator's head-major tensors.  The reference leaves
both to its callers (README.md:22-98); the statements they match are in `oracle/glue.py`.

    last_eta = eta_gate(logits, scale)                   # [B, T, H] bf16 -> [B, H, T // 64, 64] bf16
    d_logits = eta_gate_backward(logits, d_last_eta, scale)
    y = unpack_layernorm(out, gamma, beta, eps)          # [B, H, NC, 64, 64] bf16 -> [B, T, H * 64] bf16
    d_out, d_gamma, d_beta = pack_layernorm_backward(d_y, out, gamma, stats)
"""
import ctypes

import torch

from . import _lib


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _need(cond, msg):
    if not cond:
        raise ValueError(msg)


def _call(name, dev, *args):
    lib = _lib.lib()
    with torch.cuda.device(dev):
        rc = getattr(lib, name)(*args, _stream(dev))
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {lib.ttt_b200_last_error().decode()}")


def eta_gate(logits, scale):
    """last_eta[b, h, n, t] = scale * sigmoid(logits[b, n * 64 + t, h]).  `logits`: bf16 [B, T, H], the
    per-head output of the layer's learning-rate projection; `scale` = base learning rate x token weight
    of the mini-batch's last row / 64.  Returns bf16 [B, H, T // 64, 64], the operator's `last_eta`."""
    _need(logits.is_cuda and logits.dtype == torch.bfloat16 and logits.is_contiguous() and logits.dim() == 3,
          "logits must be a contiguous bf16 CUDA tensor [B, T, H]")
    B, T, H = logits.shape
    _need(T % 64 == 0, "T must be a multiple of 64")
    out = torch.empty(B, H, T // 64, 64, dtype=torch.bfloat16, device=logits.device)
    _call("ttt_b200_eta_gate", logits.device, logits.data_ptr(), out.data_ptr(), ctypes.c_float(scale), B, T, H)
    return out


def eta_gate_backward(logits, grad_last_eta, scale):
    """Gradient of `eta_gate` with respect to the logits: bf16 [B, T, H].  `grad_last_eta` is the
    operator's grad_L_last_eta, bf16 [B, H, NC, 64] or [B, H, NC, 64, 1]."""
    B, T, H = logits.shape
    _need(grad_last_eta.is_cuda and grad_last_eta.dtype == torch.bfloat16 and grad_last_eta.is_contiguous()
          and grad_last_eta.numel() == B * T * H and grad_last_eta.shape[:2] == (B, H),
          "grad_last_eta must be a contiguous bf16 CUDA tensor [B, H, T // 64, 64(, 1)]")
    out = torch.empty_like(logits)
    _call("ttt_b200_eta_gate_backward", logits.device, logits.data_ptr(), grad_last_eta.data_ptr(), out.data_ptr(),
          ctypes.c_float(scale), B, T, H)
    return out


def unpack_layernorm(out, gamma, beta, eps=1e-6, return_stats=False):
    """y[b, t, :] = gamma * LayerNorm(x[b, t, :]) + beta over the H * 64 features of a token, where
    x[b, t, h * 64 + f] = out[b, h, t // 64, t % 64, f].  `out`: the operator's Out, bf16 [B, H, NC, 64, 64];
    gamma, beta: fp32 [H * 64].  Returns bf16 [B, NC * 64, H * 64]; with `return_stats` also the per-token
    (mean, 1 / std), fp32 [B, NC * 64, 2], which `pack_layernorm_backward` takes."""
    _need(out.is_cuda and out.dtype == torch.bfloat16 and out.is_contiguous() and out.dim() == 5
          and out.shape[3] == 64 and out.shape[4] == 64, "out must be a contiguous bf16 CUDA tensor [B, H, NC, 64, 64]")
    B, H, NC = out.shape[:3]
    for v, n in ((gamma, "gamma"), (beta, "beta")):
        _need(v.is_cuda and v.dtype == torch.float32 and v.is_contiguous() and v.numel() == H * 64,
              f"{n} must be a contiguous fp32 CUDA tensor with H * 64 elements")
    y = torch.empty(B, NC * 64, H * 64, dtype=torch.bfloat16, device=out.device)
    stats = torch.empty(B, NC * 64, 2, dtype=torch.float32, device=out.device) if return_stats else None
    _call("ttt_b200_unpack_layernorm", out.device, out.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(),
          stats.data_ptr() if return_stats else None, ctypes.c_float(eps), B, NC * 64, H)
    return (y, stats) if return_stats else y


def pack_layernorm_backward(grad_y, out, gamma, stats):
    """Backward of `unpack_layernorm`: returns (grad_out, grad_gamma, grad_beta) with grad_out bf16
    [B, H, NC, 64, 64] (what `ttt_backward` takes as grad_L_XQW_mini_batch) and the parameter gradients fp32
    [H * 64].  `grad_y`: bf16 [B, NC * 64, H * 64]; `out`, `gamma`: as in the forward; `stats`: its second result."""
    B, H, NC = out.shape[:3]
    T = NC * 64
    _need(grad_y.is_cuda and grad_y.dtype == torch.bfloat16 and grad_y.is_contiguous()
          and tuple(grad_y.shape) == (B, T, H * 64), "grad_y must be a contiguous bf16 CUDA tensor [B, T, H * 64]")
    _need(out.dtype == torch.bfloat16 and out.is_contiguous(), "out must be contiguous bf16")
    _need(stats.dtype == torch.float32 and stats.is_contiguous() and tuple(stats.shape) == (B, T, 2),
          "stats must be the fp32 [B, T, 2] tensor the forward returned")
    _need(gamma.dtype == torch.float32 and gamma.is_contiguous() and gamma.numel() == H * 64, "gamma: fp32 [H * 64]")
    grad_out = torch.empty_like(out)
    g_gamma = torch.zeros(H * 64, dtype=torch.float32, device=out.device)
    g_beta = torch.zeros(H * 64, dtype=torch.float32, device=out.device)
    _call("ttt_b200_pack_layernorm_backward", out.device, grad_y.data_ptr(), out.data_ptr(), gamma.data_ptr(),
          stats.data_ptr(), grad_out.data_ptr(), g_gamma.data_ptr(), g_beta.data_ptr(), B, T, H)
    return grad_out, g_gamma, g_beta
