"""Token layout transforms either side of the operator (CUDA, `csrc/ttt_layout.cu`).

A model keeps activations token-major, `[B, T, H*64]`; `ttt_forward` / `ttt_backward` take
contiguous head-major `[B, H, NC, 64, 64]` tensors (the reference's requirement, README.md:98 of
the reference).  `pack_tokens` moves up to four tensors model -> operator in one launch,
`unpack_tokens` the other way.  Bit-exact with `x.view(B, T, H, 64).permute(0, 2, 1, 3)`.

    xq, xk, xv = pack_tokens(q, k, v)              # each [B, T, H*64] bf16 -> [B, H, T//64, 64, 64]
    (y,) = unpack_tokens(out)                      # [B, H, NC, 64, 64] -> [B, T, H*64]
"""
import ctypes

import torch

from . import _lib

_MAX = 4


def _check(ts, ndim_ok):
    if not 1 <= len(ts) <= _MAX:
        raise ValueError(f"1 to {_MAX} tensors per call")
    t0 = ts[0]
    for t in ts:
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("tensors must be contiguous bf16 CUDA tensors")
        if t.shape != t0.shape or t.device != t0.device:
            raise ValueError("tensors of one call must share shape and device")
        if t.dim() not in ndim_ok:
            raise ValueError(f"expected a tensor of rank {ndim_ok}, got shape {tuple(t.shape)}")


def _run(name, srcs, dsts, B, T, H):
    n = len(srcs)
    a_src = (ctypes.c_void_p * n)(*[t.data_ptr() for t in srcs])
    a_dst = (ctypes.c_void_p * n)(*[t.data_ptr() for t in dsts])
    with torch.cuda.device(srcs[0].device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = getattr(_lib.lib(), name)(a_src, a_dst, n, B, T, H, ctypes.c_void_p(stream))
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {_lib.lib().ttt_b200_last_error().decode()}")
    return dsts


def pack_tokens(*xs):
    """[B, T, H*64] (or [B, T, H, 64]) -> [B, H, T//64, 64, 64] for each tensor, one launch."""
    _check(xs, (3, 4))
    x = xs[0]
    B, T = x.shape[0], x.shape[1]
    F = x.shape[2] if x.dim() == 3 else x.shape[2] * x.shape[3]
    if F % 64 or T % 64 or (x.dim() == 4 and x.shape[3] != 64):
        raise ValueError("the feature dimension must be H*64 and T a multiple of 64")
    H = F // 64
    outs = [torch.empty(B, H, T // 64, 64, 64, dtype=x.dtype, device=x.device) for _ in xs]
    return _run("ttt_b200_pack_tokens", xs, outs, B, T, H)


def unpack_tokens(*ys):
    """[B, H, NC, 64, 64] -> [B, NC*64, H*64] for each tensor, one launch."""
    _check(ys, (5,))
    y = ys[0]
    B, H, NC = y.shape[:3]
    if y.shape[3] != 64 or y.shape[4] != 64:
        raise ValueError("expected [B, H, NC, 64, 64]")
    outs = [torch.empty(B, NC * 64, H * 64, dtype=y.dtype, device=y.device) for _ in ys]
    return _run("ttt_b200_unpack_tokens", ys, outs, B, NC * 64, H)
