"""Host-side mirror of the reference's operator interface.

`ttt_forward` and `ttt_backward` take the same positional tensors, in the same order, as the
functions the reference's extension module exports (test_time_training.cpp:24-104;
launchers kernels/ttt/ttt.cu:594-611 and kernels/ttt_backward/ttt.cu:1451-1495) and return
the `Out` tensor like they do.  They validate like the reference's TORCH_CHECKs
(kernels/ttt/ttt.cu:621-630, kernels/ttt_backward/ttt.cu:1507-1760) -- on every call, and a
little more strictly -- raising RuntimeError, then hand raw device pointers to the C ABI
(include/ttt_mlp_b200.h).  torch is used only for device memory and the current stream.

Differences from the reference, all documented in the header:
  * calls are stream-ordered and do not synchronise;
  * backward overwrites grad_L_XQ/XK/XV/last_eta (the reference accumulates into zero-filled
    buffers) and never writes `Out`.
"""
import ctypes
import math

import torch

from . import _lib

CS, F, HID = 64, 64, 256


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _chk_tensor(t, name, dtype, shape, device):
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.device == device, f"{name} must be on {device}")
    _check(t.dtype == dtype, f"{name} must have dtype {dtype}, got {t.dtype}")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    if shape is not None:
        _check(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def _dims(XQ, checkpoint_group_size, W1_checkpoints):
    _check(isinstance(XQ, torch.Tensor) and XQ.dim() == 5, "XQ must be 5-D [B, H, NC, 64, 64]")
    B, H, NC, cs, f = XQ.shape
    _check(f == F, "head dimension must be 64")
    _check(cs == CS, "mini-batch size must be 64")
    _check(NC >= 1, "need at least one mini-batch")
    cgs = int(checkpoint_group_size)
    _check(cgs >= 1, "checkpoint_group_size must be >= 1")
    n = math.ceil(NC / cgs)
    _check(isinstance(W1_checkpoints, torch.Tensor) and W1_checkpoints.dim() == 5
           and W1_checkpoints.shape[2] == n,
           f"checkpoint tensors must hold ceil(NC / checkpoint_group_size) = {n} states")
    return B, H, NC, cgs, n


def _chk_eta(t, name, B, H, NC, device):
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    ok = tuple(t.shape) in ((B, H, NC, CS), (B, H, NC, CS, 1))
    _check(ok, f"{name} must have shape [B, H, NC, 64] or [B, H, NC, 64, 1], got {tuple(t.shape)}")
    _chk_tensor(t, name, torch.bfloat16, None, device)


def _raise(lib, rc, what):
    msg = lib.ttt_b200_last_error().decode()
    raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _flags(sync, cluster, lost_load=False):
    """Flag word of the C ABI: bit 0 synchronise, bit 1 the failure-path test hook, bits 8..11 the number
    of CTAs (1, 2 or 4) that share one stream (0 / None: chosen from B*H and the SM count)."""
    cluster = 0 if cluster is None else int(cluster)
    _check(cluster in (0, 1, 2, 4), "cluster must be None, 1, 2 or 4")
    return (_lib.FLAG_SYNC if sync else 0) | (_lib.FLAG_TEST_LOST_LOAD if lost_load else 0) | (cluster << 8)


def ttt_forward(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W2, b2,
                W1_checkpoints, b1_checkpoints, W2_checkpoints, b2_checkpoints, Out,
                checkpoint_group_size, *, final_state=None, sync=False, cluster=None, _lost_load=False):
    """TTT-MLP forward over the whole sequence; writes `Out` and the state checkpoints.

    Positional arguments: exactly the reference's (kernels/ttt/ttt.cu:594-611).
    Keyword-only extras (not in the reference): `final_state` = (W1, b1, W2, b2) fp32 tensors
    that receive the state after the last mini-batch; `sync` blocks until the result is ready
    and raises on a device-side failure; `cluster` forces how many CTAs share one (batch, head)
    stream (1, 2 or 4; default: chosen from B*H and the GPU's SM count).
    """
    lib = _lib.lib()
    B, H, NC, cgs, n = _dims(XQ, checkpoint_group_size, W1_checkpoints)
    dev = XQ.device
    bf, f32 = torch.bfloat16, torch.float32
    tok = (B, H, NC, CS, F)
    _chk_tensor(XQ, "XQ", bf, tok, dev)
    _chk_tensor(XK, "XK", bf, tok, dev)
    _chk_tensor(XV, "XV", bf, tok, dev)
    _chk_eta(last_eta, "last_eta", B, H, NC, dev)
    _chk_tensor(ttt_norm_weight, "ttt_norm_weight", f32, (1, H, 1, F), dev)
    _chk_tensor(ttt_norm_bias, "ttt_norm_bias", f32, (1, H, 1, F), dev)
    _chk_tensor(W1, "W1", f32, (B, H, F, HID), dev)
    _chk_tensor(b1, "b1", f32, (B, H, 1, HID), dev)
    _chk_tensor(W2, "W2", f32, (B, H, HID, F), dev)
    _chk_tensor(b2, "b2", f32, (B, H, 1, F), dev)
    _chk_tensor(W1_checkpoints, "W1_checkpoints", f32, (B, H, n, F, HID), dev)
    _chk_tensor(b1_checkpoints, "b1_checkpoints", f32, (B, H, n, 1, HID), dev)
    _chk_tensor(W2_checkpoints, "W2_checkpoints", f32, (B, H, n, HID, F), dev)
    _chk_tensor(b2_checkpoints, "b2_checkpoints", f32, (B, H, n, 1, F), dev)
    _chk_tensor(Out, "Out", bf, tok, dev)

    a = _lib.FwdArgs()
    vals = [XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W2, b2,
            W1_checkpoints, b1_checkpoints, W2_checkpoints, b2_checkpoints, Out]
    for name, t in zip(_lib.FWD_FIELDS, vals):
        setattr(a, name, t.data_ptr())
    if final_state is not None:
        _check(len(final_state) == 4, "final_state must be (W1, b1, W2, b2)")
        shapes = [(B, H, F, HID), (B, H, 1, HID), (B, H, HID, F), (B, H, 1, F)]
        for name, t, shp in zip(_lib.FWD_TAIL, final_state, shapes):
            _chk_tensor(t, name, f32, shp, dev)
            setattr(a, name, t.data_ptr())
    a.B, a.H, a.NC, a.checkpoint_group_size, a.num_checkpoints = B, H, NC, cgs, n
    a.flags = _flags(sync, cluster, _lost_load)
    with torch.cuda.device(dev):
        rc = lib.ttt_b200_forward(ctypes.byref(a), _stream_ptr(dev))
    if rc != 0:
        _raise(lib, rc, "ttt_forward")
    return Out


def ttt_linear_forward(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1,
                       W1_checkpoints, b1_checkpoints, Out, checkpoint_group_size, *,
                       final_state=None, sync=False, _lost_load=False):
    """TTT-Linear forward over the whole sequence: `ttt_forward` with the inner model reduced to one linear
    layer (W1 [B,H,64,64], b1 [B,H,1,64]; no W2 / b2); writes `Out` and the state checkpoints.  The reference
    has no counterpart (it ships the MLP operator only).  `final_state` = (W1, b1) fp32 tensors that receive
    the state after the last mini-batch."""
    lib = _lib.lib()
    B, H, NC, cgs, n = _dims(XQ, checkpoint_group_size, W1_checkpoints)
    dev = XQ.device
    bf, f32 = torch.bfloat16, torch.float32
    tok = (B, H, NC, CS, F)
    _chk_tensor(XQ, "XQ", bf, tok, dev)
    _chk_tensor(XK, "XK", bf, tok, dev)
    _chk_tensor(XV, "XV", bf, tok, dev)
    _chk_eta(last_eta, "last_eta", B, H, NC, dev)
    _chk_tensor(ttt_norm_weight, "ttt_norm_weight", f32, (1, H, 1, F), dev)
    _chk_tensor(ttt_norm_bias, "ttt_norm_bias", f32, (1, H, 1, F), dev)
    _chk_tensor(W1, "W1", f32, (B, H, F, F), dev)
    _chk_tensor(b1, "b1", f32, (B, H, 1, F), dev)
    _chk_tensor(W1_checkpoints, "W1_checkpoints", f32, (B, H, n, F, F), dev)
    _chk_tensor(b1_checkpoints, "b1_checkpoints", f32, (B, H, n, 1, F), dev)
    _chk_tensor(Out, "Out", bf, tok, dev)
    a = _lib.LinearFwdArgs()
    vals = [XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1, b1, W1_checkpoints, b1_checkpoints, Out]
    for name, t in zip(_lib.LINEAR_FWD_FIELDS, vals):
        setattr(a, name, t.data_ptr())
    if final_state is not None:
        _check(len(final_state) == 2, "final_state must be (W1, b1)")
        for name, t, shp in zip(_lib.LINEAR_FWD_TAIL, final_state, [(B, H, F, F), (B, H, 1, F)]):
            _chk_tensor(t, name, f32, shp, dev)
            setattr(a, name, t.data_ptr())
    a.B, a.H, a.NC, a.checkpoint_group_size, a.num_checkpoints = B, H, NC, cgs, n
    a.flags = _flags(sync, None, _lost_load)
    with torch.cuda.device(dev):
        rc = lib.ttt_b200_linear_forward(ctypes.byref(a), _stream_ptr(dev))
    if rc != 0:
        _raise(lib, rc, "ttt_linear_forward")
    return Out


def ttt_linear_backward(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1_checkpoints, b1_checkpoints,
                        grad_L_W1_last, grad_L_b1_last, grad_L_XQW_mini_batch, grad_L_ttt_norm_weight,
                        grad_L_ttt_norm_bias, grad_L_W1_init, grad_L_b1_init, grad_L_last_eta, grad_L_XQ, grad_L_XK,
                        grad_L_XV, checkpoint_group_size, *, scratch=None, sync=False, _lost_load=False):
    """TTT-Linear backward: gradients of `ttt_linear_forward` from its checkpoints.  Outputs (overwritten):
    norm gradients per batch element fp32 [B,H,1,64], dL/d(initial state) fp32 [B,H,64,64] / [B,H,1,64],
    grad_L_last_eta bf16 [B,H,NC,64] (or [..., 64, 1]), grad_L_XQ / XK / XV bf16 [B,H,NC,64,64].  `scratch`: a
    uint8 CUDA tensor of at least `linear_backward_scratch_bytes(B, H, checkpoint_group_size)` bytes (allocated
    here when not given).  The reference has no counterpart."""
    lib = _lib.lib()
    B, H, NC, cgs, n = _dims(XQ, checkpoint_group_size, W1_checkpoints)
    dev = XQ.device
    bf, f32 = torch.bfloat16, torch.float32
    tok = (B, H, NC, CS, F)
    for t, name in ((XQ, "XQ"), (XK, "XK"), (XV, "XV"), (grad_L_XQW_mini_batch, "grad_L_XQW_mini_batch"),
                    (grad_L_XQ, "grad_L_XQ"), (grad_L_XK, "grad_L_XK"), (grad_L_XV, "grad_L_XV")):
        _chk_tensor(t, name, bf, tok, dev)
    _chk_eta(last_eta, "last_eta", B, H, NC, dev)
    _chk_eta(grad_L_last_eta, "grad_L_last_eta", B, H, NC, dev)
    _chk_tensor(ttt_norm_weight, "ttt_norm_weight", f32, (1, H, 1, F), dev)
    _chk_tensor(ttt_norm_bias, "ttt_norm_bias", f32, (1, H, 1, F), dev)
    _chk_tensor(W1_checkpoints, "W1_checkpoints", f32, (B, H, n, F, F), dev)
    _chk_tensor(b1_checkpoints, "b1_checkpoints", f32, (B, H, n, 1, F), dev)
    _chk_tensor(grad_L_W1_last, "grad_L_W1_last", f32, (B, H, F, F), dev)
    _chk_tensor(grad_L_b1_last, "grad_L_b1_last", f32, (B, H, 1, F), dev)
    _chk_tensor(grad_L_ttt_norm_weight, "grad_L_ttt_norm_weight", f32, (B, H, 1, F), dev)
    _chk_tensor(grad_L_ttt_norm_bias, "grad_L_ttt_norm_bias", f32, (B, H, 1, F), dev)
    _chk_tensor(grad_L_W1_init, "grad_L_W1_init", f32, (B, H, F, F), dev)
    _chk_tensor(grad_L_b1_init, "grad_L_b1_init", f32, (B, H, 1, F), dev)
    need = linear_backward_scratch_bytes(B, H, cgs)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    _check(isinstance(scratch, torch.Tensor) and scratch.is_cuda and scratch.device == dev and scratch.is_contiguous()
           and scratch.dtype == torch.uint8 and scratch.numel() >= need,
           f"scratch must be a contiguous uint8 CUDA tensor of at least {need} bytes")
    a = _lib.LinearBwdArgs()
    vals = [XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias, W1_checkpoints, b1_checkpoints, grad_L_W1_last,
            grad_L_b1_last, grad_L_XQW_mini_batch, scratch, grad_L_ttt_norm_weight, grad_L_ttt_norm_bias, grad_L_W1_init,
            grad_L_b1_init, grad_L_last_eta, grad_L_XQ, grad_L_XK, grad_L_XV]
    for name, t in zip(_lib.LINEAR_BWD_FIELDS, vals):
        setattr(a, name, t.data_ptr())
    a.B, a.H, a.NC, a.checkpoint_group_size, a.num_checkpoints = B, H, NC, cgs, n
    a.flags = _flags(sync, None, _lost_load)
    a.scratch_bytes = scratch.numel()
    with torch.cuda.device(dev):
        rc = lib.ttt_b200_linear_backward(ctypes.byref(a), _stream_ptr(dev))
    if rc != 0:
        _raise(lib, rc, "ttt_linear_backward")


def linear_backward_scratch_bytes(B, H, checkpoint_group_size):
    """Bytes of scratch `ttt_linear_backward` needs."""
    return int(_lib.lib().ttt_b200_linear_backward_scratch_bytes(int(B), int(H), int(checkpoint_group_size)))


def ttt_backward(XQ, XK, XV, last_eta, ttt_norm_weight, ttt_norm_bias,
                 W1_checkpoints, b1_checkpoints, W2_checkpoints, b2_checkpoints, Out,
                 W1_init_group, b1_init_group, W2_init_group, b2_init_group,
                 x_hat_ln_group, std_ln_group, X2_group, Z1_group, Z1_bar_group, X2_bar_group,
                 grad_l_wrt_Z2_group, grad_l_wrt_Z1_group, x_hat_fused_group, grad_x_hat_fused_group,
                 grad_output_fused_group, std_fused_group,
                 grad_L_W1_last, grad_L_b1_last, grad_L_W2_last, grad_L_b2_last, grad_L_XQW_mini_batch,
                 grad_L_ttt_norm_weight, grad_L_ttt_norm_bias, grad_L_W1_init, grad_L_b1_init,
                 grad_L_W2_init, grad_L_b2_init, grad_L_last_eta, grad_L_XQ, grad_L_XK, grad_L_XV,
                 checkpoint_group_size, *, sync=False, cluster=None, _lost_load=False):
    """TTT-MLP backward with per-checkpoint-group rematerialisation.

    Positional arguments: exactly the reference's 42 tensors + int
    (kernels/ttt_backward/ttt.cu:1451-1495).  grad_L_ttt_norm_weight / bias hold one row per
    batch element ([B, H, 1, 64]); the caller sums over dim 0 as with the reference
    (kernels/ttt_backward/matching.py:522-523).
    """
    lib = _lib.lib()
    B, H, NC, cgs, n = _dims(XQ, checkpoint_group_size, W1_checkpoints)
    dev = XQ.device
    bf, f32 = torch.bfloat16, torch.float32
    tok = (B, H, NC, CS, F)
    g = cgs
    spec = {
        "XQ": (bf, tok), "XK": (bf, tok), "XV": (bf, tok),
        "ttt_norm_weight": (f32, (1, H, 1, F)), "ttt_norm_bias": (f32, (1, H, 1, F)),
        "W1_checkpoints": (f32, (B, H, n, F, HID)), "b1_checkpoints": (f32, (B, H, n, 1, HID)),
        "W2_checkpoints": (f32, (B, H, n, HID, F)), "b2_checkpoints": (f32, (B, H, n, 1, F)),
        "Out": (bf, tok),
        "W1_init_group": (f32, (B, H, g, F, HID)), "b1_init_group": (f32, (B, H, g, 1, HID)),
        "W2_init_group": (f32, (B, H, g, HID, F)), "b2_init_group": (f32, (B, H, g, 1, F)),
        "x_hat_ln_group": (bf, (B, H, g, CS, F)), "std_ln_group": (f32, (B, H, g, CS, 1)),
        "X2_group": (bf, (B, H, g, CS, HID)), "Z1_group": (bf, (B, H, g, CS, HID)),
        "Z1_bar_group": (bf, (B, H, g, CS, HID)), "X2_bar_group": (bf, (B, H, g, CS, HID)),
        "grad_l_wrt_Z2_group": (bf, (B, H, g, CS, F)), "grad_l_wrt_Z1_group": (bf, (B, H, g, CS, HID)),
        "x_hat_fused_group": (bf, (B, H, g, CS, F)), "grad_x_hat_fused_group": (bf, (B, H, g, CS, F)),
        "grad_output_fused_group": (bf, (B, H, g, CS, F)), "std_fused_group": (f32, (B, H, g, CS, 1)),
        "grad_L_W1_last": (f32, (B, H, F, HID)), "grad_L_b1_last": (f32, (B, H, 1, HID)),
        "grad_L_W2_last": (f32, (B, H, HID, F)), "grad_L_b2_last": (f32, (B, H, 1, F)),
        "grad_L_XQW_mini_batch": (bf, tok),
        "grad_L_ttt_norm_weight": (f32, (B, H, 1, F)), "grad_L_ttt_norm_bias": (f32, (B, H, 1, F)),
        "grad_L_W1_init": (f32, (B, H, F, HID)), "grad_L_b1_init": (f32, (B, H, 1, HID)),
        "grad_L_W2_init": (f32, (B, H, HID, F)), "grad_L_b2_init": (f32, (B, H, 1, F)),
        "grad_L_XQ": (bf, tok), "grad_L_XK": (bf, tok), "grad_L_XV": (bf, tok),
    }
    loc = locals()
    a = _lib.BwdArgs()
    for name in _lib.BWD_FIELDS:
        t = loc[name]
        if name in ("last_eta", "grad_L_last_eta"):
            _chk_eta(t, name, B, H, NC, dev)
        else:
            dt, shp = spec[name]
            _chk_tensor(t, name, dt, shp, dev)
        setattr(a, name, t.data_ptr())
    a.B, a.H, a.NC, a.checkpoint_group_size, a.num_checkpoints = B, H, NC, cgs, n
    a.flags = _flags(sync, cluster, _lost_load)
    with torch.cuda.device(dev):
        rc = lib.ttt_b200_backward(ctypes.byref(a), _stream_ptr(dev))
    if rc != 0:
        _raise(lib, rc, "ttt_backward")
    return Out


def take_status():
    """0, or 3 if a kernel of this process gave up on a bounded wait since the last take."""
    return _lib.lib().ttt_b200_take_status()
