"""The backward entry point that allocates no device memory (ttt_b200_backward_noalloc).

Some hosts of the library pre-commit all of HBM to their own pools, or run loops in which an
allocation's implicit device synchronisation is unacceptable; they cannot hand the backward its
sixteen scratch tensors.  This entry point keeps the scratch in a fixed array inside the
library instead.  It must give the same gradients as the ordinary entry point, call after call
(the array is shared between calls and keeps the previous call's contents), and it must refuse
problems larger than the array.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes on its own in a fresh process as well.
"""
import ctypes

import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import _lib

TOL = 3e-2   # the gradient gate of the backward parity tests


def _noalloc_args(B, H, NC, cgs, n):
    a = _lib.BwdNoAllocArgs()
    a.B, a.H, a.NC, a.checkpoint_group_size, a.num_checkpoints, a.flags = B, H, NC, cgs, n, _lib.FLAG_SYNC
    return a


def test_oversize_problem_is_refused_before_any_cuda_call():
    lib = _lib.lib()
    # 4 * 8 * 8 = 256 slots > 128
    a = _noalloc_args(4, 8, 16, 8, 2)
    assert lib.ttt_b200_backward_noalloc(ctypes.byref(a), None) == 1
    assert b"TTT_B200_NOALLOC_MAX_SLOTS" in lib.ttt_b200_last_error()
    assert lib.ttt_b200_backward_noalloc(None, None) == 1
    b = _noalloc_args(1, 1, 4, 2, 3)          # wrong checkpoint count
    assert lib.ttt_b200_backward_noalloc(ctypes.byref(b), None) == 1
    assert _lib.NOALLOC_MAX_SLOTS == 128


@pytest.mark.gpu
def test_noalloc_backward_equals_ordinary_backward_twice_in_a_row():
    from ttt_tk_b200 import ttt_backward, take_status
    from ttt_tk_b200.buffers import alloc_backward_buffers, GRAD_NAMES, CHECKPOINT_NAMES
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    # calls in a row with different shapes and data: each sees its predecessor's leftovers.  The last case
    # fills the built-in scratch to its limit (2 * 8 * 8 = 128 slots, ragged last group), so the last slot
    # of every region is written and read.
    assert 2 * 8 * 8 == _lib.NOALLOC_MAX_SLOTS
    for (B, H, NC, cgs, seed) in [(2, 3, 5, 2, 21), (1, 4, 8, 4, 22), (2, 8, 9, 8, 23)]:
        d = orc.make_inputs(B, H, NC, seed=seed, backward=True)
        ck = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                             d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], cgs)
        n = orc.num_checkpoints(NC, cgs)
        t = {k: v.to(dev) for k, v in d.items()}
        t["last_eta"] = t["last_eta"].unsqueeze(-1).contiguous()
        ckd = {k: ck[k].to(dev).contiguous() for k in CHECKPOINT_NAMES}

        # ordinary entry point, caller-provided scratch
        scratch, want = alloc_backward_buffers(B, H, NC, cgs, dev, fill=float("nan"))
        out_fwd = torch.zeros_like(t["XQ"])
        # (one CTA per stream, which is what the entry point under test runs)
        ttt_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                     *[ckd[k] for k in CHECKPOINT_NAMES], out_fwd, *scratch,
                     t["grad_L_W1_last"], t["grad_L_b1_last"], t["grad_L_W2_last"], t["grad_L_b2_last"],
                     t["grad_L_XQW_mini_batch"], *[want[k] for k in GRAD_NAMES], cgs, cluster=1)
        torch.cuda.synchronize()
        assert take_status() == 0

        # the entry point under test, through the C ABI, no scratch passed
        _, got = alloc_backward_buffers(B, H, NC, cgs, dev, fill=float("nan"))
        a = _noalloc_args(B, H, NC, cgs, n)
        if seed == 22:
            a.flags = 0        # asynchronous call: nothing may be left in the status word afterwards
        src = dict(t)
        src.update(ckd)
        src.update(got)
        for name in _lib.BWD_NOALLOC_FIELDS:
            setattr(a, name, src[name].data_ptr())
        rc = lib.ttt_b200_backward_noalloc(ctypes.byref(a),
                                           ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        assert rc == 0, lib.ttt_b200_last_error()
        torch.cuda.synchronize()
        assert take_status() == 0
        # the same deterministic kernel ran on the same inputs; only the home of the scratch differs
        for k in GRAD_NAMES:
            assert torch.isfinite(got[k].float()).all(), k
            assert torch.equal(got[k], want[k]), f"{k} differs from the ordinary entry point"
        # and against the oracle, like every other backward test
        ref = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                               d["ttt_norm_bias"], ck["W1_checkpoints"], ck["b1_checkpoints"],
                               ck["W2_checkpoints"], ck["b2_checkpoints"], d["grad_L_W1_last"],
                               d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                               d["grad_L_XQW_mini_batch"], cgs)
        for k in GRAD_NAMES:
            assert orc.rel_l2(got[k].float().cpu(), ref[k]) <= TOL, k
