"""Device-side failure handling without faulting the GPU: a bounded wait that nothing satisfies
runs out, the kernel reports code 3 through the status word and exits normally, and the very next
operator call works."""
import ctypes

import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import _lib, ttt_forward, take_status
from ttt_tk_b200.buffers import alloc_checkpoints

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_context_survives():
    lib = _lib.lib()
    waited = ctypes.c_ulonglong(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ttt_b200_wait_selftest(2000, ctypes.byref(waited), stream)      # 2 ms limit
    assert rc == 3, lib.ttt_b200_last_error()
    assert b"bounded wait" in lib.ttt_b200_last_error()
    assert 2e6 <= waited.value < 50e6, f"waited {waited.value} ns for a 2 ms limit"
    assert take_status() == 0            # the report was taken by the call itself
    # the context is alive: a normal forward right afterwards is correct
    d = orc.make_inputs(1, 2, 3, seed=0)
    t = {k: v.cuda() for k, v in d.items()}
    ck = alloc_checkpoints(1, 2, 3, 2)
    out = torch.empty_like(t["XQ"])
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                t["W1"], t["b1"], t["W2"], t["b2"], *ck, out, 2, sync=True)
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], 2)
    assert orc.rel_l2(out.float().cpu(), ref["Out"]) <= 1e-2


def test_wait_selftest_rejects_bad_limit():
    lib = _lib.lib()
    assert lib.ttt_b200_wait_selftest(0, None, None) == 1
