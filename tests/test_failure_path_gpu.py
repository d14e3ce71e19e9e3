"""Device-side failure handling without faulting the GPU: a bounded wait that nothing satisfies
runs out, the kernel reports code 3 through the status word and exits normally, and the very next
operator call works."""
import ctypes
import os
import subprocess
import sys

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


def test_operator_kernels_report_a_lost_load_and_the_context_survives():
    """The abort paths of the operator kernels themselves (one CTA per stream and cluster-sharded): a
    child process with a 5 ms wait limit launches each kernel with the test hook that withholds one
    mini-batch's loads; see lost_load_child.py."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TTT_B200_WAIT_LIMIT_MS="5", PYTHONPATH=root)
    res = subprocess.run([sys.executable, os.path.join(root, "tests", "lost_load_child.py")], env=env, cwd=root,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "LOST_LOAD_OK" in res.stdout
