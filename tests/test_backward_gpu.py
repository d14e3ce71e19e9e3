"""Parity of the sm_100a backward with the CPU oracle, through the C ABI.

Gate: relative L2 <= 3e-2 for every gradient, against the fp32 oracle run on the same
bf16-rounded inputs and the same checkpoints."""
import os

import numpy as np
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, ttt_backward, take_status
from ttt_tk_b200.buffers import alloc_backward_buffers, GRAD_NAMES

pytestmark = pytest.mark.gpu
TOL = 3e-2
GRADS = GRAD_NAMES
CK = ["W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints"]


def run_backward(d, ck, cgs):
    dev = "cuda"
    B, H, NC = d["XQ"].shape[:3]
    t = {k: v.to(dev) for k, v in d.items()}
    ckd = [ck[k].to(dev).float().contiguous() for k in CK]
    scratch, outs = alloc_backward_buffers(B, H, NC, cgs, fill=float("nan"))
    out_fwd = torch.zeros_like(t["XQ"])
    sentinel = out_fwd.clone()
    ret = ttt_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"].unsqueeze(-1).contiguous(),
                       t["ttt_norm_weight"], t["ttt_norm_bias"], *ckd, out_fwd, *scratch,
                       t["grad_L_W1_last"], t["grad_L_b1_last"], t["grad_L_W2_last"], t["grad_L_b2_last"],
                       t["grad_L_XQW_mini_batch"], *[outs[k] for k in GRADS], cgs)
    torch.cuda.synchronize()
    assert take_status() == 0
    assert ret is out_fwd and torch.equal(out_fwd, sentinel), "backward must not touch Out"
    return {k: v.float().cpu() for k, v in outs.items()}


def oracle_backward(d, ck, cgs):
    return orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                            ck["W1_checkpoints"], ck["b1_checkpoints"], ck["W2_checkpoints"], ck["b2_checkpoints"],
                            d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                            d["grad_L_XQW_mini_batch"], cgs)


def check(res, ref, tol=TOL):
    errs = {k: orc.rel_l2(res[k], ref[k]) for k in GRADS}
    for k in GRADS:
        assert torch.isfinite(res[k]).all(), f"{k} has non-finite values"
        assert errs[k] <= tol, f"{k}: rel-L2 {errs[k]:.3e} > {tol}; all: " + \
            ", ".join(f"{a}={b:.2e}" for a, b in errs.items())
    return errs


@pytest.mark.parametrize("B,H,NC,cgs", [(1, 1, 1, 1), (1, 1, 2, 2), (1, 2, 3, 2), (2, 2, 8, 4), (1, 4, 32, 4)])
def test_backward_matches_oracle(B, H, NC, cgs):
    d = orc.make_inputs(B, H, NC, seed=1, backward=True)
    ck = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    check(run_backward(d, ck, cgs), oracle_backward(d, ck, cgs))


def test_backward_matches_reference_fixture():
    blob = np.load(os.path.join(os.path.dirname(__file__), "golden", "ttt_mlp_golden.npz"))
    for name in ("ragged", "even"):
        B, H, NC, cgs, seed = [int(x) for x in blob[f"{name}/cfg"]]
        d = orc.make_inputs(B, H, NC, seed=seed, eta_scale=float(blob[f"{name}/eta_scale"][0]), backward=True)
        ck = {k: torch.from_numpy(blob[f"{name}/{k}"]) for k in CK}
        ref = {k: torch.from_numpy(blob[f"{name}/{k}"]) for k in GRADS}
        check(run_backward(d, ck, cgs), ref)


def test_backward_with_independent_random_checkpoints():
    """Like the reference's script (kernels/ttt_backward/matching.py:393-396): every group restarts
    from its own checkpoint, whatever it holds."""
    B, H, NC, cgs = 1, 2, 6, 2
    d = orc.make_inputs(B, H, NC, seed=4, backward=True)
    g = torch.Generator().manual_seed(8)
    n = 3
    ck = {"W1_checkpoints": 0.02 * torch.randn(B, H, n, 64, 256, generator=g),
          "b1_checkpoints": 0.02 * torch.randn(B, H, n, 1, 256, generator=g),
          "W2_checkpoints": 0.02 * torch.randn(B, H, n, 256, 64, generator=g),
          "b2_checkpoints": 0.02 * torch.randn(B, H, n, 1, 64, generator=g)}
    check(run_backward(d, ck, cgs), oracle_backward(d, ck, cgs))


def test_forward_then_backward_end_to_end():
    """Checkpoints produced by the forward kernel feed the backward kernel; compare with autograd
    through the oracle forward (fp64)."""
    B, H, NC, cgs = 2, 2, 8, 4
    d = orc.make_inputs(B, H, NC, seed=6, backward=True)
    dev = "cuda"
    t = {k: v.to(dev) for k, v in d.items()}
    n = 2
    ckd = [torch.empty(B, H, n, *s, device=dev) for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
    out = torch.empty_like(t["XQ"])
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                t["W1"], t["b1"], t["W2"], t["b2"], *ckd, out, cgs)
    ck = {k: v.cpu() for k, v in zip(CK, ckd)}
    res = run_backward(d, ck, cgs)
    ref = orc.ttt_backward_autograd(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                    d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"],
                                    d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"],
                                    d["grad_L_b2_last"], d["grad_L_XQW_mini_batch"])
    check(res, {k: v.float() for k, v in ref.items()})


def test_backward_is_deterministic():
    d = orc.make_inputs(1, 2, 4, seed=2, backward=True)
    ck = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         d["W1"], d["b1"], d["W2"], d["b2"], 2)
    a, b = run_backward(d, ck, 2), run_backward(d, ck, 2)
    for k in GRADS:
        assert torch.equal(a[k], b[k]), k
