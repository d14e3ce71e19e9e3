"""Parity of the sm_100a forward with the CPU oracle, through the C ABI.

Gates (relative L2 against the fp32 oracle on the same bf16-rounded inputs):
Out <= 1e-2, every stored checkpoint <= 1e-2 (same bound for the optional final state)."""
import os

import numpy as np
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, take_status

pytestmark = pytest.mark.gpu
TOL_OUT = 1e-2
TOL_STATE = 1e-2
CK = ["W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints"]


def run_forward(d, cgs, final=False):
    dev = "cuda"
    B, H, NC = d["XQ"].shape[:3]
    n = orc.num_checkpoints(NC, cgs)
    t = {k: v.to(dev) for k, v in d.items()}
    ck = [torch.full((B, H, n, *s), float("nan"), device=dev)
          for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
    out = torch.full_like(t["XQ"], float("nan"))
    fin = None
    if final:
        fin = tuple(torch.full((B, H, *s), float("nan"), device=dev)
                    for s in ((64, 256), (1, 256), (256, 64), (1, 64)))
    ret = ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                      t["W1"], t["b1"], t["W2"], t["b2"], *ck, out, cgs, final_state=fin)
    torch.cuda.synchronize()
    assert take_status() == 0
    assert ret is out
    res = {"Out": out.float().cpu()}
    res.update({k: v.cpu() for k, v in zip(CK, ck)})
    if final:
        res.update({k: v.cpu() for k, v in zip(["W1_final", "b1_final", "W2_final", "b2_final"], fin)})
    return res


def check(res, ref, keys_tol):
    errs = {k: orc.rel_l2(res[k], ref[k]) for k, _ in keys_tol}
    for k, tol in keys_tol:
        assert errs[k] <= tol, f"{k}: rel-L2 {errs[k]:.3e} > {tol} (all: {errs})"
    return errs


@pytest.mark.parametrize("B,H,NC,cgs", [(1, 1, 1, 1), (1, 2, 3, 2), (2, 3, 8, 4), (1, 4, 32, 4)])
def test_forward_matches_oracle(B, H, NC, cgs):
    d = orc.make_inputs(B, H, NC, seed=0)
    # non-zero initial biases (the recipe's zeros would leave the bias gates comparing pure update noise)
    g = torch.Generator().manual_seed(77)
    d["b1"] = 0.02 * torch.randn(d["b1"].shape, generator=g)
    d["b2"] = 0.02 * torch.randn(d["b2"].shape, generator=g)
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    res = run_forward(d, cgs, final=True)
    assert torch.isfinite(res["Out"]).all()
    check(res, ref, [("Out", TOL_OUT)] + [(k, TOL_STATE) for k in CK]
          + [(k, TOL_STATE) for k in ("W1_final", "b1_final", "W2_final", "b2_final")])
    # checkpoint 0 is the initial state, bit for bit
    assert torch.equal(res["W1_checkpoints"][:, :, 0], d["W1"])
    assert torch.equal(res["W2_checkpoints"][:, :, 0], d["W2"])


def test_forward_matches_reference_fixture():
    blob = np.load(os.path.join(os.path.dirname(__file__), "golden", "ttt_mlp_golden.npz"))
    for name in ("ragged", "even"):
        B, H, NC, cgs, seed = [int(x) for x in blob[f"{name}/cfg"]]
        d = orc.make_inputs(B, H, NC, seed=seed, eta_scale=float(blob[f"{name}/eta_scale"][0]), backward=True)
        res = run_forward(d, cgs)
        ref = {k: torch.from_numpy(blob[f"{name}/{k}"]) for k in ["Out"] + CK}
        check(res, ref, [("Out", TOL_OUT)] + [(k, TOL_STATE) for k in ("W1_checkpoints", "W2_checkpoints")])


def test_forward_is_deterministic_and_last_eta_rank5():
    d = orc.make_inputs(1, 2, 4, seed=5)
    a = run_forward(d, 2)
    d5 = dict(d)
    d5["last_eta"] = d["last_eta"].unsqueeze(-1).contiguous()
    b = run_forward(d5, 2)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_forward_large_eta_and_nonzero_bias():
    d = orc.make_inputs(2, 2, 6, seed=11, eta_scale=1.0)
    g = torch.Generator().manual_seed(99)
    d["b1"] = 0.02 * torch.randn(d["b1"].shape, generator=g)
    d["b2"] = 0.02 * torch.randn(d["b2"].shape, generator=g)
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], 4)
    res = run_forward(d, 4)
    check(res, ref, [("Out", TOL_OUT)] + [(k, TOL_STATE) for k in CK])


def test_forward_rejects_bad_arguments_on_device():
    d = orc.make_inputs(1, 1, 2, seed=0)
    t = {k: v.cuda() for k, v in d.items()}
    ck = [torch.empty(1, 1, 1, *s, device="cuda") for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
    out = torch.empty_like(t["XQ"])
    args = [t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
            t["W1"], t["b1"], t["W2"], t["b2"], *ck, out, 2]
    bad = list(args); bad[1] = t["XK"].float()
    with pytest.raises(RuntimeError, match="dtype"):
        ttt_forward(*bad)
    bad = list(args); bad[2] = t["XV"].transpose(-1, -2)
    with pytest.raises(RuntimeError, match="contiguous"):
        ttt_forward(*bad)
    bad = list(args); bad[6] = t["W1"][:, :, :, :128].contiguous()
    with pytest.raises(RuntimeError, match="shape"):
        ttt_forward(*bad)
    ttt_forward(*args, sync=True)     # and the good call still works afterwards
