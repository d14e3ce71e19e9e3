"""Parity of the TTT-Linear forward kernel with its CPU oracle, through the C ABI.  Gates as for the MLP
operator: Out <= 1e-2, stored state <= 1e-2 relative L2 against the fp32 oracle on the same bf16-rounded
inputs."""
import pytest
import torch

from oracle import ttt_linear as lin
from ttt_tk_b200 import ttt_linear_forward, take_status

pytestmark = pytest.mark.gpu
TOL = 1e-2


def run(d, cgs, **kw):
    dev = "cuda"
    B, H, NC = d["XQ"].shape[:3]
    n = lin.num_checkpoints(NC, cgs)
    t = {k: v.to(dev) for k, v in d.items()}
    nan = float("nan")
    ck = [torch.full((B, H, n, 64, 64), nan, device=dev), torch.full((B, H, n, 1, 64), nan, device=dev)]
    fin = (torch.full((B, H, 64, 64), nan, device=dev), torch.full((B, H, 1, 64), nan, device=dev))
    out = torch.full_like(t["XQ"], nan)
    ttt_linear_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                       t["W1"], t["b1"], *ck, out, cgs, final_state=fin, **kw)
    torch.cuda.synchronize()
    assert take_status() == 0
    return {"Out": out.float().cpu(), "W1_checkpoints": ck[0].cpu(), "b1_checkpoints": ck[1].cpu(),
            "W1_final": fin[0].cpu(), "b1_final": fin[1].cpu()}


def check(res, ref):
    for k in ("Out", "W1_checkpoints", "b1_checkpoints", "W1_final", "b1_final"):
        assert torch.isfinite(res[k]).all(), k
        err = lin.rel_l2(res[k], ref[k])
        assert err <= TOL, f"{k}: rel-L2 {err:.3e} > {TOL}"


@pytest.mark.parametrize("B,H,NC,cgs,eta_scale", [(1, 1, 1, 1, 0.1), (1, 2, 4, 2, 0.1), (2, 3, 7, 3, 0.1),
                                                    (1, 2, 16, 4, 1.0), (2, 2, 5, 8, 0.01)])
def test_linear_forward_matches_oracle(B, H, NC, cgs, eta_scale):
    d = lin.make_inputs(B, H, NC, seed=NC, eta_scale=eta_scale)
    ref = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                 d["ttt_norm_bias"], d["W1"], d["b1"], cgs)
    check(run(d, cgs), ref)


def test_linear_forward_many_streams_two_ctas_per_sm():
    """More streams than SMs: two CTAs share an SM."""
    d = lin.make_inputs(8, 40, 6, seed=11)
    ref = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                 d["ttt_norm_bias"], d["W1"], d["b1"], 4)
    check(run(d, 4), ref)


def test_linear_forward_long_sequence_and_reruns_are_bit_identical():
    d = lin.make_inputs(1, 2, 128, seed=2)
    ref = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                 d["ttt_norm_bias"], d["W1"], d["b1"], 16)
    a = run(d, 16)
    check(a, ref)
    b = run(d, 16, sync=True)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_linear_forward_two_chunks_equal_one_call():
    d = lin.make_inputs(1, 2, 8, seed=4)
    whole = run(d, 2)
    first = {k: (v[:, :, :4] if v.dim() >= 4 and k in ("XQ", "XK", "XV", "last_eta") else v) for k, v in d.items()}
    a = run(first, 2)
    second = {k: (v[:, :, 4:] if k in ("XQ", "XK", "XV", "last_eta") else v) for k, v in d.items()}
    second["W1"], second["b1"] = a["W1_final"], a["b1_final"]
    b = run(second, 2)
    assert torch.equal(torch.cat([a["Out"], b["Out"]], dim=2), whole["Out"])
    assert torch.equal(b["W1_final"], whole["W1_final"]) and torch.equal(b["b1_final"], whole["b1_final"])


def test_linear_forward_rejects_bad_arguments():
    d = lin.make_inputs(1, 1, 2, seed=0)
    t = {k: v.cuda() for k, v in d.items()}
    ck = [torch.empty(1, 1, 1, 64, 64, device="cuda"), torch.empty(1, 1, 1, 1, 64, device="cuda")]
    out = torch.empty_like(t["XQ"])
    with pytest.raises((RuntimeError, ValueError)):      # W1 of the MLP shape
        ttt_linear_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                           torch.empty(1, 1, 64, 256, device="cuda"), t["b1"], *ck, out, 2)
    with pytest.raises((RuntimeError, ValueError)):      # wrong number of checkpoints
        ttt_linear_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                           t["W1"], t["b1"], *ck, out, 1)
