"""Parity of the cluster-sharded backward (2 or 4 CTAs per (batch, head) stream; hidden units split,
dQ / A2 / dK partial tiles summed through distributed shared memory) with the CPU oracle and with the
one-CTA kernel, through the C ABI.

Gate as for the one-CTA kernel: relative L2 <= 3e-2 for every gradient against the fp32 oracle."""
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, ttt_backward, take_status
from ttt_tk_b200.buffers import alloc_backward_buffers, alloc_checkpoints, GRAD_NAMES, CHECKPOINT_NAMES

pytestmark = pytest.mark.gpu
TOL = 3e-2


def run_backward(d, ck, cgs, cluster):
    dev = "cuda"
    B, H, NC = d["XQ"].shape[:3]
    t = {k: v.to(dev) for k, v in d.items()}
    ckd = [ck[k].to(dev).float().contiguous() for k in CHECKPOINT_NAMES]
    scratch, outs = alloc_backward_buffers(B, H, NC, cgs, fill=float("nan"))
    out_fwd = torch.zeros_like(t["XQ"])
    ttt_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"].unsqueeze(-1).contiguous(),
                 t["ttt_norm_weight"], t["ttt_norm_bias"], *ckd, out_fwd, *scratch,
                 t["grad_L_W1_last"], t["grad_L_b1_last"], t["grad_L_W2_last"], t["grad_L_b2_last"],
                 t["grad_L_XQW_mini_batch"], *[outs[k] for k in GRAD_NAMES], cgs, cluster=cluster)
    torch.cuda.synchronize()
    assert take_status() == 0
    assert not out_fwd.any(), "backward must not touch Out"
    return {k: v.float().cpu() for k, v in outs.items()}


def oracle_forward(d, cgs):
    return orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                           d["W1"], d["b1"], d["W2"], d["b2"], cgs)


def oracle_backward(d, ck, cgs):
    return orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                            ck["W1_checkpoints"], ck["b1_checkpoints"], ck["W2_checkpoints"], ck["b2_checkpoints"],
                            d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                            d["grad_L_XQW_mini_batch"], cgs)


def inputs(B, H, NC, seed, eta_scale=0.1):
    d = orc.make_inputs(B, H, NC, seed=seed, eta_scale=eta_scale, backward=True)
    g = torch.Generator().manual_seed(seed + 500)
    d["b1"] = 0.02 * torch.randn(d["b1"].shape, generator=g)
    d["b2"] = 0.02 * torch.randn(d["b2"].shape, generator=g)
    return d


def check(res, ref, tol, what):
    errs = {k: orc.rel_l2(res[k], ref[k]) for k in GRAD_NAMES}
    for k in GRAD_NAMES:
        assert torch.isfinite(res[k]).all(), f"{k} has non-finite values ({what})"
        assert errs[k] <= tol, f"{k}: rel-L2 {errs[k]:.3e} > {tol} ({what}); all: " + \
            ", ".join(f"{a}={b:.2e}" for a, b in errs.items())


@pytest.mark.parametrize("cluster", [2, 4])
@pytest.mark.parametrize("B,H,NC,cgs", [(1, 1, 1, 1), (1, 1, 2, 2), (1, 2, 3, 2), (2, 2, 8, 4), (1, 4, 32, 4)])
def test_cluster_backward_matches_oracle(cluster, B, H, NC, cgs):
    d = inputs(B, H, NC, seed=1)
    ck = oracle_forward(d, cgs)
    check(run_backward(d, ck, cgs, cluster), oracle_backward(d, ck, cgs), TOL, f"cluster {cluster}")


@pytest.mark.parametrize("cluster", [2, 4])
def test_cluster_backward_agrees_with_one_cta_kernel_and_is_deterministic(cluster):
    B, H, NC, cgs = 2, 2, 10, 4            # ragged last group
    d = inputs(B, H, NC, seed=2, eta_scale=1.0)
    ck = oracle_forward(d, cgs)
    one = run_backward(d, ck, cgs, 1)
    a = run_backward(d, ck, cgs, cluster)
    b = run_backward(d, ck, cgs, cluster)
    for k in GRAD_NAMES:
        assert torch.equal(a[k], b[k]), f"{k} differs between two runs at cluster {cluster}"
    # different summation order over the hidden units: equal within the bf16 operand rounding
    check(a, one, 1e-2, f"cluster {cluster} against one CTA per stream")


@pytest.mark.parametrize("cluster", [2, 4])
def test_cluster_forward_then_backward_against_autograd(cluster):
    """Checkpoints produced by the cluster forward feed the cluster backward; the result is compared with
    autograd through the oracle forward (fp64)."""
    B, H, NC, cgs = 2, 2, 8, 4
    d = orc.make_inputs(B, H, NC, seed=6, backward=True)
    dev = "cuda"
    t = {k: v.to(dev) for k, v in d.items()}
    ckd = alloc_checkpoints(B, H, NC, cgs, dev)
    out = torch.empty_like(t["XQ"])
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                t["W1"], t["b1"], t["W2"], t["b2"], *ckd, out, cgs, cluster=cluster)
    ck = {k: v.cpu() for k, v in zip(CHECKPOINT_NAMES, ckd)}
    res = run_backward(d, ck, cgs, cluster)
    ref = orc.ttt_backward_autograd(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                    d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"],
                                    d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"],
                                    d["grad_L_b2_last"], d["grad_L_XQW_mini_batch"])
    check(res, {k: v.float() for k, v in ref.items()}, TOL, f"cluster {cluster} against autograd")


def test_long_context_shape_with_the_launchers_own_cluster_choice():
    """The long-context configuration's structure (B = 1, few streams, many mini-batches, deep checkpoint
    groups): with 2 streams the launcher gives every stream a cluster of 4 CTAs; forward and backward
    against the oracle at a length it finishes quickly."""
    B, H, NC, cgs = 1, 2, 96, 32
    d = orc.make_inputs(B, H, NC, seed=5, backward=True)
    dev = "cuda"
    t = {k: v.to(dev) for k, v in d.items()}
    ckd = alloc_checkpoints(B, H, NC, cgs, dev)
    out = torch.empty_like(t["XQ"])
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                t["W1"], t["b1"], t["W2"], t["b2"], *ckd, out, cgs)
    f = oracle_forward(d, cgs)
    assert orc.rel_l2(out.float().cpu(), f["Out"]) <= 1e-2
    ck = {k: v.cpu() for k, v in zip(CHECKPOINT_NAMES, ckd)}
    check(run_backward(d, ck, cgs, None), oracle_backward(d, ck, cgs), TOL, "launcher's choice")
