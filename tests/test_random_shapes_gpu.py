"""Randomised parity: seeded random problem shapes (batch, heads, mini-batches, checkpoint group size, ragged last
groups included), eta scales, non-zero initial biases and CTAs per stream, both operator pairs (TTT-MLP and
TTT-Linear), forward and backward, against the CPU oracles with the usual gates (Out and state <= 1e-2, gradients
<= 3e-2 relative L2)."""
import random

import pytest
import torch

from oracle import ttt_linear as lin
from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_backward, ttt_forward, ttt_linear_backward, ttt_linear_forward, take_status
from ttt_tk_b200.buffers import CHECKPOINT_NAMES, GRAD_NAMES, alloc_backward_buffers, alloc_checkpoints

pytestmark = pytest.mark.gpu
LIN_NAMES = ["grad_L_ttt_norm_weight", "grad_L_ttt_norm_bias", "grad_L_W1_init", "grad_L_b1_init", "grad_L_last_eta",
             "grad_L_XQ", "grad_L_XK", "grad_L_XV"]


def cases(seed, n):
    rnd = random.Random(seed)
    return [(i, rnd.choice([1, 1, 2, 3]), rnd.choice([1, 2, 3, 5]), rnd.choice([1, 2, 3, 5, 7, 9, 12]),
             rnd.choice([1, 2, 3, 4, 8]), rnd.choice([1, 2, 4]), rnd.choice([0.01, 0.1, 1.0])) for i in range(n)]


@pytest.mark.parametrize("it,B,H,NC,cgs,cluster,eta_scale", cases(1234, 12))
def test_mlp_pair_on_a_random_shape(it, B, H, NC, cgs, cluster, eta_scale):
    dev = "cuda"
    d = orc.make_inputs(B, H, NC, seed=it, eta_scale=eta_scale, backward=True)
    g = torch.Generator().manual_seed(it + 500)
    d["b1"] = 0.02 * torch.randn(d["b1"].shape, generator=g)
    d["b2"] = 0.02 * torch.randn(d["b2"].shape, generator=g)
    t = {k: v.to(dev) for k, v in d.items()}
    f = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                        d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    r = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"], f["b2_checkpoints"],
                         d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                         d["grad_L_XQW_mini_batch"], cgs)
    ck = alloc_checkpoints(B, H, NC, cgs, dev)
    out = torch.full_like(t["XQ"], float("nan"))
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"], t["W1"], t["b1"],
                t["W2"], t["b2"], *ck, out, cgs, cluster=cluster)
    scratch, outs = alloc_backward_buffers(B, H, NC, cgs, dev, fill=float("nan"))
    ttt_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"].unsqueeze(-1).contiguous(), t["ttt_norm_weight"],
                 t["ttt_norm_bias"], *ck, out, *scratch, t["grad_L_W1_last"], t["grad_L_b1_last"], t["grad_L_W2_last"],
                 t["grad_L_b2_last"], t["grad_L_XQW_mini_batch"], *[outs[k] for k in GRAD_NAMES], cgs, cluster=cluster)
    torch.cuda.synchronize()
    assert take_status() == 0
    assert orc.rel_l2(out.float().cpu(), f["Out"]) <= 1e-2
    for k, c in zip(CHECKPOINT_NAMES, ck):
        assert orc.rel_l2(c.cpu(), f[k]) <= 1e-2, k
    for k in GRAD_NAMES:
        res = outs[k].float().cpu()
        assert torch.isfinite(res).all(), k
        assert orc.rel_l2(res.reshape(r[k].shape), r[k]) <= 3e-2, k


@pytest.mark.parametrize("it,B,H,NC,cgs,cluster,eta_scale", cases(4321, 12))
def test_linear_pair_on_a_random_shape(it, B, H, NC, cgs, cluster, eta_scale):
    dev = "cuda"
    d = lin.make_inputs(B, H, NC, seed=it, eta_scale=eta_scale)
    g = torch.Generator().manual_seed(it + 900)
    go = torch.randn(B, H, NC, 64, 64, generator=g).bfloat16()
    gW, gb = 1e-3 * torch.randn(B, H, 64, 64, generator=g), 1e-3 * torch.randn(B, H, 1, 64, generator=g)
    t = {k: v.to(dev) for k, v in d.items()}
    f = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                               d["W1"], d["b1"], cgs)
    r = lin.ttt_linear_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                                f["W1_checkpoints"], f["b1_checkpoints"], go, gW, gb, cgs)
    n = lin.num_checkpoints(NC, cgs)
    ck = [torch.empty(B, H, n, 64, 64, device=dev), torch.empty(B, H, n, 1, 64, device=dev)]
    out = torch.full_like(t["XQ"], float("nan"))
    ttt_linear_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"], t["W1"],
                       t["b1"], *ck, out, cgs)
    nan = float("nan")
    outs = [torch.full((B, H, 1, 64), nan, device=dev), torch.full((B, H, 1, 64), nan, device=dev),
            torch.full((B, H, 64, 64), nan, device=dev), torch.full((B, H, 1, 64), nan, device=dev),
            torch.full((B, H, NC, 64), nan, device=dev, dtype=torch.bfloat16), torch.full_like(t["XQ"], nan),
            torch.full_like(t["XQ"], nan), torch.full_like(t["XQ"], nan)]
    ttt_linear_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"], *ck,
                        gW.to(dev), gb.to(dev), go.to(dev), *outs, cgs)
    torch.cuda.synchronize()
    assert take_status() == 0
    assert lin.rel_l2(out.float().cpu(), f["Out"]) <= 1e-2
    for k, o in zip(LIN_NAMES, outs):
        res = o.float().cpu()
        assert torch.isfinite(res).all(), k
        assert lin.rel_l2(res.reshape(r[k].shape), r[k]) <= 3e-2, k
