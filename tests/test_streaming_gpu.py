"""Chunked-sequence streaming: a long sequence processed as two calls, the state after the first
chunk's last mini-batch (`final_state`) carried into the second as its initial state, and in the
backward the second chunk's grad_L_W*_init carried into the first as its grad_L_W*_last, must equal one
long call.  The kernels do the same arithmetic in the same order either way (the state crosses the
chunk boundary as fp32), so everything per token and per state entry is bit-identical; only the norm
gradients are sums over mini-batches that the two chunks associate differently."""
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, ttt_backward, take_status
from ttt_tk_b200.buffers import alloc_backward_buffers, alloc_checkpoints, GRAD_NAMES

pytestmark = pytest.mark.gpu
STATE = ["W1", "b1", "W2", "b2"]
UP = ["grad_L_W1_last", "grad_L_b1_last", "grad_L_W2_last", "grad_L_b2_last"]
INIT = ["grad_L_W1_init", "grad_L_b1_init", "grad_L_W2_init", "grad_L_b2_init"]


def forward(t, state, lo, hi, cgs, cluster):
    B, H = t["XQ"].shape[:2]
    dev = t["XQ"].device
    sl = (slice(None), slice(None), slice(lo, hi))
    ck = alloc_checkpoints(B, H, hi - lo, cgs, dev)
    out = torch.empty_like(t["XQ"][sl].contiguous())
    fin = tuple(torch.empty_like(s) for s in state)
    ttt_forward(t["XQ"][sl].contiguous(), t["XK"][sl].contiguous(), t["XV"][sl].contiguous(),
                t["last_eta"][sl].contiguous(), t["ttt_norm_weight"], t["ttt_norm_bias"], *state, *ck, out, cgs,
                final_state=fin, cluster=cluster)
    return out, ck, fin


def backward(t, ck, out, up, lo, hi, cgs, cluster):
    B, H = t["XQ"].shape[:2]
    dev = t["XQ"].device
    sl = (slice(None), slice(None), slice(lo, hi))
    scratch, outs = alloc_backward_buffers(B, H, hi - lo, cgs, dev, fill=float("nan"))
    ttt_backward(t["XQ"][sl].contiguous(), t["XK"][sl].contiguous(), t["XV"][sl].contiguous(),
                 t["last_eta"][sl].unsqueeze(-1).contiguous(), t["ttt_norm_weight"], t["ttt_norm_bias"], *ck, out,
                 *scratch, *up, t["grad_L_XQW_mini_batch"][sl].contiguous(), *[outs[k] for k in GRAD_NAMES], cgs,
                 cluster=cluster)
    return outs


@pytest.mark.parametrize("cluster", [1, 2, 4])
def test_two_chunks_equal_one_long_call(cluster):
    B, H, NC, cgs, cut = 1, 2, 8, 2, 4
    dev = "cuda"
    d = orc.make_inputs(B, H, NC, seed=17, backward=True)
    g = torch.Generator().manual_seed(18)
    d["b1"] = 0.02 * torch.randn(d["b1"].shape, generator=g)
    d["b2"] = 0.02 * torch.randn(d["b2"].shape, generator=g)
    t = {k: v.to(dev) for k, v in d.items()}
    s0 = [t[k] for k in STATE]
    up = [t[k] for k in UP]

    out, ck, fin = forward(t, s0, 0, NC, cgs, cluster)
    grads = backward(t, ck, out, up, 0, NC, cgs, cluster)

    out1, ck1, fin1 = forward(t, s0, 0, cut, cgs, cluster)
    out2, ck2, fin2 = forward(t, list(fin1), cut, NC, cgs, cluster)
    g2 = backward(t, ck2, out2, up, cut, NC, cgs, cluster)
    g1 = backward(t, ck1, out1, [g2[k] for k in INIT], 0, cut, cgs, cluster)
    torch.cuda.synchronize()
    assert take_status() == 0

    assert torch.equal(torch.cat([out1, out2], dim=2), out)
    for a, b in zip(fin2, fin):
        assert torch.equal(a, b)
    for c_long, c1, c2 in zip(ck, ck1, ck2):
        assert torch.equal(torch.cat([c1, c2], dim=2), c_long)
    for k in ("grad_L_XQ", "grad_L_XK", "grad_L_XV", "grad_L_last_eta"):
        assert torch.equal(torch.cat([g1[k], g2[k]], dim=2), grads[k]), k
    for k in INIT:
        assert torch.equal(g1[k], grads[k]), k
    for k in ("grad_L_ttt_norm_weight", "grad_L_ttt_norm_bias"):
        assert torch.allclose(g1[k] + g2[k], grads[k], rtol=1e-4, atol=1e-5), k
    # and the long call itself against the oracle, final state included, with non-zero initial biases
    f = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                        d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    assert orc.rel_l2(out.float().cpu(), f["Out"]) <= 1e-2
    for a, k in zip(fin, ["W1_final", "b1_final", "W2_final", "b2_final"]):
        assert orc.rel_l2(a.cpu(), f[k]) <= 1e-2, k
