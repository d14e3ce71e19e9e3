"""The `test_time_training` extension module (the reference's module and function names,
test_time_training.cpp:95-104) built over the C ABI."""
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import build
from ttt_tk_b200.buffers import alloc_backward_buffers, alloc_checkpoints, GRAD_NAMES, CHECKPOINT_NAMES


@pytest.fixture(scope="module")
def ttt():
    return build.load_extension()


def test_module_exports_reference_names(ttt):
    assert ttt.__name__ == "test_time_training"
    assert callable(ttt.ttt_forward) and callable(ttt.ttt_backward)
    assert "TTT Forward" in ttt.ttt_forward.__doc__ and "TTT Backward" in ttt.ttt_backward.__doc__


def test_rejects_cpu_tensors_like_torch_check(ttt):
    d = orc.make_inputs(1, 1, 2, seed=0)
    ck = alloc_checkpoints(1, 1, 2, 2, device="cpu")
    with pytest.raises(RuntimeError, match="CUDA"):
        ttt.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                        d["W1"], d["b1"], d["W2"], d["b2"], *ck, torch.empty_like(d["XQ"]), 2)
    with pytest.raises(RuntimeError, match="head dimension"):
        ttt.ttt_forward(d["XQ"][..., :32], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                        d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"], d["b2"], *ck, torch.empty_like(d["XQ"]), 2)


@pytest.mark.gpu
def test_readme_usage_forward_and_backward(ttt):
    """The call sequence of the reference's README.md:22-96, with `.contiguous()` on every argument."""
    B, H, NC, cgs = 2, 3, 6, 4
    dev = "cuda"
    d = orc.make_inputs(B, H, NC, seed=12, backward=True)
    t = {k: v.to(dev) for k, v in d.items()}
    last_eta = t["last_eta"].unsqueeze(-1)
    ck = alloc_checkpoints(B, H, NC, cgs, dev)
    XQW = torch.empty_like(t["XQ"])
    ret = ttt.ttt_forward(t["XQ"].contiguous(), t["XK"].contiguous(), t["XV"].contiguous(), last_eta.contiguous(),
                          t["ttt_norm_weight"].contiguous(), t["ttt_norm_bias"].contiguous(),
                          t["W1"].contiguous(), t["b1"].contiguous(), t["W2"].contiguous(), t["b2"].contiguous(),
                          *[c.contiguous() for c in ck], XQW.contiguous(), cgs)
    assert ret.data_ptr() == XQW.data_ptr()
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    assert orc.rel_l2(XQW.float().cpu(), ref["Out"]) <= 1e-2
    for k, c in zip(CHECKPOINT_NAMES, ck):
        if k.startswith("W"):
            assert orc.rel_l2(c.cpu(), ref[k]) <= 1e-2, k

    scratch, outs = alloc_backward_buffers(B, H, NC, cgs, dev)   # zero-filled, as the reference asks
    ttt.ttt_backward(t["XQ"].contiguous(), t["XK"].contiguous(), t["XV"].contiguous(), last_eta.contiguous(),
                     t["ttt_norm_weight"].contiguous(), t["ttt_norm_bias"].contiguous(),
                     *[c.contiguous() for c in ck], XQW.contiguous(), *[s.contiguous() for s in scratch],
                     t["grad_L_W1_last"].contiguous(), t["grad_L_b1_last"].contiguous(),
                     t["grad_L_W2_last"].contiguous(), t["grad_L_b2_last"].contiguous(),
                     t["grad_L_XQW_mini_batch"].contiguous(), *[outs[k].contiguous() for k in GRAD_NAMES], cgs)
    ckc = {k: c.cpu() for k, c in zip(CHECKPOINT_NAMES, ck)}
    refb = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                            ckc["W1_checkpoints"], ckc["b1_checkpoints"], ckc["W2_checkpoints"],
                            ckc["b2_checkpoints"], d["grad_L_W1_last"], d["grad_L_b1_last"],
                            d["grad_L_W2_last"], d["grad_L_b2_last"], d["grad_L_XQW_mini_batch"], cgs)
    # the caller sums the per-batch norm-gradient rows (kernels/ttt_backward/matching.py:522-523)
    for k in GRAD_NAMES:
        got, want = outs[k].float().cpu(), refb[k]
        if "ttt_norm" in k:
            got, want = got.sum(0), want.sum(0)
        assert orc.rel_l2(got, want) <= 3e-2, k

    with pytest.raises(RuntimeError, match="contiguous"):
        ttt.ttt_forward(t["XQ"].transpose(-1, -2), t["XK"], t["XV"], last_eta, t["ttt_norm_weight"],
                        t["ttt_norm_bias"], t["W1"], t["b1"], t["W2"], t["b2"], *ck, XQW, cgs)
