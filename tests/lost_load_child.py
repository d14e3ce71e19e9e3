"""Child process of test_failure_path_gpu.py: runs with a millisecond wait limit (the library reads
TTT_B200_WAIT_LIMIT_MS once per process).  For the forward and the backward, with 1, 2 and 4 CTAs per
stream: a launch whose stream never issues the loads of one mini-batch must come back with code 3 (the
bounded wait for them ran out, the kernel exited through its abort path), and the next, ordinary launch
on the same context must be correct.  Nothing traps, faults or spins without a limit."""
import sys

import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, ttt_backward, take_status
from ttt_tk_b200.buffers import alloc_backward_buffers, alloc_checkpoints, GRAD_NAMES, CHECKPOINT_NAMES


def main():
    dev = "cuda"
    B, H, NC, cgs = 1, 1, 3, 2
    d = orc.make_inputs(B, H, NC, seed=0, backward=True)
    t = {k: v.to(dev) for k, v in d.items()}
    eta5 = t["last_eta"].unsqueeze(-1).contiguous()
    f = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                        d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    g = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"], f["b2_checkpoints"],
                         d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                         d["grad_L_XQW_mini_batch"], cgs)
    ckd = [f[k].to(dev).contiguous() for k in CHECKPOINT_NAMES]
    for cluster in (1, 2, 4):
        def fwd(lost):
            ck = alloc_checkpoints(B, H, NC, cgs, dev)
            out = torch.zeros_like(t["XQ"])
            ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                        t["W1"], t["b1"], t["W2"], t["b2"], *ck, out, cgs, sync=True, cluster=cluster, _lost_load=lost)
            return out

        def bwd(lost):
            scratch, outs = alloc_backward_buffers(B, H, NC, cgs, dev)
            ttt_backward(t["XQ"], t["XK"], t["XV"], eta5, t["ttt_norm_weight"], t["ttt_norm_bias"], *ckd,
                         torch.zeros_like(t["XQ"]), *scratch, t["grad_L_W1_last"], t["grad_L_b1_last"],
                         t["grad_L_W2_last"], t["grad_L_b2_last"], t["grad_L_XQW_mini_batch"],
                         *[outs[k] for k in GRAD_NAMES], cgs, sync=True, cluster=cluster, _lost_load=lost)
            return outs

        for name, fn in (("forward", fwd), ("backward", bwd)):
            try:
                fn(True)
            except RuntimeError as e:
                assert "code 3" in str(e) and "bounded wait" in str(e), str(e)
            else:
                raise AssertionError(f"{name} at cluster {cluster}: the lost load went unnoticed")
            assert take_status() == 0, "the synchronous call takes the report itself"
            res = fn(False)                      # the context is alive and the kernel path intact
            if name == "forward":
                e = orc.rel_l2(res.float().cpu(), f["Out"])
                assert e <= 1e-2, (name, cluster, e)
            else:
                for k in GRAD_NAMES:
                    e = orc.rel_l2(res[k].float().cpu(), g[k])
                    assert e <= 3e-2, (name, cluster, k, e)
            print(f"{name} cluster {cluster}: lost load reported, next launch correct", flush=True)
    # the TTT-Linear forward has the same hook
    from oracle import ttt_linear as lin
    from ttt_tk_b200 import ttt_linear_forward
    dl = lin.make_inputs(B, H, NC, seed=1)
    tl = {k: v.to(dev) for k, v in dl.items()}
    fl = lin.ttt_linear_forward(dl["XQ"], dl["XK"], dl["XV"], dl["last_eta"], dl["ttt_norm_weight"],
                                dl["ttt_norm_bias"], dl["W1"], dl["b1"], cgs)

    def linear(lost):
        n = lin.num_checkpoints(NC, cgs)
        ck = [torch.zeros(B, H, n, 64, 64, device=dev), torch.zeros(B, H, n, 1, 64, device=dev)]
        out = torch.zeros_like(tl["XQ"])
        ttt_linear_forward(tl["XQ"], tl["XK"], tl["XV"], tl["last_eta"], tl["ttt_norm_weight"], tl["ttt_norm_bias"],
                           tl["W1"], tl["b1"], *ck, out, cgs, sync=True, _lost_load=lost)
        return out

    try:
        linear(True)
    except RuntimeError as e:
        assert "code 3" in str(e) and "bounded wait" in str(e), str(e)
    else:
        raise AssertionError("linear forward: the lost load went unnoticed")
    assert take_status() == 0
    e = lin.rel_l2(linear(False).float().cpu(), fl["Out"])
    assert e <= 1e-2, ("linear forward", e)
    print("linear forward: lost load reported, next launch correct", flush=True)
    from ttt_tk_b200 import ttt_linear_backward
    gl = torch.Generator().manual_seed(3)
    go = torch.randn(B, H, NC, 64, 64, generator=gl).bfloat16()
    gW, gb = 1e-3 * torch.randn(B, H, 64, 64, generator=gl), 1e-3 * torch.randn(B, H, 1, 64, generator=gl)
    rl = lin.ttt_linear_backward(dl["XQ"], dl["XK"], dl["XV"], dl["last_eta"], dl["ttt_norm_weight"],
                                 dl["ttt_norm_bias"], fl["W1_checkpoints"], fl["b1_checkpoints"], go, gW, gb, cgs)
    ckl = [fl["W1_checkpoints"].to(dev).contiguous(), fl["b1_checkpoints"].to(dev).contiguous()]

    def linear_bwd(lost):
        outs = [torch.zeros(B, H, 1, 64, device=dev), torch.zeros(B, H, 1, 64, device=dev),
                torch.zeros(B, H, 64, 64, device=dev), torch.zeros(B, H, 1, 64, device=dev),
                torch.zeros(B, H, NC, 64, device=dev, dtype=torch.bfloat16), torch.zeros_like(tl["XQ"]),
                torch.zeros_like(tl["XQ"]), torch.zeros_like(tl["XQ"])]
        ttt_linear_backward(tl["XQ"], tl["XK"], tl["XV"], tl["last_eta"], tl["ttt_norm_weight"], tl["ttt_norm_bias"],
                            *ckl, gW.to(dev), gb.to(dev), go.to(dev), *outs, cgs, sync=True, _lost_load=lost)
        return outs

    try:
        linear_bwd(True)
    except RuntimeError as e:
        assert "code 3" in str(e) and "bounded wait" in str(e), str(e)
    else:
        raise AssertionError("linear backward: the lost load went unnoticed")
    assert take_status() == 0
    res = linear_bwd(False)
    e = lin.rel_l2(res[5].float().cpu(), rl["grad_L_XQ"])
    assert e <= 3e-2, ("linear backward", e)
    e = lin.rel_l2(res[2].cpu(), rl["grad_L_W1_init"])
    assert e <= 3e-2, ("linear backward", e)
    print("linear backward: lost load reported, next launch correct", flush=True)
    print("LOST_LOAD_OK")


if __name__ == "__main__":
    sys.exit(main())
