"""Parity of the TTT-Linear backward kernel with its CPU oracle (the hand-derived reverse step, itself equal to
torch.autograd through the forward: tests/test_linear_oracle.py), through the C ABI.  Gate as for the MLP
operator: every gradient <= 3e-2 relative L2 against the fp32 oracle on the same bf16-rounded inputs."""
import pytest
import torch

from oracle import ttt_linear as lin
from ttt_tk_b200 import ttt_linear_forward, ttt_linear_backward, take_status

pytestmark = pytest.mark.gpu
TOL = 3e-2
NAMES = ["grad_L_ttt_norm_weight", "grad_L_ttt_norm_bias", "grad_L_W1_init", "grad_L_b1_init", "grad_L_last_eta",
         "grad_L_XQ", "grad_L_XK", "grad_L_XV"]


def make(B, H, NC, seed, eta_scale=0.1):
    d = lin.make_inputs(B, H, NC, seed=seed, eta_scale=eta_scale)
    g = torch.Generator().manual_seed(seed + 77)
    d["grad_out"] = torch.randn(B, H, NC, 64, 64, generator=g).bfloat16()
    d["grad_W1_last"] = 1e-3 * torch.randn(B, H, 64, 64, generator=g)
    d["grad_b1_last"] = 1e-3 * torch.randn(B, H, 1, 64, generator=g)
    return d


def oracle(d, cgs):
    f = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                               d["W1"], d["b1"], cgs)
    g = lin.ttt_linear_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                                f["W1_checkpoints"], f["b1_checkpoints"], d["grad_out"], d["grad_W1_last"],
                                d["grad_b1_last"], cgs)
    g["grad_L_last_eta"] = g["grad_L_last_eta"].squeeze(-1)
    return f, g


def run(d, cgs, ck=None, **kw):
    dev = "cuda"
    B, H, NC = d["XQ"].shape[:3]
    n = lin.num_checkpoints(NC, cgs)
    t = {k: v.to(dev) for k, v in d.items()}
    if ck is None:
        ck = [torch.empty(B, H, n, 64, 64, device=dev), torch.empty(B, H, n, 1, 64, device=dev)]
        out = torch.empty_like(t["XQ"])
        ttt_linear_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                           t["W1"], t["b1"], *ck, out, cgs)
    nan = float("nan")
    outs = {"grad_L_ttt_norm_weight": torch.full((B, H, 1, 64), nan, device=dev),
            "grad_L_ttt_norm_bias": torch.full((B, H, 1, 64), nan, device=dev),
            "grad_L_W1_init": torch.full((B, H, 64, 64), nan, device=dev),
            "grad_L_b1_init": torch.full((B, H, 1, 64), nan, device=dev),
            "grad_L_last_eta": torch.full((B, H, NC, 64), nan, device=dev, dtype=torch.bfloat16),
            "grad_L_XQ": torch.full_like(t["XQ"], nan), "grad_L_XK": torch.full_like(t["XQ"], nan),
            "grad_L_XV": torch.full_like(t["XQ"], nan)}
    ttt_linear_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"], *ck,
                        t["grad_W1_last"], t["grad_b1_last"], t["grad_out"], *[outs[k] for k in NAMES], cgs, **kw)
    torch.cuda.synchronize()
    assert take_status() == 0
    return {k: v.float().cpu() for k, v in outs.items()}


def check(res, ref):
    errs = {k: lin.rel_l2(res[k], ref[k]) for k in NAMES}
    for k in NAMES:
        assert torch.isfinite(res[k]).all(), k
        assert errs[k] <= TOL, f"{k}: rel-L2 {errs[k]:.3e} > {TOL}; all: " + ", ".join(f"{a}={b:.2e}" for a, b in errs.items())


@pytest.mark.parametrize("B,H,NC,cgs,eta_scale", [(1, 1, 1, 1, 0.1), (1, 2, 4, 2, 0.1), (2, 3, 7, 3, 0.1),
                                                    (1, 2, 16, 4, 1.0), (2, 2, 5, 8, 0.01), (1, 1, 6, 1, 0.1)])
def test_linear_backward_matches_oracle(B, H, NC, cgs, eta_scale):
    d = make(B, H, NC, seed=NC + 10 * B, eta_scale=eta_scale)
    _, ref = oracle(d, cgs)
    check(run(d, cgs), ref)


def test_linear_backward_from_oracle_checkpoints_many_streams_and_deterministic():
    """More streams than SMs (two waves), checkpoints taken from the oracle; reruns are bit-identical."""
    d = make(4, 40, 6, seed=5)
    f, ref = oracle(d, 4)
    ck = [f["W1_checkpoints"].cuda().contiguous(), f["b1_checkpoints"].cuda().contiguous()]
    a = run(d, 4, ck=ck)
    check(a, ref)
    b = run(d, 4, ck=ck, sync=True)
    for k in NAMES:
        assert torch.equal(a[k], b[k]), k


def test_linear_backward_rejects_small_scratch():
    d = make(1, 1, 2, seed=0)
    with pytest.raises(RuntimeError, match="scratch"):
        run(d, 2, scratch=torch.empty(1024, dtype=torch.uint8, device="cuda"))


def test_linear_backward_stays_inside_its_scratch_and_leaves_inputs_alone():
    """The scratch buffer and every output sit between guard zones; the kernel stores scratch as raw bulk copies at
    computed slot offsets, so a mis-sized slot would land in a guard zone.  (compute-sanitizer is not available.)"""
    from ttt_tk_b200.ops import linear_backward_scratch_bytes
    B, H, NC, cgs = 2, 3, 5, 2
    GUARD, PAT = 4096, 0xA5
    dev = "cuda"
    d = make(B, H, NC, seed=21)
    f, ref = oracle(d, cgs)
    t = {k: v.to(dev) for k, v in d.items()}
    ck = [f["W1_checkpoints"].to(dev).contiguous(), f["b1_checkpoints"].to(dev).contiguous()]
    need = linear_backward_scratch_bytes(B, H, cgs)
    assert need == B * H * cgs * 33280
    raws = []

    def guarded(nbytes):
        raw = torch.full((GUARD + nbytes + GUARD,), PAT, dtype=torch.uint8, device=dev)
        raws.append((raw, nbytes))
        return raw[GUARD:GUARD + nbytes]

    scratch = guarded(need)
    shapes = [((B, H, 1, 64), torch.float32)] * 2 + [((B, H, 64, 64), torch.float32), ((B, H, 1, 64), torch.float32),
                                                    ((B, H, NC, 64), torch.bfloat16)] + [((B, H, NC, 64, 64), torch.bfloat16)] * 3
    outs = []
    for shp, dt in shapes:
        n = 1
        for x in shp:
            n *= x
        outs.append(guarded(n * (4 if dt == torch.float32 else 2)).view(dt).view(*shp))
    before = {k: v.clone() for k, v in t.items()}
    ttt_linear_backward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"], *ck,
                        t["grad_W1_last"], t["grad_b1_last"], t["grad_out"], *outs, cgs, scratch=scratch)
    torch.cuda.synchronize()
    assert take_status() == 0
    for i, (raw, nbytes) in enumerate(raws):
        assert bool((raw[:GUARD] == PAT).all()) and bool((raw[GUARD + nbytes:] == PAT).all()), f"guard zone of buffer {i}"
    for k, v in t.items():
        assert torch.equal(v, before[k]), k
    check({k: o.float().cpu() for k, o in zip(NAMES, outs)}, ref)


def test_linear_autograd_function_against_oracle_autograd():
    """The torch.autograd.Function over the operator pair: loss.backward() through it gives the oracle's autograd
    gradients (norm gradients summed over the batch, the final state an output with its own upstream gradient)."""
    from ttt_tk_b200.autograd import ttt_linear
    B, H, NC = 2, 2, 6
    d = make(B, H, NC, seed=31)
    ref = lin.ttt_linear_backward_autograd(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"],
                                           d["ttt_norm_bias"], d["W1"], d["b1"], d["grad_out"], d["grad_W1_last"],
                                           d["grad_b1_last"], cgs=1)
    keys = ["XQ", "XK", "XV", "last_eta", "ttt_norm_weight", "ttt_norm_bias", "W1", "b1"]
    leaves = {k: d[k].cuda().requires_grad_(True) for k in keys}
    out, (Wf, bf) = ttt_linear(*[leaves[k] for k in keys], checkpoint_group_size=4)
    loss = (out.float() * d["grad_out"].cuda().float()).sum() + (Wf * d["grad_W1_last"].cuda()).sum() + \
        (bf * d["grad_b1_last"].cuda()).sum()
    loss.backward()
    torch.cuda.synchronize()
    assert take_status() == 0
    names = {"XQ": "grad_L_XQ", "XK": "grad_L_XK", "XV": "grad_L_XV", "last_eta": "grad_L_last_eta",
             "ttt_norm_weight": "grad_L_ttt_norm_weight", "ttt_norm_bias": "grad_L_ttt_norm_bias",
             "W1": "grad_L_W1_init", "b1": "grad_L_b1_init"}
    for k, n in names.items():
        err = lin.rel_l2(leaves[k].grad.float().cpu(), ref[n])
        assert err <= TOL, f"{k}: rel-L2 {err:.3e}"


def test_linear_pair_at_the_longest_configured_sequence():
    """NC = 1024 mini-batches (the sequence length of the longest benchmark configuration) on two heads: the
    errors do not grow past the gates over a thousand state updates."""
    B, H, NC, cgs = 1, 2, 1024, 32
    d = make(B, H, NC, seed=3)
    f, ref = oracle(d, cgs)
    t = {k: v.cuda() for k, v in d.items()}
    n = lin.num_checkpoints(NC, cgs)
    ck = [torch.empty(B, H, n, 64, 64, device="cuda"), torch.empty(B, H, n, 1, 64, device="cuda")]
    out = torch.empty_like(t["XQ"])
    fin = (torch.empty(B, H, 64, 64, device="cuda"), torch.empty(B, H, 1, 64, device="cuda"))
    ttt_linear_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"], t["W1"],
                       t["b1"], *ck, out, cgs, final_state=fin)
    assert lin.rel_l2(out.float().cpu(), f["Out"]) <= 1e-2
    assert lin.rel_l2(fin[0].cpu(), f["W1_final"]) <= 1e-2 and lin.rel_l2(ck[0].cpu(), f["W1_checkpoints"]) <= 1e-2
    check(run(d, cgs, ck=ck), ref)
