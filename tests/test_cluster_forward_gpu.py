"""Parity of the cluster-sharded forward (2 or 4 CTAs per (batch, head) stream, the hidden units split
between them, Z2 partial sums exchanged through distributed shared memory) with the CPU oracle and
with the one-CTA kernel, through the C ABI.

Gates as for the one-CTA kernel: Out <= 1e-2, stored state <= 1e-2 relative L2 against the fp32 oracle."""
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, take_status

pytestmark = pytest.mark.gpu
TOL = 1e-2
CK = ["W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints"]
FIN = ["W1_final", "b1_final", "W2_final", "b2_final"]


def run_forward(d, cgs, cluster):
    dev = "cuda"
    B, H, NC = d["XQ"].shape[:3]
    n = orc.num_checkpoints(NC, cgs)
    t = {k: v.to(dev) for k, v in d.items()}
    ck = [torch.full((B, H, n, *s), float("nan"), device=dev) for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
    fin = tuple(torch.full((B, H, *s), float("nan"), device=dev) for s in ((64, 256), (1, 256), (256, 64), (1, 64)))
    out = torch.full_like(t["XQ"], float("nan"))
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                t["W1"], t["b1"], t["W2"], t["b2"], *ck, out, cgs, final_state=fin, cluster=cluster)
    torch.cuda.synchronize()
    assert take_status() == 0
    res = {"Out": out.float().cpu()}
    res.update({k: v.cpu() for k, v in zip(CK, ck)})
    res.update({k: v.cpu() for k, v in zip(FIN, fin)})
    return res


def nonzero_bias_inputs(B, H, NC, seed, eta_scale=0.1):
    d = orc.make_inputs(B, H, NC, seed=seed, eta_scale=eta_scale)
    g = torch.Generator().manual_seed(seed + 1000)
    d["b1"] = 0.02 * torch.randn(d["b1"].shape, generator=g)
    d["b2"] = 0.02 * torch.randn(d["b2"].shape, generator=g)
    return d


@pytest.mark.parametrize("cluster", [2, 4])
@pytest.mark.parametrize("B,H,NC,cgs", [(1, 1, 1, 1), (1, 2, 3, 2), (2, 3, 8, 4), (1, 4, 32, 4)])
def test_cluster_forward_matches_oracle(cluster, B, H, NC, cgs):
    d = nonzero_bias_inputs(B, H, NC, seed=3)
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    res = run_forward(d, cgs, cluster)
    for k in ["Out"] + CK + FIN:
        assert torch.isfinite(res[k]).all(), k
        e = orc.rel_l2(res[k], ref[k])
        assert e <= TOL, f"{k}: rel-L2 {e:.3e} at cluster {cluster}"
    # checkpoint 0 is the initial state, bit for bit, whichever CTA wrote which rows
    assert torch.equal(res["W1_checkpoints"][:, :, 0], d["W1"])
    assert torch.equal(res["W2_checkpoints"][:, :, 0], d["W2"])
    assert torch.equal(res["b1_checkpoints"][:, :, 0], d["b1"])
    assert torch.equal(res["b2_checkpoints"][:, :, 0], d["b2"])


@pytest.mark.parametrize("cluster", [2, 4])
def test_cluster_forward_agrees_with_one_cta_kernel_and_is_deterministic(cluster):
    d = nonzero_bias_inputs(2, 2, 12, seed=7, eta_scale=1.0)
    one = run_forward(d, 4, 1)
    a = run_forward(d, 4, cluster)
    b = run_forward(d, 4, cluster)
    for k in a:
        assert torch.equal(a[k], b[k]), f"{k} differs between two runs at cluster {cluster}"
        # different summation order over the hidden units: equal within the bf16 operand rounding
        assert orc.rel_l2(a[k], one[k]) <= 5e-3, k


def test_cluster_forward_long_sequence_heads_only():
    """The long-context shape's structure (B = 1, few streams, many mini-batches) at a length the oracle
    finishes quickly; the cluster size is the launcher's own choice (4 CTAs per stream here)."""
    B, H, NC, cgs = 1, 2, 96, 32
    d = orc.make_inputs(B, H, NC, seed=5)
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    res = run_forward(d, cgs, None)
    assert orc.rel_l2(res["Out"], ref["Out"]) <= TOL
    for k in ("W1_checkpoints", "W2_checkpoints", "W1_final", "W2_final"):
        assert orc.rel_l2(res[k], ref[k]) <= TOL, k


def test_launcher_choice_follows_the_cluster_capacity():
    """The launcher gives a stream four CTAs only while the device runs that many clusters of four at
    the same time (the occupancy query, not SMs / 4), the forward two while those fit, else one; the
    backward never picks two."""
    from ttt_tk_b200 import _lib
    lib = _lib.lib()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for backward in (0, 1):
        c2, c4 = lib.ttt_b200_cluster_capacity(2, backward), lib.ttt_b200_cluster_capacity(4, backward)
        assert 0 < c4 <= sms // 4 and 0 < c2 <= sms // 2 and c4 <= c2
        assert lib.ttt_b200_cluster_capacity(3, backward) == 0
        assert lib.ttt_b200_pick_cluster(1, backward) == 4
        assert lib.ttt_b200_pick_cluster(c4, backward) == 4
        assert lib.ttt_b200_pick_cluster(c4 + 1, backward) == (1 if backward else 2)
        assert lib.ttt_b200_pick_cluster(c2, backward) == (1 if backward else 2)
        assert lib.ttt_b200_pick_cluster(c2 + 1, backward) == 1
        assert lib.ttt_b200_pick_cluster(0, backward) == -1


def test_a_problem_at_the_capacity_of_four_cta_clusters_runs_in_one_wave():
    """B*H equal to the capacity for clusters of four: the launcher picks four CTAs per stream and the
    result matches the oracle (every cluster is resident, none waits for a peer that is not running)."""
    from ttt_tk_b200 import _lib
    cap = _lib.lib().ttt_b200_cluster_capacity(4, 0)
    d = orc.make_inputs(1, cap, 2, seed=5)
    ref = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                          d["W1"], d["b1"], d["W2"], d["b2"], 2)
    res = run_forward(d, 2, None)
    assert orc.rel_l2(res["Out"], ref["Out"]) <= TOL
