"""World-size-2 `gloo` test of the multi-rank host logic on CPU: batch sharding and the one
all-reduce of the per-head norm gradients.  The per-rank compute is stood in for by the CPU
oracle (the sharding and the exchange are what is under test, not the kernel)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ttt_mlp as orc
from ttt_tk_b200 import dist as tdist


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    B, H, NC, cgs = 4, 2, 2, 2
    d = orc.make_inputs(B, H, NC, seed=5, backward=True)
    mine = tdist.shard_batch(d, rank, world)
    assert mine["XQ"].shape[0] == B // world and mine["ttt_norm_weight"].shape[0] == 1
    f = orc.ttt_forward(mine["XQ"], mine["XK"], mine["XV"], mine["last_eta"], mine["ttt_norm_weight"],
                        mine["ttt_norm_bias"], mine["W1"], mine["b1"], mine["W2"], mine["b2"], cgs)
    g = orc.ttt_backward(mine["XQ"], mine["XK"], mine["XV"], mine["last_eta"], mine["ttt_norm_weight"],
                         mine["ttt_norm_bias"], f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"],
                         f["b2_checkpoints"], mine["grad_L_W1_last"], mine["grad_L_b1_last"],
                         mine["grad_L_W2_last"], mine["grad_L_b2_last"], mine["grad_L_XQW_mini_batch"], cgs)
    gw, gb = tdist.reduce_norm_grads(g["grad_L_ttt_norm_weight"], g["grad_L_ttt_norm_bias"])
    if rank == 0:
        q.put((gw, gb, g["grad_L_XQ"]))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    for n in (1, 7, 128, 129):
        for world in (1, 2, 3, 8):
            spans = [tdist.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.timeout(300)
def test_two_ranks_match_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    gw, gb, dxq0 = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    B, H, NC, cgs = 4, 2, 2, 2
    d = orc.make_inputs(B, H, NC, seed=5, backward=True)
    f = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                        d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    g = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"], f["b2_checkpoints"],
                         d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                         d["grad_L_XQW_mini_batch"], cgs)
    assert orc.rel_l2(gw, g["grad_L_ttt_norm_weight"].sum(0, keepdim=True)) < 1e-5
    assert orc.rel_l2(gb, g["grad_L_ttt_norm_bias"].sum(0, keepdim=True)) < 1e-5
    assert torch.allclose(dxq0, g["grad_L_XQ"][:2], atol=1e-6)      # rank 0 owns batch elements 0..1
