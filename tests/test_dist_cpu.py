"""`gloo` tests of the multi-rank host logic on CPU: the (batch x head) stream partition of one problem
(batch split at world 2, head split at world 2 with one batch element and at world 4 with two) and the
one all-reduce of the per-head norm gradients.  The per-rank compute is stood in for by the CPU oracle
(the partition and the exchange are what is under test, not the kernel)."""
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


def _worker(rank, world, port, q, B=4, H=2):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    NC, cgs = 2, 2
    d = orc.make_inputs(B, H, NC, seed=5, backward=True)
    mine, (b0, b1, h0, h1) = tdist.shard_tensors(d, rank, world)
    assert mine["XQ"].shape[:2] == (b1 - b0, h1 - h0) and mine["ttt_norm_weight"].shape[:2] == (1, h1 - h0)
    assert (b1 - b0) * (h1 - h0) * world == B * H
    f = orc.ttt_forward(mine["XQ"], mine["XK"], mine["XV"], mine["last_eta"], mine["ttt_norm_weight"],
                        mine["ttt_norm_bias"], mine["W1"], mine["b1"], mine["W2"], mine["b2"], cgs)
    g = orc.ttt_backward(mine["XQ"], mine["XK"], mine["XV"], mine["last_eta"], mine["ttt_norm_weight"],
                         mine["ttt_norm_bias"], f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"],
                         f["b2_checkpoints"], mine["grad_L_W1_last"], mine["grad_L_b1_last"],
                         mine["grad_L_W2_last"], mine["grad_L_b2_last"], mine["grad_L_XQW_mini_batch"], cgs)
    gw, gb = tdist.reduce_norm_grads(g["grad_L_ttt_norm_weight"], g["grad_L_ttt_norm_bias"],
                                     heads=(h0, h1), total_heads=H)
    # every rank's dXQ block, gathered on rank 0 into the full tensor
    full = torch.zeros(B, H, *g["grad_L_XQ"].shape[2:])
    full[b0:b1, h0:h1] = g["grad_L_XQ"]
    dist.reduce(full, dst=0)
    if rank == 0:
        q.put((gw, gb, full))
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


def test_stream_partition_is_a_disjoint_cover_of_whole_heads():
    for (B, H) in [(4, 32), (1, 32), (64, 24), (2, 3), (4, 12)]:
        for world in (1, 2, 4, 8):
            if world > B * H:
                continue
            seen = torch.zeros(B, H, dtype=torch.int32)
            sizes = []
            for r in range(world):
                b0, b1, h0, h1 = tdist.shard_streams(B, H, r, world)
                assert 0 <= b0 < b1 <= B and 0 <= h0 < h1 <= H
                seen[b0:b1, h0:h1] += 1
                sizes.append((b1 - b0) * (h1 - h0))
            assert (seen == 1).all(), (B, H, world)
            if (B * H) % world == 0 and world in (1, 2, 4, 8) and (B, H) != (2, 3):
                assert max(sizes) == min(sizes), (B, H, world, sizes)
    # the forward+backward configuration on 8 GPUs: half the heads of one batch element per rank
    assert tdist.shard_streams(4, 32, 5, 8) == (2, 3, 16, 32)
    # the long-context configuration: B = 1, heads over 8 GPUs
    assert tdist.shard_streams(1, 32, 7, 8) == (0, 1, 28, 32)
    with pytest.raises(ValueError):
        tdist.shard_streams(1, 2, 0, 4)


def _run_world(world, B, H):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, B, H)) for r in range(world)]
    for p in procs:
        p.start()
    gw, gb, dxq = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    NC, cgs = 2, 2
    d = orc.make_inputs(B, H, NC, seed=5, backward=True)
    f = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                        d["W1"], d["b1"], d["W2"], d["b2"], cgs)
    g = orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"], f["b2_checkpoints"],
                         d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                         d["grad_L_XQW_mini_batch"], cgs)
    assert orc.rel_l2(gw, g["grad_L_ttt_norm_weight"].sum(0, keepdim=True)) < 1e-5
    assert orc.rel_l2(gb, g["grad_L_ttt_norm_bias"].sum(0, keepdim=True)) < 1e-5
    assert torch.allclose(dxq, g["grad_L_XQ"], atol=1e-6)


@pytest.mark.timeout(300)
def test_two_ranks_batch_split_match_single_process():
    _run_world(2, B=4, H=2)


@pytest.mark.timeout(300)
def test_two_ranks_head_split_with_fewer_batch_elements_than_ranks():
    _run_world(2, B=1, H=4)


@pytest.mark.timeout(300)
def test_four_ranks_batch_and_head_split():
    _run_world(4, B=2, H=2)
