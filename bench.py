#!/usr/bin/env python
"""Benchmark of the TTT-MLP forward + backward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c1|c3|c4|c0|small|prof|glue] [--scaling strong|weak] [--cluster 0|1|2|4]

One "step" = one forward + one backward over one batch of synthetic input of the named workload
(default: the forward+backward configuration, B=4 H=32 seq 8192 cgs 8).  With N > 1 (launched by
torch.distributed.run, one rank per GPU) the (batch x head) streams of that ONE problem are
partitioned across the ranks (strong scaling: 128 / N streams per GPU) and the per-head norm gradients
are summed with one NCCL all-reduce, the only exchange the path has; the same run then also times N
replicas of the whole problem (weak scaling) and reports that number under "weak".

Prints ONE JSON line (rank 0).  `value` is device-timed with the inputs resident in HBM; `e2e` is
measured through the public operator API with pinned host buffers, host<->device copies inside the
timed region: every step copies all of its inputs in and all of its results out; the independent
(batch element, head range) chunks run on their own CUDA streams and are not joined between steps, so
a step's copies overlap the neighbouring steps' kernels.  `--impl reference` times the CPU oracle (the
PyTorch-eager restatement of the reference's own PyTorch functions; the reference's CUDA kernels are
sm_90a-only and cannot run on this GPU) on the host cores on a bounded sample of the same workload.
`--workload glue` times the layer-side kernels around the operator (eta gate, token layout transforms,
output norm) instead; they are HBM-bound.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, NC, cgs, description)
    "c2": (4, 32, 128, 8, "configs[2]: fwd+bwd, B=4 H=32 seq=8192 (NC=128) cgs=8, per GPU"),
    "c1": (4, 12, 32, 4, "configs[1] shape run fwd+bwd, B=4 H=12 seq=2048 (NC=32) cgs=4, per GPU"),
    "c0": (1, 4, 32, 4, "configs[0] shape, B=1 H=4 seq=2048 (NC=32) cgs=4"),
    "c3": (1, 32, 1024, 32, "configs[3] shape on one GPU, B=1 H=32 seq=65536 (NC=1024) cgs=32"),
    "c4": (64, 24, 64, 16, "configs[4] shape run fwd+bwd on one GPU, B=64 H=24 seq=4096 (NC=64) cgs=16"),
    "small": (1, 8, 16, 4, "small case, B=1 H=8 seq=1024 cgs=4"),
    "prof": (4, 32, 16, 8, "profiling case: configs[2] streams (B=4 H=32) at seq=1024 (NC=16) cgs=8"),
    "profc": (1, 32, 16, 8, "profiling case of the cluster kernels: 32 streams (B=1 H=32) at seq=1024 (NC=16) cgs=8"),
    "c2half": (2, 32, 128, 8, "half of configs[2] (what each of two GPUs gets): B=2 H=32 seq=8192 (NC=128) cgs=8"),
    "profc2": (2, 32, 16, 8, "profiling case with 64 streams (B=2 H=32) at seq=1024 (NC=16) cgs=8"),
    "glue": (4, 32, 128, 8, "layer-side kernels at the configs[2] shape: B=4 T=8192 H=32"),
    "linear": (64, 24, 64, 16, "TTT-Linear forward at the configs[4] shape: B=64 H=24 seq=4096 (NC=64) cgs=16"),
    "linear_c2": (4, 32, 128, 8, "TTT-Linear forward at the configs[2] shape: B=4 H=32 seq=8192 (NC=128) cgs=8"),
}
U_FLOP = 2 * 64 * 64 * 256            # one GEMM unit per mini-batch per (b,h)
FWD_U, BWD_U = 7, 22                  # algorithmic GEMM units: forward; backward (7 recompute + 15 sweep)
STATE_BYTES = 132352                  # fp32 W1 + b1 + W2 + b2 of one (b,h)
# DRAM bytes per (stream, mini-batch) of the one-CTA kernels from an ncu capture of the `prof` workload
# (dram__bytes_read.sum + dram__bytes_write.sum over 128 streams x 16 mini-batches); the traffic grows in
# proportion to the number of (stream, mini-batch) pairs, so a full-size launch is scaled from it.
NCU_BWD_DRAM_BYTES_PER_MB = (583610880 + 585072384) / 2048
NCU_FWD_DRAM_BYTES_PER_MB = (67620096 + 8762112) / 2048
# Scratch bytes the backward asks for per (stream, mini-batch): the recompute writes seven [256][64] bf16 images
# (X2, Z1, dl/dZ1, gelu'(Z1_bar), X2_bar, W1^T, W2), three [64][64] bf16 tiles and two fp32[64] vectors; the sweep
# reads the same back, X2 twice.
SCRATCH_WRITE_PER_MB = 7 * 32768 + 3 * 8192 + 512
SCRATCH_READ_PER_MB = 8 * 32768 + 3 * 8192 + 512


def algorithmic_bytes(B, H, NC, cgs):
    """HBM bytes the path must move per step (inputs, outputs, checkpoints), per GPU."""
    T = NC * 64
    n = -(-NC // cgs)
    fwd = 514 * T + STATE_BYTES + 512 + n * STATE_BYTES
    bwd = 900 * T + n * STATE_BYTES + 2 * STATE_BYTES + 512 + 1024
    return B * H * fwd, B * H * bwd


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        """Start sampling and return once the first sample has arrived (nvidia-smi needs a moment
        to come up; the timed region is only tens of milliseconds long)."""
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "10"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.first = self.proc.stdout.readline()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():   # the sample taken before the GPU was under load is left out
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_host_inputs(B, H, NC, seed):
    from ttt_tk_b200.synthetic import make_inputs
    return make_inputs(B, H, NC, seed=seed, eta_scale=0.1, backward=True)


class DeviceStep:
    """Device-resident buffers of one rank's streams and the fwd+bwd step through the operator API."""

    def __init__(self, host, cgs, dev, cluster=None, heads=None, total_heads=None):
        from ttt_tk_b200.buffers import alloc_backward_buffers, GRAD_NAMES
        self.GRADS = GRAD_NAMES
        self.cgs = cgs
        self.dev = dev
        self.cluster = cluster
        B, H, NC = host["XQ"].shape[:3]
        self.B, self.H, self.NC = B, H, NC
        self.heads = (0, H) if heads is None else heads          # this rank's heads within the whole problem
        self.total_heads = H if total_heads is None else total_heads
        n = -(-NC // cgs)
        self.t = {k: v.to(dev) for k, v in host.items()}
        self.t["last_eta5"] = self.t["last_eta"].unsqueeze(-1).contiguous()
        self.ck = [torch.empty(B, H, n, *s, device=dev) for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
        self.out = torch.empty_like(self.t["XQ"])
        self.scratch, self.outs = alloc_backward_buffers(B, H, NC, cgs, device=dev, fill=0.0)
        self.norm_grads = None

    def forward(self, sl=(slice(None), slice(None)), norm=None):
        """Forward over the streams `sl` = (batch element b:b+1 or all, head range): such a slice of a
        contiguous [B, H, ...] tensor is contiguous."""
        from ttt_tk_b200 import ttt_forward
        t = self.t
        hs = (slice(None), sl[1])
        nw, nb = norm if norm is not None else (t["ttt_norm_weight"][hs], t["ttt_norm_bias"][hs])
        ttt_forward(t["XQ"][sl], t["XK"][sl], t["XV"][sl], t["last_eta"][sl], nw,
                    nb, t["W1"][sl], t["b1"][sl], t["W2"][sl], t["b2"][sl],
                    *[c[sl] for c in self.ck], self.out[sl], self.cgs, cluster=self.cluster)

    def backward(self, sl=(slice(None), slice(None)), norm=None):
        from ttt_tk_b200 import ttt_backward
        t = self.t
        hs = (slice(None), sl[1])
        nw, nb = norm if norm is not None else (t["ttt_norm_weight"][hs], t["ttt_norm_bias"][hs])
        ttt_backward(t["XQ"][sl], t["XK"][sl], t["XV"][sl], t["last_eta5"][sl], nw,
                     nb, *[c[sl] for c in self.ck], self.out[sl],
                     *[x[sl] for x in self.scratch],
                     t["grad_L_W1_last"][sl], t["grad_L_b1_last"][sl], t["grad_L_W2_last"][sl],
                     t["grad_L_b2_last"][sl], t["grad_L_XQW_mini_batch"][sl],
                     *[self.outs[k][sl] for k in self.GRADS], self.cgs, cluster=self.cluster)

    def reduce_norm_grads(self):
        # the caller-side batch sum the operator's layout asks for, then the one exchange of the path
        from ttt_tk_b200.dist import reduce_norm_grads
        self.norm_grads = reduce_norm_grads(self.outs["grad_L_ttt_norm_weight"], self.outs["grad_L_ttt_norm_bias"],
                                            heads=self.heads, total_heads=self.total_heads)


def timed_steps(step, K, W, world, dev):
    """W warm-up steps, then K steps timed with CUDA events between a barrier + synchronize on both sides.
    Returns (total ms, mean forward ms, mean backward ms), each the maximum over the ranks."""
    import torch.distributed as dist
    from ttt_tk_b200 import take_status

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        step.forward()
        step.backward()
        step.reduce_norm_grads()
    barrier()
    assert take_status() == 0, "device-side wait ran out during warm-up"
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    t_end = torch.cuda.Event(enable_timing=True)
    barrier()
    for k in range(K):
        ev[k][0].record()
        step.forward()
        ev[k][1].record()
        step.backward()
        ev[k][2].record()
        step.reduce_norm_grads()
    t_end.record()
    barrier()
    assert take_status() == 0, "device-side wait ran out during the timed region"
    total_ms = ev[0][0].elapsed_time(t_end)
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    tt = torch.tensor([total_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    return tt.tolist()


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from ttt_tk_b200 import _lib
    from ttt_tk_b200.dist import shard_tensors
    B, H, NC, cgs, desc = WORKLOADS[args.workload]
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    strong = args.scaling == "strong"
    cluster = args.cluster or None
    K, W = args.steps, args.warmup

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the measured arm: ONE problem, its (batch x head) streams partitioned over the ranks (strong), or
    # one whole problem per rank (weak)
    if strong:
        full = make_host_inputs(B, H, NC, seed=0)
        host, (b0, b1, h0, h1) = shard_tensors(full, rank, world)
        del full
        step = DeviceStep(host, cgs, dev, cluster, heads=(h0, h1), total_heads=H)
    else:
        host = make_host_inputs(B, H, NC, seed=rank)
        b0, b1, h0, h1 = 0, B, 0, H
        step = DeviceStep(host, cgs, dev, cluster)
    Bl, Hl = b1 - b0, h1 - h0
    lib = _lib.lib()
    cl_used = cluster or lib.ttt_b200_pick_cluster(Bl * Hl, 1)
    cl_fwd = cluster or lib.ttt_b200_pick_cluster(Bl * Hl, 0)

    sampler = ClockSampler(local_rank)
    # warm-up happens inside timed_steps; the sampler is started just before so that most of its samples
    # fall into the timed region (the first one, taken at idle, is dropped)
    if rank == 0:
        sampler.start()
    total_ms, fwd_ms, bwd_ms = timed_steps(step, K, W, world, dev)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the operator API with pinned host buffers
    e2e_steps = max(1, min(K, args.e2e_steps))
    in_keys = ["XQ", "XK", "XV", "last_eta", "ttt_norm_weight", "ttt_norm_bias", "W1", "b1", "W2", "b2",
               "grad_L_XQW_mini_batch", "grad_L_W1_last", "grad_L_b1_last", "grad_L_W2_last", "grad_L_b2_last"]
    pin_in = {k: host[k].contiguous().pin_memory() for k in in_keys}
    out_t = {"Out": step.out, **step.outs}
    pin_out = {k: torch.empty(v.shape, dtype=v.dtype).pin_memory() for k, v in out_t.items()}
    h2d = sum(v.numel() * v.element_size() for v in pin_in.values())
    d2h = sum(v.numel() * v.element_size() for v in pin_out.values())

    # The (batch element, head range) chunks are independent, so each one runs on its own CUDA stream:
    # its host->device copies, forward, backward and device->host copies follow one another there, and
    # the chunks are not joined at a step boundary.  Chunk c of step i+1 therefore starts copying in
    # while other chunks of step i still compute or copy out (a training loop that prefetches its
    # next batch): both copy directions and the kernels stay busy.  Every step still copies all of its
    # inputs in and all of its results out, and the norm-gradient batch sum of a step is taken before
    # the next step's backward may overwrite its addends.
    hsplit = max(1, min(args.e2e_head_chunks, Hl))
    hb = [(i * Hl // hsplit, (i + 1) * Hl // hsplit) for i in range(hsplit)]
    bpc = max(1, min(args.e2e_batch_per_chunk, Bl))
    if Bl == 1 and hsplit == 1 and Hl >= 2:
        hb = [(0, Hl // 2), (Hl // 2, Hl)]           # one batch element per rank: two head ranges keep two chunks in flight
        hsplit = 2
    if hsplit > 1:
        bpc = 1                                      # a head range of several batch elements is not contiguous
    chunks = [(slice(b, min(b + bpc, Bl)), slice(x0, x1)) for b in range(0, Bl, bpc) for (x0, x1) in hb]
    streams = [torch.cuda.Stream(device=dev) for _ in chunks]        # copies in + kernels of a chunk
    out_streams = [torch.cuda.Stream(device=dev) for _ in chunks]    # copies out of a chunk
    shared_keys = ["ttt_norm_weight", "ttt_norm_bias"]
    step.t["last_eta5"] = step.t["last_eta"].unsqueeze(-1)     # a view: follows the copies into last_eta
    # every chunk keeps its own device copy of its heads' norm parameters (no chunk reads what another writes)
    norm_dev = [tuple(torch.empty_like(step.t[k][:, sl[1]]) for k in shared_keys) for sl in chunks]

    def e2e_steps_run(n_steps):
        main = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(main)
        reduced = None
        copied_out = [None] * len(chunks)
        for _ in range(n_steps):
            done = []
            for i, sl in enumerate(chunks):
                st, so = streams[i], out_streams[i]
                with torch.cuda.stream(st):
                    st.wait_event(start)
                    # the inputs of this step go in while the chunk's previous results still go out
                    for k, v in pin_in.items():
                        if k not in shared_keys:
                            step.t[k][sl].copy_(v[sl], non_blocking=True)
                    for k, d in zip(shared_keys, norm_dev[i]):
                        d.copy_(pin_in[k][:, sl[1]], non_blocking=True)
                    if copied_out[i] is not None:
                        st.wait_event(copied_out[i])     # the kernels overwrite the previous step's results
                    step.forward(sl, norm=norm_dev[i])
                    if reduced is not None:
                        st.wait_event(reduced)      # the previous step's norm gradients have been summed
                    step.backward(sl, norm=norm_dev[i])
                    ev_c = torch.cuda.Event()
                    ev_c.record(st)
                    done.append(ev_c)
                with torch.cuda.stream(so):
                    so.wait_event(ev_c)
                    for k, v in out_t.items():
                        pin_out[k][sl].copy_(v[sl], non_blocking=True)
                    copied_out[i] = torch.cuda.Event()
                    copied_out[i].record(so)
            for ev_c in done:
                main.wait_event(ev_c)
            step.reduce_norm_grads()
            reduced = torch.cuda.Event()
            reduced.record(main)
        for so in out_streams:
            main.wait_stream(so)

    def timed(fn):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        fn()
        host_ms = (time.perf_counter() - t0) * 1e3
        e1.record()
        barrier()
        et = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        return et.item(), host_ms

    e2e_steps_run(2)
    e2e_total, issue_total = timed(lambda: e2e_steps_run(e2e_steps))
    e2e_ms, t_issue = e2e_total / e2e_steps, issue_total / e2e_steps

    # each copy direction alone, all ranks at once: what the host side gives one rank when the others copy too
    def copy_in():
        for k, v in pin_in.items():
            step.t[k].copy_(v, non_blocking=True)

    def copy_out():
        for k, v in out_t.items():
            pin_out[k].copy_(v, non_blocking=True)

    copy_in(); copy_out()
    h2d_ms, _ = timed(copy_in)
    d2h_ms, _ = timed(copy_out)

    # both directions at once (two streams): the floor of an end-to-end step, whose copies in and out overlap
    side = torch.cuda.Stream(device=dev)

    def copy_both():
        main = torch.cuda.current_stream()
        side.wait_stream(main)
        copy_in()
        with torch.cuda.stream(side):
            copy_out()
        main.wait_stream(side)

    copy_both()
    duplex_ms, _ = timed(copy_both)

    # ---- N replicas of the whole problem (weak scaling), as an extra number of the same run
    weak = None
    if strong and world > 1:
        del step, pin_in, pin_out, out_t, norm_dev
        torch.cuda.empty_cache()
        wstep = DeviceStep(make_host_inputs(B, H, NC, seed=rank), cgs, dev, cluster)
        wK = max(2, K // 2)
        w_total, w_fwd, w_bwd = timed_steps(wstep, wK, 3, world, dev)
        weak = {"value": world * B * NC * 64 / (w_total / wK * 1e-3), "unit": "tokens/s", "ms_per_step": w_total / wK,
                "steps": wK, "streams_per_gpu": B * H, "note": "one whole problem per GPU (replicas), same run"}

    if rank != 0:
        return None
    pk, pk_src = peaks()
    tokens_per_step = (B if strong else world * B) * NC * 64
    ms_per_step = total_ms / K
    th = Bl * Hl * NC * 64                  # token-heads per GPU per step
    fwd_flop, bwd_flop = th * 32768 * FWD_U, th * 32768 * BWD_U
    fwd_bytes, bwd_bytes = algorithmic_bytes(Bl, Hl, NC, cgs)
    burst, sustained = pk["bf16_tflops"], pk.get("bf16_tflops_sustained", pk["bf16_tflops"])
    # A kernel timed inside a short region at full clock is held against the burst figure; one that ran
    # under the power cap (clock well below maximum) or for seconds, against the sustained one.
    at_max = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                  and clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"])
    use_burst = at_max and total_ms < 1000.0
    peak_tf = burst if use_burst else sustained
    bwd_tf = bwd_flop / (bwd_ms * 1e-3) / 1e12
    both_tf = (fwd_flop + bwd_flop) / ((fwd_ms + bwd_ms) * 1e-3) / 1e12
    n = -(-NC // cgs)
    remat_bytes = Bl * Hl * (2 * n * STATE_BYTES + NC * (SCRATCH_WRITE_PER_MB + SCRATCH_READ_PER_MB))
    bwd_kernel = "ttt_bwd_kernel" if cl_used == 1 else f"ttt_bwd_cluster_kernel<{cl_used}>"
    res = {
        "metric": "ttt_mlp_fwd_bwd_tokens_per_s", "value": tokens_per_step / (ms_per_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": desc, "B": B, "H": H, "seq_len": NC * 64, "checkpoint_group_size": cgs,
                   "parallelism": (f"one problem, (batch x head) streams partitioned over {world} GPU(s): "
                                   f"{Bl} x {Hl} = {Bl * Hl} streams per GPU" if strong else
                                   f"one whole problem per GPU (replicas), {world} GPU(s)"),
                   "ctas_per_stream": {"forward": cl_fwd, "backward": cl_used},
                   "l2": "working set per step (~1.7 GB at c2 on one GPU) exceeds the 126 MB L2; no explicit flush"},
        "kernels": {"fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                    "fwd_tflops": fwd_flop / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": bwd_tf,
                    "fwd_bwd_tflops": both_tf,
                    "fwd_bwd_frac_of_bf16_burst_peak": both_tf / burst,
                    "fwd_bwd_frac_of_bf16_sustained_peak": both_tf / sustained,
                    "fwd_algorithmic_gbs": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                    "bwd_algorithmic_gbs": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
                    "streams_per_gpu": Bl * Hl, "ctas_per_stream_fwd": cl_fwd, "ctas_per_stream_bwd": cl_used},
        # checkpoint + recompute scratch traffic: checkpoints written by the forward and read by the backward,
        # scratch slots written by the recompute and read back by the sweep (bytes the kernels ask for)
        "remat_traffic": {"bytes_per_step": remat_bytes,
                          "hbm_gbs_achieved": remat_bytes / ((fwd_ms + bwd_ms) * 1e-3) / 1e9,
                          "frac_of_hbm_peak": remat_bytes / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / pk["hbm_gbs"],
                          "dram_bytes_measured_bwd": NCU_BWD_DRAM_BYTES_PER_MB * Bl * Hl * NC,
                          "dram_gbs_measured_bwd": NCU_BWD_DRAM_BYTES_PER_MB * Bl * Hl * NC / (bwd_ms * 1e-3) / 1e9},
        "roofline": {"kernel": bwd_kernel, "bound": "tensor", "achieved": bwd_tf, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": bwd_tf / peak_tf,
                     "frac_of_burst": bwd_tf / burst, "frac_of_sustained": bwd_tf / sustained,
                     "traffic": NCU_BWD_DRAM_BYTES_PER_MB * Bl * Hl * NC,
                     "traffic_note": "bytes per launch, scaled from an ncu capture of a smaller launch of the "
                                     "one-CTA kernel by (streams x mini-batches)",
                     "peak_source": f"{pk_src}, " + ("burst cuBLAS bf16 (timed region under 1 s at full clock)" if use_burst
                                                     else "sustained cuBLAS bf16 (clock below maximum or a long region)")},
        "e2e": {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "host_issue_ms_per_step": t_issue,
                "h2d_gbs_alone_per_rank": h2d / (h2d_ms * 1e-3) / 1e9,
                "d2h_gbs_alone_per_rank": d2h / (d2h_ms * 1e-3) / 1e9,
                "copies_both_directions_ms": duplex_ms,
                "frac_of_copy_floor": duplex_ms / e2e_ms,
                "copy_note": "bytes are per rank; the *_alone figures time one direction with all ranks copying at once "
                             "(slowest rank), i.e. what the host's PCIe / memory fabric gives each rank; "
                             "copies_both_directions_ms times one step's copies in and out running at the same time with "
                             "no kernel at all: the floor of an end-to-end step (frac_of_copy_floor = that / ms_per_step)",
                "pipelining": f"{len(chunks)} (batch element, head range) chunks, each with a stream for copies in + "
                              "kernels and one for copies out, not joined between steps: copies in, kernels and copies out "
                              "of neighbouring steps overlap"},
        "gpu_launches": 2 * K,
        "clocks": clocks,
    }
    if weak is not None:
        res["weak"] = weak
    return res


def cpu_oracle_rate(sample_B, sample_H, NC, cgs, H_full, reps, threads, warmup=1):
    """tokens/s of the CPU oracle (fwd + hand-derived bwd) on a slice of the workload.
    A token spans all H_full heads, so a slice with sample_H heads counts sample_H / H_full of it.
    Returns (tokens/s from the median repetition, median seconds, mean seconds)."""
    from oracle import ttt_mlp as orc
    torch.set_num_threads(threads)
    d = orc.make_inputs(sample_B, sample_H, NC, seed=0, backward=True)

    def once():
        f = orc.ttt_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                            d["W1"], d["b1"], d["W2"], d["b2"], cgs)
        orc.ttt_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                         f["W1_checkpoints"], f["b1_checkpoints"], f["W2_checkpoints"], f["b2_checkpoints"],
                         d["grad_L_W1_last"], d["grad_L_b1_last"], d["grad_L_W2_last"], d["grad_L_b2_last"],
                         d["grad_L_XQW_mini_batch"], cgs)

    with torch.no_grad():
        for _ in range(warmup):
            once()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            once()
            ts.append(time.perf_counter() - t0)
    sec = statistics.median(ts)
    tokens = sample_B * NC * 64 * (sample_H / H_full)
    return tokens / sec, sec, statistics.mean(ts)


def run_reference(args, rank, world):
    """The reference arm: its own CPU statement of the path (the oracle), all host threads.  One step is
    one forward + backward over a bounded sample of the workload (one batch element, all heads when that
    fits the time budget, fewer heads otherwise); exactly --warmup + --steps of them are run."""
    if rank != 0:
        return None
    B, H, NC, cgs, desc = WORKLOADS[args.workload]
    threads = os.cpu_count() or 1
    K, W = max(1, args.steps), max(0, args.warmup)
    # size the sample so that K + W steps take about two minutes: one token-head costs about 25 us of this
    # oracle on 16 cores (measured: 5-6 k tokens/s at H = 32)
    budget_s = 120.0
    est_per_head = NC * 64 * 25e-6 * (16.0 / max(1, min(threads, 16)))
    sH = int(max(1, min(H, budget_s / ((K + W) * est_per_head))))
    sB = 1
    rate, sec, mean_sec = cpu_oracle_rate(sB, sH, NC, cgs, H, reps=K, threads=threads, warmup=W)
    sample = (f"PyTorch-eager fp32 oracle, fwd + hand-derived bwd; one step = the slice B={sB} H={sH} of the "
              f"workload's B={B} H={H} at full sequence (NC={NC}); tokens/s = slice token-heads/s / {H}")
    return {
        "impl": "reference", "metric": "ttt_mlp_fwd_bwd_tokens_per_s", "value": rate, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": mean_sec * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "B": B, "H": H, "seq_len": NC * 64, "checkpoint_group_size": cgs,
                   "sample_per_step": f"B={sB} H={sH} of B={B} H={H}"},
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def run_glue(args):
    """The layer-side kernels around the operator at the forward+backward configuration's shape: token
    layout transforms (four tensors per launch), eta gate and its backward, output norm fused with the
    unpack and its backward fused with the pack.  HBM-bound byte movers: achieved = algorithmic bytes (input + output) / device time, against
    the measured copy bandwidth.  One step = all six calls."""
    from ttt_tk_b200 import glue, layout
    B, H, NC, _, desc = WORKLOADS["glue"]
    T = NC * 64
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    xs = [torch.randn(B, T, H * 64, device=dev, generator=g).bfloat16() for _ in range(4)]
    ys = layout.pack_tokens(*xs)
    logits = torch.randn(B, T, H, device=dev, generator=g).bfloat16()
    d_eta = torch.randn(B, H, NC, 64, device=dev, generator=g).bfloat16()
    gamma = 1 + 0.1 * torch.randn(H * 64, device=dev, generator=g)
    beta = 0.1 * torch.randn(H * 64, device=dev, generator=g)
    tok = xs[0].numel() * 2
    _, stats = glue.unpack_layernorm(ys[0], gamma, beta, 1e-6, return_stats=True)
    cases = [("pack_tokens x4", lambda: layout.pack_tokens(*xs), 2 * 4 * tok),
             ("unpack_tokens x4", lambda: layout.unpack_tokens(*ys), 2 * 4 * tok),
             ("eta_gate", lambda: glue.eta_gate(logits, 0.1 / 64), 2 * logits.numel() * 2),
             ("eta_gate_backward", lambda: glue.eta_gate_backward(logits, d_eta, 0.1 / 64), 3 * logits.numel() * 2),
             ("unpack_layernorm", lambda: glue.unpack_layernorm(ys[0], gamma, beta, 1e-6), 2 * tok + 2 * H * 64 * 4),
             # backward: one pass reads x and dy, writes dx and accumulates the parameter gradients
             ("pack_layernorm_backward", lambda: glue.pack_layernorm_backward(xs[1], ys[0], gamma, stats), 3 * tok)]
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(0)
    out = {}
    total_ms = 0.0
    sampler.start()
    for name, fn, nbytes in cases:
        for _ in range(W):
            fn()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
        ev[0].record()
        for i in range(K):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(K))
        out[name] = {"us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6}
        total_ms += ms
    clocks = sampler.stop()
    pk, pk_src = peaks()
    for v in out.values():
        v["frac_of_hbm_peak"] = v["gbs"] / pk["hbm_gbs"]
    dom = out["pack_tokens x4"]
    total_bytes = sum(v["bytes"] for v in out.values())
    return {
        "metric": "ttt_layer_glue_gb_per_s", "value": total_bytes / total_ms / 1e6, "unit": "GB/s", "n_gpus": 1,
        "steps": K, "warmup": W, "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "B": B, "T": T, "H": H,
                   "l2": "every tensor (268 MB) exceeds the 126 MB L2 except the eta tensors (2 MB each)"},
        "kernels": out,
        "roofline": {"kernel": "layout_kernel<pack>", "bound": "hbm", "achieved": dom["gbs"], "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": dom["gbs"] / pk["hbm_gbs"], "traffic": None,
                     "peak_source": f"{pk_src} copy bandwidth"},
        "gpu_launches": len(cases) * K, "clocks": clocks,
    }


def run_linear(args):
    """The TTT-Linear forward (the operator with a one-layer inner model): 3 x 2*64^3 FLOP against 514 bytes per
    token-head, 48 FLOP per byte, far below the ridge: HBM is the roofline.  achieved = algorithmic bytes
    (Q, K, V, eta in, Out out, initial state, checkpoints) / device time, against the measured copy bandwidth."""
    from ttt_tk_b200 import ttt_linear_forward, take_status
    B, H, NC, cgs, desc = WORKLOADS[args.workload]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    n = -(-NC // cgs)
    XQ, XK, XV = (rn(B, H, NC, 64, 64).bfloat16() for _ in range(3))
    eta = (0.1 * torch.sigmoid(rn(B, H, NC, 64)) / 64).bfloat16()
    gamma, beta = 1 + 0.02 * rn(1, H, 1, 64), 0.02 * rn(1, H, 1, 64)
    W1, b1 = 0.02 * rn(B, H, 64, 64), 0.02 * rn(B, H, 1, 64)
    ck = [torch.empty(B, H, n, 64, 64, device=dev), torch.empty(B, H, n, 1, 64, device=dev)]
    out = torch.empty_like(XQ)
    fn = lambda: ttt_linear_forward(XQ, XK, XV, eta, gamma, beta, W1, b1, *ck, out, cgs)
    # the backward of the same problem, timed separately (reported under "kernels")
    from ttt_tk_b200 import ttt_linear_backward
    from ttt_tk_b200.ops import linear_backward_scratch_bytes
    go = rn(B, H, NC, 64, 64).bfloat16()
    gW, gb = 1e-3 * rn(B, H, 64, 64), 1e-3 * rn(B, H, 1, 64)
    scratch = torch.empty(linear_backward_scratch_bytes(B, H, cgs), dtype=torch.uint8, device=dev)
    bouts = [torch.empty(B, H, 1, 64, device=dev), torch.empty(B, H, 1, 64, device=dev), torch.empty(B, H, 64, 64, device=dev),
             torch.empty(B, H, 1, 64, device=dev), torch.empty(B, H, NC, 64, device=dev, dtype=torch.bfloat16),
             torch.empty_like(XQ), torch.empty_like(XQ), torch.empty_like(XQ)]
    bfn = lambda: ttt_linear_backward(XQ, XK, XV, eta, gamma, beta, *ck, gW, gb, go, *bouts, cgs, scratch=scratch)
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(W):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        fn()
    e1.record()
    torch.cuda.synchronize()
    for _ in range(W):
        bfn()
    torch.cuda.synchronize()
    b0, b1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    b0.record()
    for _ in range(K):
        bfn()
    b1e.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if take_status() != 0:
        raise RuntimeError("a device-side wait ran out")
    ms = e0.elapsed_time(e1) / K
    bwd_ms = b0.elapsed_time(b1e) / K
    # backward: Q, K, V, eta, dOut in; dQ, dK, dV, d_eta out; checkpoints; state gradients in and out
    bwd_bytes = B * H * (NC * 64 * 900 + (n + 2) * (64 * 64 + 64) * 4 + 1024)
    bwd_scratch = B * H * NC * 2 * 33280         # every slot written once and read once
    state = (64 * 64 + 64) * 4
    nbytes = B * H * (NC * 64 * 514 + state + 512 + n * state)
    flops = B * H * NC * 3 * 2 * 64 ** 3
    pk, pk_src = peaks()
    gbs = nbytes / ms / 1e6
    return {
        "metric": "ttt_linear_fwd_bwd_tokens_per_s", "value": B * NC * 64 / ((ms + bwd_ms) * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms + bwd_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "B": B, "H": H, "seq_len": NC * 64, "checkpoint_group_size": cgs,
                   "l2": "inputs + outputs per step exceed the 126 MB L2; no explicit flush"},
        "kernels": {"fwd_ms": ms, "fwd_tflops": flops / (ms * 1e-3) / 1e12, "fwd_algorithmic_gbs": gbs,
                    "fwd_frac_of_hbm_peak": gbs / pk["hbm_gbs"],
                    # forward: three CTAs (streams) share an SM: 444 run at once on 148 SMs
                    "fwd_waves": -(-(B * H) // 444), "fwd_us_per_mini_batch_per_wave": ms * 1e3 / (NC * -(-(B * H) // 444)),
                    "bwd_ms": bwd_ms, "bwd_algorithmic_gbs": bwd_bytes / bwd_ms / 1e6,
                    "bwd_frac_of_hbm_peak": bwd_bytes / bwd_ms / 1e6 / pk["hbm_gbs"],
                    "bwd_gbs_with_scratch": (bwd_bytes + bwd_scratch) / bwd_ms / 1e6,
                    "bwd_waves": -(-(B * H) // 148), "bwd_us_per_mini_batch_per_wave": bwd_ms * 1e3 / (NC * -(-(B * H) // 148))},
        # the dominant kernel is the backward; both kernels are far below the ridge (48 FLOP per byte): HBM roofline
        "roofline": {"kernel": "ttt_linear_bwd_kernel", "bound": "hbm", "achieved": bwd_bytes / bwd_ms / 1e6,
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": bwd_bytes / bwd_ms / 1e6 / pk["hbm_gbs"], "traffic": None,
                     "peak_source": f"{pk_src} copy bandwidth"},
        "gpu_launches": 2 * K, "clocks": clocks,
    }


def linear_cpu_baseline(workload):
    """The TTT-Linear oracle (forward + hand-derived backward, PyTorch eager fp32) on all host cores, on a slice of
    the workload: one batch element, all heads, at most 32 mini-batches."""
    from oracle import ttt_linear as lin
    B, H, NC, cgs, _ = WORKLOADS[workload]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    nc = min(NC, 32)
    d = lin.make_inputs(1, H, nc, seed=0)
    g = torch.Generator().manual_seed(1)
    go = torch.randn(1, H, nc, 64, 64, generator=g)
    gW, gb = 1e-3 * torch.randn(1, H, 64, 64, generator=g), 1e-3 * torch.randn(1, H, 1, 64, generator=g)

    def once():
        f = lin.ttt_linear_forward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                                   d["W1"], d["b1"], cgs)
        lin.ttt_linear_backward(d["XQ"], d["XK"], d["XV"], d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"],
                                f["W1_checkpoints"], f["b1_checkpoints"], go, gW, gb, cgs)

    once()
    ts = []
    for _ in range(3):
        t0 = time.perf_counter()
        once()
        ts.append(time.perf_counter() - t0)
    sec = statistics.median(ts)
    return {"value": nc * 64 / sec, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"PyTorch-eager fp32 oracle, forward + backward, slice B=1 H={H} NC={nc}, median of 3 ({sec:.2f} s each)"}


def _emit(res, out_fd):
    os.write(out_fd, (json.dumps(res) + "\n").encode())


def main():
    # Libraries may write to stdout on their own (NCCL prints its version there); the one JSON line must
    # be the only thing on it, so everything else is sent to stderr and the line goes to the saved stdout.
    sys.stdout.flush()
    out_fd = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--e2e-head-chunks", type=int, default=1,
                    help="end-to-end step: split every batch element's heads into this many chunks")
    ap.add_argument("--e2e-batch-per-chunk", type=int, default=2,
                    help="end-to-end step: batch elements per chunk (with --e2e-head-chunks 1)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: partition the one problem's streams over the ranks (strong), or one whole problem per rank")
    ap.add_argument("--cluster", type=int, default=0, choices=[0, 1, 2, 4],
                    help="CTAs per (batch, head) stream; 0 = the launcher's own choice")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        res = run_reference(args, rank, world)
        if res is not None:
            _emit(res, out_fd)
        return

    if args.workload == "glue":
        if rank == 0:
            _emit(run_glue(args), out_fd)
        return
    if args.workload.startswith("linear"):
        if rank == 0:
            res = run_linear(args)
            if not args.no_cpu_baseline:
                res["cpu_baseline"] = linear_cpu_baseline(args.workload)
            _emit(res, out_fd)
        return

    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    res = run_ours(args, rank, world, local_rank)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            B, H, NC, cgs, _ = WORKLOADS[args.workload]
            threads = os.cpu_count() or 1
            sB, sH = 1, H      # one batch element, all heads (about 10-20 s of CPU work in total)
            rate, sec, _ = cpu_oracle_rate(sB, sH, NC, cgs, H, reps=3, threads=threads)
            res["cpu_baseline"] = {
                "value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": (f"PyTorch-eager fp32 oracle, fwd + hand-derived bwd, slice B={sB} H={sH} at full "
                           f"sequence (NC={NC}), median of 3 ({sec:.2f} s each); tokens/s = token-heads/s / {H}")}
        _emit(res, out_fd)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
