"""Generate tests/golden/ttt_mlp_golden.npz from the REFERENCE's own PyTorch functions.

Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/reference

It loads kernels/ttt/matching.py and kernels/ttt_backward/matching.py from that tree
(with an empty stand-in for the CUDA extension they import at line 2, which the math
functions never touch), drives `compute_mini_batch_no_dual` and `backward` with the
same loops as the scripts' `main()` (kernels/ttt/matching.py:219-252,
kernels/ttt_backward/matching.py:539-663) on seeded inputs, and stores the results.
The fixture pins the oracle on machines that do not have the reference tree.
"""
import importlib.util
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ttt_mlp as orc  # noqa: E402  (only for the seeded input recipe)

CASES = {
    # name: (B, H, NC, cgs, seed, eta_scale)
    "ragged": (1, 2, 3, 2, 0, 0.1),     # NC % cgs != 0 -> ragged last group
    "even": (2, 1, 2, 1, 1, 1.0),       # batch > 1, large eta, a checkpoint per mini-batch
}


def load_reference(ref_root):
    sys.modules.setdefault("test_time_training", types.ModuleType("test_time_training"))
    mods = []
    for name, rel in (("ref_fwd", "kernels/ttt/matching.py"),
                      ("ref_bwd", "kernels/ttt_backward/matching.py")):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        mods.append(m)
    return mods


def eta_matrix(last_eta_mb):
    """The reference functions take a [B,H,64,64] eta and use only its last row."""
    B, H, CS = last_eta_mb.shape
    e = torch.zeros(B, H, CS, CS, dtype=last_eta_mb.dtype)
    e[:, :, -1, :] = last_eta_mb
    return e


def run_reference(ref_fwd, ref_bwd, d, cgs):
    f32 = lambda t: t.to(torch.float32)
    XQ, XK, XV, eta = f32(d["XQ"]), f32(d["XK"]), f32(d["XV"]), f32(d["last_eta"])
    gam, bet = d["ttt_norm_weight"], d["ttt_norm_bias"]
    B, H, NC = XQ.shape[:3]
    n = math.ceil(NC / cgs)
    out = {}
    # ---- forward, reference loop (kernels/ttt/matching.py:219-252)
    W1, b1, W2, b2 = d["W1"], d["b1"], d["W2"], d["b2"]
    Out = torch.empty_like(XQ)
    ck = [torch.empty(B, H, n, *s) for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
    for i in range(NC):
        if i % cgs == 0:
            for t, v in zip(ck, (W1, b1, W2, b2)):
                t[:, :, i // cgs] = v
        Out[:, :, i], W1, b1, W2, b2 = ref_fwd.compute_mini_batch_no_dual(
            W1, b1, W2, b2, XQ[:, :, i], XK[:, :, i], XV[:, :, i], eta_matrix(eta[:, :, i]), gam, bet)
    out["Out"] = Out
    for k, t in zip(("W1_checkpoints", "b1_checkpoints", "W2_checkpoints", "b2_checkpoints"), ck):
        out[k] = t
    for k, t in zip(("W1_final", "b1_final", "W2_final", "b2_final"), (W1, b1, W2, b2)):
        out[k] = t
    # ---- backward, reference loop (kernels/ttt_backward/matching.py:539-663)
    gW1, gb1, gW2, gb2 = (d["grad_L_W1_last"].clone(), d["grad_L_b1_last"].clone(),
                          d["grad_L_W2_last"].clone(), d["grad_L_b2_last"].clone())
    go = f32(d["grad_L_XQW_mini_batch"])
    dXQ, dXK, dXV = torch.empty_like(XQ), torch.empty_like(XQ), torch.empty_like(XQ)
    dEta = torch.empty(B, H, NC, 64, 1)
    # the reference sums the norm grads over the batch inside backward(); run it one batch
    # element at a time so that the per-batch rows the operator writes are pinned too
    dG = torch.zeros(B, H, 1, 64)
    dB = torch.zeros(B, H, 1, 64)
    for b in range(B):
        sl = slice(b, b + 1)
        G = [gW1[sl].clone(), gb1[sl].clone(), gW2[sl].clone(), gb2[sl].clone()]
        for c in range(n - 1, -1, -1):
            cur = [t[sl, :, c] for t in ck]
            saved = {}
            for j in range(cgs):
                i = c * cgs + j
                if i >= NC:
                    continue
                init = list(cur)
                r = ref_bwd.compute_mini_batch_no_dual(
                    *cur, XQ[sl, :, i], XK[sl, :, i], XV[sl, :, i], eta_matrix(eta[sl, :, i]), gam, bet)
                cur = list(r[:4])
                saved[j] = (init, r[4:])
            for j in range(cgs - 1, -1, -1):
                i = c * cgs + j
                if i >= NC:
                    continue
                init, (Z1, std_f, xh_f, go_f, gxh_f, gZ2, gZ1, X2, Z1b, X2b, std_ln, xh_ln) = saved[j]
                r = ref_bwd.backward(
                    XQ[sl, :, i], XK[sl, :, i], Z1, init[0], init[1], init[2], init[3], cur[2], cur[0],
                    gam, bet, std_f, xh_f, go_f, gxh_f, gZ2, gZ1, eta_matrix(eta[sl, :, i]), X2, Z1b, X2b,
                    std_ln, xh_ln, gam, bet, G[0], G[1], G[2], G[3], go[sl, :, i])
                dG[b] += r[0].reshape(H, 1, 64)
                dB[b] += r[1].reshape(H, 1, 64)
                G = [r[2], r[3], r[4], r[5]]
                dXQ[sl, :, i], dXV[sl, :, i], dXK[sl, :, i] = r[6], r[7], r[8]
                # r[9] is the zero-padded eta-matrix gradient; its last row is d last_eta
                dEta[sl, :, i] = r[9][:, :, -1, :, None]
                cur = init
        gW1[sl], gb1[sl], gW2[sl], gb2[sl] = G
    out.update({"grad_L_ttt_norm_weight": dG, "grad_L_ttt_norm_bias": dB,
                "grad_L_W1_init": gW1, "grad_L_b1_init": gb1, "grad_L_W2_init": gW2, "grad_L_b2_init": gb2,
                "grad_L_last_eta": dEta, "grad_L_XQ": dXQ, "grad_L_XK": dXK, "grad_L_XV": dXV})
    return out


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "TTT_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))
    ref_fwd, ref_bwd = load_reference(ref_root)
    blob = {}
    with torch.no_grad():
        for name, (B, H, NC, cgs, seed, es) in CASES.items():
            d = orc.make_inputs(B, H, NC, seed=seed, eta_scale=es, backward=True)
            res = run_reference(ref_fwd, ref_bwd, d, cgs)
            blob[f"{name}/cfg"] = np.array([B, H, NC, cgs, seed], dtype=np.int64)
            blob[f"{name}/eta_scale"] = np.array([es], dtype=np.float64)
            # input fingerprint: guards against generator drift between machines
            blob[f"{name}/input_sum"] = np.array(
                [float(v.double().sum()) for v in d.values()], dtype=np.float64)
            for k, v in res.items():
                blob[f"{name}/{k}"] = v.numpy().astype(np.float32)
    path = os.path.join(HERE, "ttt_mlp_golden.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
