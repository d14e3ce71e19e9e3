"""Out-of-bounds evidence without a sanitizer: every caller-owned buffer the kernels write (outputs,
checkpoints, final state, all sixteen scratch tensors) and every input sits between two guard zones
filled with a known byte pattern; after the forward and the backward the zones must be untouched and
the inputs unchanged.  The kernels store scratch as raw bulk copies at computed slot offsets, so an
off-by-one slot or a mis-sized image would land in a guard zone."""
import pytest
import torch

from oracle import ttt_mlp as orc
from ttt_tk_b200 import ttt_forward, ttt_backward, take_status
from ttt_tk_b200.buffers import GRAD_NAMES

pytestmark = pytest.mark.gpu
GUARD = 8192          # bytes on either side (one 64 x 64 bf16 tile)
PATTERN = 0xA5


class Guarded:
    """Tensors carved out of byte buffers with guard zones before and after each of them."""

    def __init__(self, dev):
        self.dev = dev
        self.items = []

    def make(self, shape, dtype, src=None, fill=None):
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        pad = (-nbytes) % 256
        raw = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device=self.dev)
        view = raw[GUARD:GUARD + nbytes].view(dtype).view(*shape)
        if src is not None:
            view.copy_(src)
        elif fill is not None:
            view.fill_(fill)
        self.items.append((raw, nbytes, src.clone() if src is not None else None, view))
        return view

    def check(self, what):
        for i, (raw, nbytes, src, view) in enumerate(self.items):
            assert bool((raw[:GUARD] == PATTERN).all()), f"{what}: bytes before buffer {i} were overwritten"
            assert bool((raw[GUARD + nbytes:] == PATTERN).all()), f"{what}: bytes after buffer {i} were overwritten"
            if src is not None:
                assert torch.equal(view.cpu(), src.cpu()), f"{what}: input buffer {i} was modified"


@pytest.mark.parametrize("cluster", [1, 2, 4])
@pytest.mark.parametrize("B,H,NC,cgs", [(1, 2, 3, 2), (2, 1, 5, 4)])
def test_forward_and_backward_stay_inside_their_buffers(cluster, B, H, NC, cgs):
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32
    d = orc.make_inputs(B, H, NC, seed=13, backward=True)
    n = orc.num_checkpoints(NC, cgs)
    G = Guarded(dev)
    t = {k: G.make(tuple(v.shape), v.dtype, src=v.to(dev)) for k, v in d.items()}
    nan = float("nan")
    ck = [G.make((B, H, n, *s), f32, fill=nan) for s in ((64, 256), (1, 256), (256, 64), (1, 64))]
    fin = tuple(G.make((B, H, *s), f32, fill=nan) for s in ((64, 256), (1, 256), (256, 64), (1, 64)))
    out = G.make((B, H, NC, 64, 64), bf, fill=nan)
    ttt_forward(t["XQ"], t["XK"], t["XV"], t["last_eta"], t["ttt_norm_weight"], t["ttt_norm_bias"],
                t["W1"], t["b1"], t["W2"], t["b2"], *ck, out, cgs, final_state=fin, cluster=cluster)
    torch.cuda.synchronize()
    assert take_status() == 0
    G.check(f"forward, {cluster} CTA(s) per stream")
    for x in ck + list(fin) + [out]:
        assert torch.isfinite(x.float()).all()

    # backward: the checkpoints and Out are inputs now (checked for modification through a second registry)
    G2 = Guarded(dev)
    ck_in = [G2.make(tuple(c.shape), f32, src=c) for c in ck]
    out_in = G2.make(tuple(out.shape), bf, src=out)
    t2 = {k: G2.make(tuple(v.shape), v.dtype, src=v.to(dev)) for k, v in d.items()}
    eta5 = G2.make((B, H, NC, 64, 1), bf, src=d["last_eta"].unsqueeze(-1).to(dev))
    g = cgs
    scratch_shapes = [((B, H, g, 64, 256), f32), ((B, H, g, 1, 256), f32), ((B, H, g, 256, 64), f32), ((B, H, g, 1, 64), f32),
                      ((B, H, g, 64, 64), bf), ((B, H, g, 64, 1), f32),
                      ((B, H, g, 64, 256), bf), ((B, H, g, 64, 256), bf), ((B, H, g, 64, 256), bf), ((B, H, g, 64, 256), bf),
                      ((B, H, g, 64, 64), bf), ((B, H, g, 64, 256), bf), ((B, H, g, 64, 64), bf),
                      ((B, H, g, 64, 64), bf), ((B, H, g, 64, 64), bf), ((B, H, g, 64, 1), f32)]
    scratch = [G2.make(s, dt, fill=0.0) for s, dt in scratch_shapes]
    out_shapes = {"grad_L_ttt_norm_weight": ((B, H, 1, 64), f32), "grad_L_ttt_norm_bias": ((B, H, 1, 64), f32),
                  "grad_L_W1_init": ((B, H, 64, 256), f32), "grad_L_b1_init": ((B, H, 1, 256), f32),
                  "grad_L_W2_init": ((B, H, 256, 64), f32), "grad_L_b2_init": ((B, H, 1, 64), f32),
                  "grad_L_last_eta": ((B, H, NC, 64, 1), bf), "grad_L_XQ": ((B, H, NC, 64, 64), bf),
                  "grad_L_XK": ((B, H, NC, 64, 64), bf), "grad_L_XV": ((B, H, NC, 64, 64), bf)}
    outs = {k: G2.make(s, dt, fill=nan) for k, (s, dt) in out_shapes.items()}
    ttt_backward(t2["XQ"], t2["XK"], t2["XV"], eta5, t2["ttt_norm_weight"], t2["ttt_norm_bias"], *ck_in, out_in,
                 *scratch, t2["grad_L_W1_last"], t2["grad_L_b1_last"], t2["grad_L_W2_last"], t2["grad_L_b2_last"],
                 t2["grad_L_XQW_mini_batch"], *[outs[k] for k in GRAD_NAMES], cgs, cluster=cluster)
    torch.cuda.synchronize()
    assert take_status() == 0
    G2.check(f"backward, {cluster} CTA(s) per stream")
    for k in GRAD_NAMES:
        assert torch.isfinite(outs[k].float()).all(), k
