"""Token layout transforms: bit-exact against torch's permute, through the C ABI."""
import pytest
import torch

from ttt_tk_b200.layout import pack_tokens, unpack_tokens

pytestmark = pytest.mark.gpu


def _ref_pack(x, H):
    B, T = x.shape[:2]
    return x.view(B, T, H, 64).permute(0, 2, 1, 3).contiguous().view(B, H, T // 64, 64, 64)


@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (2, 128, 3), (1, 192, 12), (4, 2048, 32), (3, 64, 24)])
def test_pack_and_unpack_are_permutations(B, T, H):
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + T + H)
    xs = [torch.randn(B, T, H * 64, device="cuda", generator=g).bfloat16() for _ in range(3)]
    ys = pack_tokens(*xs)
    for x, y in zip(xs, ys):
        assert y.shape == (B, H, T // 64, 64, 64)
        assert torch.equal(y, _ref_pack(x, H))
    zs = unpack_tokens(*ys)
    for x, z in zip(xs, zs):
        assert torch.equal(z, x)


def test_single_tensor_rank4_and_four_tensors():
    x = torch.randn(2, 128, 5, 64, device="cuda").bfloat16()
    (y,) = pack_tokens(x)
    assert torch.equal(y, _ref_pack(x.view(2, 128, 320), 5))
    four = [torch.randn(1, 64, 128, device="cuda").bfloat16() for _ in range(4)]
    out = pack_tokens(*four)
    assert all(torch.equal(o, _ref_pack(f, 2)) for o, f in zip(out, four))


def test_rejects_bad_arguments():
    x = torch.randn(1, 64, 64, device="cuda").bfloat16()
    with pytest.raises(ValueError):
        pack_tokens(x.float())
    with pytest.raises(ValueError):
        pack_tokens(torch.randn(1, 96, 64, device="cuda").bfloat16())        # T not a multiple of 64
    with pytest.raises(ValueError):
        pack_tokens(torch.randn(1, 64, 96, device="cuda").bfloat16())        # features not H*64
    with pytest.raises(ValueError):
        pack_tokens(x, x, x, x, x)
    with pytest.raises(ValueError):
        unpack_tokens(torch.randn(1, 1, 2, 64, 32, device="cuda").bfloat16())


def test_feeds_the_operator():
    """pack -> forward -> unpack equals the forward on torch-permuted inputs."""
    from ttt_tk_b200 import ttt_forward
    from ttt_tk_b200.buffers import alloc_checkpoints
    from ttt_tk_b200.synthetic import make_inputs
    B, H, NC, cgs = 2, 3, 4, 2
    d = {k: v.cuda() for k, v in make_inputs(B, H, NC, seed=3).items()}
    tok = {k: d[k].view(B, H, NC * 64, 64).permute(0, 2, 1, 3).contiguous().view(B, NC * 64, H * 64)
           for k in ("XQ", "XK", "XV")}
    xq, xk, xv = pack_tokens(tok["XQ"], tok["XK"], tok["XV"])
    assert torch.equal(xq, d["XQ"]) and torch.equal(xk, d["XK"]) and torch.equal(xv, d["XV"])
    outs = []
    for q, k, v in ((xq, xk, xv), (d["XQ"], d["XK"], d["XV"])):
        ck = alloc_checkpoints(B, H, NC, cgs, "cuda")
        out = torch.empty_like(q)
        ttt_forward(q, k, v, d["last_eta"], d["ttt_norm_weight"], d["ttt_norm_bias"], d["W1"], d["b1"], d["W2"],
                    d["b2"], *ck, out, cgs, sync=True)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    (y,) = unpack_tokens(outs[0])
    assert torch.equal(y, outs[1].view(B, H, NC * 64, 64).permute(0, 2, 1, 3).reshape(B, NC * 64, H * 64))
