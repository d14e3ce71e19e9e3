"""The layer-side kernels around the operator against their torch statements (oracle/glue.py).

Tolerances (floating point): the kernels and the statement compute in fp32 and round once to bf16, so
results agree except where the two fp32 values straddle a bf16 rounding boundary: every element within
2 bf16 ulps (|diff| <= 2^-7 |ref| + 1e-6 abs for eta, + 2e-2 abs for the O(1) LayerNorm output) and at
least 99 % of the elements bit-identical; relative L2 <= 2e-3."""
import pytest
import torch

from oracle import glue as og
from oracle.ttt_mlp import rel_l2
from ttt_tk_b200 import glue

pytestmark = pytest.mark.gpu


def close(got, ref, abs_tol):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert torch.isfinite(got).all()
    d = (got - ref).abs()
    assert bool((d <= ref.abs() * 2 ** -7 + abs_tol).all()), f"max diff {d.max().item():.3e}"
    assert (got == ref).float().mean().item() >= 0.99
    assert rel_l2(got, ref) <= 2e-3


@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (2, 128, 3), (2, 256, 32), (1, 192, 12)])
def test_eta_gate_and_its_backward(B, T, H):
    g = torch.Generator().manual_seed(B * 100 + T + H)
    logits = torch.randn(B, T, H, generator=g).bfloat16()
    scale = 0.1 / 64
    got = glue.eta_gate(logits.cuda(), scale)
    assert got.shape == (B, H, T // 64, 64)
    close(got, og.eta_gate(logits, scale), 1e-7)
    d_eta = torch.randn(B, H, T // 64, 64, 1, generator=g).bfloat16()
    got_b = glue.eta_gate_backward(logits.cuda(), d_eta.cuda(), scale)
    assert got_b.shape == (B, T, H)
    close(got_b, og.eta_gate_backward(logits, d_eta, scale), 1e-7)


@pytest.mark.parametrize("B,NC,H", [(1, 1, 1), (2, 2, 3), (1, 3, 32), (2, 1, 12), (1, 1, 64)])
def test_unpack_layernorm(B, NC, H):
    g = torch.Generator().manual_seed(B * 100 + NC * 10 + H)
    out = (torch.randn(B, H, NC, 64, 64, generator=g) * 1.5 + 0.3).bfloat16()
    gamma = 1 + 0.1 * torch.randn(H * 64, generator=g)
    beta = 0.1 * torch.randn(H * 64, generator=g)
    got = glue.unpack_layernorm(out.cuda(), gamma.cuda(), beta.cuda(), 1e-6)
    assert got.shape == (B, NC * 64, H * 64)
    close(got, og.unpack_layernorm(out, gamma, beta, 1e-6), 2e-2)


@pytest.mark.parametrize("B,NC,H", [(1, 1, 1), (2, 2, 3), (1, 5, 32), (2, 1, 12), (1, 1, 64), (1, 2, 38), (3, 9, 8)])
def test_pack_layernorm_backward(B, NC, H):
    g = torch.Generator().manual_seed(B * 100 + NC * 10 + H + 7)
    out = (torch.randn(B, H, NC, 64, 64, generator=g) * 1.5 + 0.3).bfloat16()
    gamma = 1 + 0.1 * torch.randn(H * 64, generator=g)
    beta = 0.1 * torch.randn(H * 64, generator=g)
    dy = torch.randn(B, NC * 64, H * 64, generator=g).bfloat16()
    y, stats = glue.unpack_layernorm(out.cuda(), gamma.cuda(), beta.cuda(), 1e-6, return_stats=True)
    close(y, og.unpack_layernorm(out, gamma, beta, 1e-6), 2e-2)
    d_out, d_gamma, d_beta = glue.pack_layernorm_backward(dy.cuda(), out.cuda(), gamma.cuda(), stats)
    r_out, r_gamma, r_beta = og.pack_layernorm_backward(dy, out, gamma, beta, 1e-6)
    assert d_out.shape == out.shape
    # the gradient has small entries next to O(1) ones: bf16 rounding of both sides, 2 ulps + a small absolute term
    close(d_out, r_out, 2e-3)
    # fp32 sums over B * T tokens in a different order (and with atomics): relative L2
    assert rel_l2(d_gamma.cpu(), r_gamma) <= 1e-4
    assert rel_l2(d_beta.cpu(), r_beta) <= 1e-4


def test_glue_rejects_bad_arguments():
    x = torch.zeros(1, 64, 2, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        glue.eta_gate(x.float(), 1.0)
    with pytest.raises(ValueError):
        glue.eta_gate(torch.zeros(1, 60, 2, dtype=torch.bfloat16, device="cuda"), 1.0)
    o = torch.zeros(1, 65, 1, 64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="64"):
        glue.unpack_layernorm(o, torch.ones(65 * 64, device="cuda"), torch.zeros(65 * 64, device="cuda"))
