"""tcgen05 building blocks against a host matmul: every operand form the TTT kernels use."""
import ctypes

import pytest
import torch

from ttt_tk_b200 import _lib

pytestmark = pytest.mark.gpu

CASES = [
    # M,  N,  K, a_mn, b_mn, neg, repeat     used by
    (128, 64, 64, 0, 0, 0, 1),   # Z1^T = W1^T K^T ; R^T = W2 U2^T
    (128, 64, 64, 0, 1, 0, 1),   # state update: A K-major, B token tile read MN-major
    (128, 64, 64, 0, 1, 1, 2),   # negated A, accumulation across calls
    (64, 64, 256, 1, 1, 0, 1),   # Z2 = X2 W2 (both operands MN-major, M = 64)
    (64, 64, 64, 0, 0, 0, 1),    # M = 64 tensor-memory lane mapping, K-major
    (128, 64, 256, 1, 1, 0, 1),  # MN-major A spanning two 64-blocks (leading byte offset)
    (128, 128, 128, 0, 0, 0, 1),
    (64, 64, 256, 1, 1, 0, 1 | 256),   # same product, result read back as 16x256b fragments
    (64, 64, 64, 0, 0, 1, 2 | 256),
    (64, 64, 64, 0, 1, 0, 1 | 256),    # 64-row block of the cluster-sharded kernels: state update form at M = 64
    (64, 8, 64, 1, 0, 0, 1),           # column sums of a token tile on the tensor pipe: A = the tile read MN-major, B = 8 rows of ones
]


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,neg,rep", CASES)
def test_umma_forms(M, N, K, a_mn, b_mn, neg, rep):
    lib = _lib.lib()
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K + a_mn * 2 + b_mn)
    A = torch.randn(M, K, generator=g).bfloat16().float().cuda()
    B = torch.randn(N, K, generator=g).bfloat16().float().cuda()
    D = torch.full((M, N), float("nan"), device="cuda")
    rc = lib.ttt_b200_umma_selftest(A.data_ptr(), B.data_ptr(), D.data_ptr(), M, N, K, a_mn, b_mn, neg, rep,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.ttt_b200_last_error()
    torch.cuda.synchronize()
    want = (A.double() @ B.double().T) * (rep & 0xff) * (-1 if neg else 1)
    err = (D.double() - want).abs().max().item()
    assert err < 1e-3 * K ** 0.5, f"max abs err {err}"
