"""Split-K GEMM for skinny (decode) problems against an fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(80, 4096, 12288), (1, 4096, 4096), (128, 6144, 4096), (37, 1024, 2048), (64, 24576, 4096)])
def test_skinny_linear_splitk(M, N, K):
    from relax_b200.ops import cuda as C

    assert C.available()
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    ref = x.float() @ w.float().t()
    tol = 0.02 * math.sqrt(K) * 0.05 + 0.05
    with torch.no_grad():
        y = C.linear(x, w)
        assert (y.float() - ref).abs().max() < tol
        y2 = C.matmul_nt_skinny(x, w, b, r)
        assert (y2.float() - (ref + b.float() + r.float())).abs().max() < tol + 0.05
    splits, bn = C._load().gemm_splitk_plan(M, N, K)
    assert splits >= 1 and bn in (64, 128)
    C.check_error_flag()
