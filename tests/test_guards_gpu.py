"""Kernels write inside their outputs and nowhere else (canary zones), write all of it (poison), and
give the same bits twice.  New as a test, so its first GPU run is opt-in."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 136, 192), (1, 8, 64), (333, 1000, 128)])
def test_gemm_stays_inside_its_output(m, n, k):
    from ferrotorch_b200.ops import functional as F
    from ferrotorch_b200.utils import guards as G

    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    g = G.GuardedBuffer((m, n), torch.bfloat16, "cuda")
    F.gemm_nt(a, b, out=g.view)
    torch.cuda.synchronize()
    g.check(fully_written=True)
    torch.testing.assert_close(g.view.float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-1)
    G.run_twice_bitwise(lambda: F.gemm_nt(a, b))


def test_inplace_rope_and_norm_are_contained_and_deterministic():
    from ferrotorch_b200.ops import functional as F
    from ferrotorch_b200.ops import reference as R
    from ferrotorch_b200.utils import guards as G

    torch.manual_seed(1)
    x = torch.randn(2, 37, 8, 64, device="cuda", dtype=torch.bfloat16)
    cos, sin = (t.cuda() for t in R.rope_tables(64, 128, 10000.0, None))
    g = G.guarded_like(x)
    F.rope_(g.view, cos, sin, seq_len=37)
    torch.cuda.synchronize()
    g.check()
    h = torch.randn(75, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    G.run_twice_bitwise(lambda: F.rmsnorm(h, w, 1e-5))
