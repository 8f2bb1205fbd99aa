"""Canary / poison / run-twice checks: they must catch what they claim to catch."""
import pytest
import torch

from ferrotorch_b200.utils import guards as G


def test_clean_kernel_passes_and_overrun_is_caught():
    g = G.GuardedBuffer((5, 7), torch.bfloat16)
    assert g.view.shape == (5, 7) and g.view.dtype == torch.bfloat16 and g.unwritten_bytes() == 70 and g.canaries_intact()
    with pytest.raises(G.GuardViolation, match="unwritten"):
        g.check(fully_written=True)
    g.view.copy_(torch.randn(5, 7))
    g.check(fully_written=True)
    g.raw[g.pad + g.nbytes + 3] = 0                                  # one byte past the end, inside the alignment slack
    with pytest.raises(G.GuardViolation, match="offset 73"):
        g.check()
    h = G.GuardedBuffer((16,), torch.float32)
    h.view.fill_(1.0)
    h.raw[h.pad - 1] = 7                                             # one byte before the start
    assert h.first_violation() == -1 and not h.canaries_intact()
    with pytest.raises(ValueError):
        G.GuardedBuffer((4,), pad=100)


def test_partial_write_and_inplace_form():
    g = G.GuardedBuffer((8, 8), torch.float32)
    g.view[:, :7] = 0.5                                              # a kernel that forgets the last column
    with pytest.raises(G.GuardViolation, match="unwritten"):
        g.check(fully_written=True)
    g.check()                                                        # but it stayed inside its output
    x = torch.randn(3, 4)
    gi = G.guarded_like(x)
    gi.view.mul_(2.0)
    gi.check(fully_written=True)
    torch.testing.assert_close(gi.view, x * 2)


def test_run_twice_bitwise():
    x = torch.randn(64)
    assert torch.equal(G.run_twice_bitwise(lambda t: (t * 2, [t + 1]), x)[0], x * 2)
    state = {"n": 0}

    def flaky(t):
        state["n"] += 1
        return t + (1e-7 if state["n"] == 2 else 0.0)

    with pytest.raises(G.GuardViolation, match="differs"):
        G.run_twice_bitwise(flaky, torch.ones(8))
    G.run_twice_bitwise(lambda t: torch.full_like(t, float("nan")), x)   # NaN payloads compare by bits, not by value
