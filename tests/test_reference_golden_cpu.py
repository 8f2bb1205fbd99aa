"""Expectations taken from the reference's own unit tests (read as text) and restated here:
the same inputs must give the same answers in this framework."""
import math

import pytest
import torch

from ferrotorch_b200.ops import reference as R
from ferrotorch_b200.train import tensorboard as TB


def _inv_freq(dim, base, scaling=None):
    """Recover inv_freq from the tables: the angle at position 1 (all angles here are < pi)."""
    cos, sin = R.rope_tables(dim, 4, base, scaling)
    return torch.atan2(sin[1].double(), cos[1].double())


# ferrotorch-train/src/tensorboard.rs:568-593 (RFC 3720 vectors)
def test_crc32c_vectors():
    assert TB.crc32c(b"") == 0x00000000
    assert TB.crc32c(bytes(32)) == 0x8A9136AA
    assert TB.crc32c(bytes([0xFF] * 32)) == 0x62A8AB43
    assert TB.crc32c(bytes(range(32))) == 0x46DD794E
    assert TB.crc32c(b"abc") != TB.masked_crc(b"abc")


# ferrotorch-nn/src/transformer.rs:2165-2216
def test_rope_ntk_and_linear_inv_freq():
    dim, base, factor = 64, 10000.0, 4.0
    plain = _inv_freq(dim, base)
    ntk = _inv_freq(dim, base, {"type": "ntk", "factor": factor, "original_max": 2048})
    assert plain.numel() == 32 and abs(float(ntk[0] - plain[0])) < 1e-6      # highest frequency unchanged
    assert abs(float(ntk[31] / plain[31]) - 1.0 / factor) < 0.05            # lowest ~ linear interpolation
    cos, _ = R.rope_tables(8, 16, base, {"type": "linear", "factor": 2.0})
    cos_plain, _ = R.rope_tables(8, 16, base)
    assert torch.allclose(cos[2::2], cos_plain[1:8], atol=1e-6)              # position p/2


# ferrotorch-nn/src/transformer.rs:2219-2245 and the schedule at :357-392
def test_rope_yarn_inv_freq_piecewise_and_exact_schedule():
    dim, base, factor, orig = 64, 10000.0, 4.0, 2048
    plain = _inv_freq(dim, base)
    yarn = _inv_freq(dim, base, {"type": "yarn", "factor": factor, "original_max": orig})
    assert abs(float(yarn[0] - plain[0])) < 1e-6
    assert abs(float(yarn[31] / (plain[31] / factor)) - 1.0) < 0.1

    def corr(n_rot):
        return dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))

    low, high = max(math.floor(corr(32.0)), 0.0) / 2.0, min(math.ceil(corr(1.0)), dim - 1) / 2.0
    want = []
    for i in range(dim // 2):
        p = base ** (2.0 * i / dim)
        t = min(max((i - low) / (0.001 if high == low else high - low), 0.0), 1.0)
        want.append((1.0 / (factor * p)) * t + (1.0 / p) * (1.0 - t))
    assert torch.allclose(yarn, torch.tensor(want, dtype=torch.float64), rtol=2e-5, atol=1e-9)
    # no attention temperature in the reference's YaRN: cos(0) stays exactly 1
    cos, _ = R.rope_tables(dim, 4, base, {"type": "yarn", "factor": factor, "original_max": orig})
    assert float(cos[0].max()) == 1.0
    cos_hf, _ = R.rope_tables(dim, 4, base, {"type": "yarn", "factor": factor, "original_max": orig, "mscale": True})
    assert float(cos_hf[0, 0]) == pytest.approx(0.1 * math.log(factor) + 1.0)


# ferrotorch-nn/src/transformer.rs:2068-2080: position zero is the identity for both conventions
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_position_zero_is_identity(interleaved):
    from ferrotorch_b200.ops import functional as F

    cos, sin = R.rope_tables(8, 16, 10000.0)
    x = torch.randn(1, 1, 2, 8)
    y = F.rope_(x.clone(), cos, sin, n_rot_heads=2, seq_len=1, interleaved=interleaved)
    assert torch.allclose(y, x, atol=1e-7)
