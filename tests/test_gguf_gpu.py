"""Device-side GGUF dequantisation against the host reader (first GPU run is opt-in)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_every_quantised_type_matches_the_host_reader():
    from ferrotorch_b200.serialize import gguf as G

    g = torch.Generator().manual_seed(0)
    for t in (G.GGML_Q4_0, G.GGML_Q4_1, G.GGML_Q5_0, G.GGML_Q5_1, G.GGML_Q8_0, G.GGML_Q8_1):
        be, bb = G._BLOCK[t]
        rows, cols = 96, 256
        nblk = rows * cols // be
        raw = torch.randint(0, 256, (nblk, bb), dtype=torch.uint8, generator=g)
        raw[:, 0:2] = (torch.rand(nblk, generator=g) * 0.1 + 1e-3).to(torch.float16).view(torch.uint8).view(nblk, 2)
        if t in (G.GGML_Q4_1, G.GGML_Q5_1, G.GGML_Q8_1):
            raw[:, 2:4] = (torch.randn(nblk, generator=g) * 0.5).to(torch.float16).view(torch.uint8).view(nblk, 2)
        ref = G.dequantize_blocks(raw.reshape(-1), t, rows * cols).reshape(rows, cols)
        dev = raw.reshape(-1).cuda()
        f32 = G.dequantize_on_device(dev, t, (rows, cols), torch.float32)
        assert torch.equal(f32.cpu(), ref), "type %d" % t
        bf = G.dequantize_on_device(dev, t, (rows, cols), torch.bfloat16)
        assert torch.equal(bf.cpu(), ref.to(torch.bfloat16)), "type %d" % t
