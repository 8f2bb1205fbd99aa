"""Explicit begin / end graph capture and private pools on a device (first GPU run is opt-in)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_capture_guard_replays():
    from ferrotorch_b200 import cuda as C

    C.init_cuda_backend(0)
    x = torch.ones(1024, device="cuda")
    y = torch.zeros_like(x)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            y.copy_(x * 2 + 1)                                   # warm-up outside capture
    torch.cuda.current_stream().wait_stream(s)
    pool = C.GraphPoolHandle()
    guard = C.begin_capture_with_pool_mode(pool, C.CaptureMode.ThreadLocal)
    assert C.capture_status() is C.CaptureStatus.Active
    y.copy_(x * 2 + 1)
    graph = C.end_capture(guard)
    assert C.capture_status() is C.CaptureStatus.NotCapturing
    x.fill_(5.0)
    graph.launch()
    torch.cuda.synchronize()
    assert graph.num_replays == 1 and torch.equal(y, torch.full_like(y, 11.0))
    captured, out = C.capture_into_private_pool(lambda t: t * 3, x, pool=pool)
    x.fill_(2.0)
    captured.launch()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full_like(out, 6.0))
    C.release_graph_pool_handle(pool)
