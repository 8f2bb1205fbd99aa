"""Device Philox (csrc/rng.cu, ops/random.py) against the host generator of utils/philox.py."""
import ctypes

import numpy as np
import pytest
import torch

from ferrotorch_b200 import _native
from ferrotorch_b200.ops import random as R
from ferrotorch_b200.utils.philox import PhiloxGenerator


def test_device_function_compiled_for_the_host_equals_the_host_generator():
    # csrc/rng.cu's Philox rounds are one __host__ __device__ function; its host side must give the
    # stream of the C++ / numpy host generator word for word
    if _native._nvcc() is None and not _native.KERNELS_SO.exists():
        pytest.skip("kernels library not built on this machine")
    lib = _native.kernels(required=False)
    if lib is None:
        pytest.skip("kernels library not loadable on this machine")
    n = 4099
    out = np.empty(n, np.uint32)
    rc = lib.ft_philox_words_host(out.ctypes.data_as(ctypes.c_void_p), n, 0xDEADBEEFCAFE, 2 ** 40 + 17)
    assert rc == 0
    g = PhiloxGenerator(0xDEADBEEFCAFE)
    g.counter = 2 ** 40 + 17
    assert np.array_equal(out, g.words(n))


def test_cpu_generator_matches_host_stream_and_dropout_regenerates_its_mask():
    g, h = R.DevicePhilox(99, "cpu"), PhiloxGenerator(99)
    assert np.array_equal(g.words(1001).numpy(), h.words(1001).astype(np.int64))
    assert (g.counter, h.counter, h.offset) == (251, 250, 1)
    h.counter, h.offset = g.counter, 0             # a device draw always starts on a fresh counter
    assert np.array_equal(g.uniform(640).numpy(), h.generate_uniform(640))
    x = torch.randn(33, 65, requires_grad=True)
    gen = R.DevicePhilox(5, "cpu")
    y = R.dropout(x, 0.4, generator=gen)
    keep = R.keep_mask(x.numel(), 0.4, 5, 0).view(x.shape)
    torch.testing.assert_close(y, torch.where(keep, x / 0.6, torch.zeros(())))
    y.backward(torch.ones_like(y))
    torch.testing.assert_close(x.grad, keep.float() / 0.6)
    assert R.dropout(x, 0.4, training=False) is x


@pytest.mark.parametrize("n", [1, 3, 4, 5, 31, 32, 33, 70001, 300003])
def test_threaded_host_fill_follows_the_stream_of_the_scalar_generator(n):
    """The host library's fill (eight counters per trip, several threads above 32 K values) against
    the numpy form of the rounds: uniforms bitwise, normals to the rounding of log / sin / cos, for
    sizes around the group width and the thread split, and across the 2^32 counter carry."""
    start = 2 ** 32 - 7
    g = R.DevicePhilox(4242, "cpu")
    g.counter = start
    u = g.uniform(n, low=-1.0, high=3.0)
    assert g.counter == start + (n + 3) // 4
    ref = -1.0 + 4.0 * R._host_u01(n, 4242, start)
    assert torch.equal(u, ref)
    g.counter = start
    z = g.normal(n, mean=0.5, std=1.5)
    h = PhiloxGenerator(4242)
    h.counter = start
    zr = 0.5 + 1.5 * torch.from_numpy(h.generate_normal(4 * ((n + 3) // 4))[:n])
    torch.testing.assert_close(z, zr, rtol=0, atol=3e-6)
    g.counter = start
    zb = g.normal(n, mean=0.5, std=1.5, dtype=torch.bfloat16)          # other dtypes go through an fp32 buffer
    assert torch.equal(zb, z.to(torch.bfloat16))
    if n > 60000:
        assert abs(float(z.mean()) - 0.5) < 0.03 and abs(float(z.std()) - 1.5) < 0.03


@pytest.mark.gpu
def test_device_words_and_uniform_equal_the_host_generator_bitwise():
    n = 1 << 20
    g, h = R.DevicePhilox(2024, "cuda"), PhiloxGenerator(2024)
    w = g.words(n + 3)
    assert np.array_equal(w.cpu().numpy(), h.words(n + 3).astype(np.int64))
    h.counter, h.offset = g.counter, 0             # a device draw always starts on a fresh counter
    u = g.uniform(n)
    assert np.array_equal(u.cpu().numpy(), h.generate_uniform(n))
    assert _native.device_status(0) == 0


@pytest.mark.gpu
def test_device_normal_matches_host_box_muller():
    g, h = R.DevicePhilox(7, "cuda"), PhiloxGenerator(7)
    z = g.normal(1 << 16, mean=0.5, std=2.0)
    want = 0.5 + 2.0 * h.generate_normal(1 << 16)
    np.testing.assert_allclose(z.cpu().numpy(), want, rtol=1e-4, atol=1e-4)
    zb = R.DevicePhilox(7, "cuda").normal(4096, dtype=torch.bfloat16)
    assert abs(float(zb.float().mean())) < 0.1 and abs(float(zb.float().std()) - 1.0) < 0.1


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_device_dropout_forward_backward_against_host_mask(dtype):
    torch.manual_seed(0)
    x = torch.randn(257, 1031, device="cuda").to(dtype).requires_grad_()
    gen = R.DevicePhilox(31337, "cuda")
    gen.counter = 12345
    y = R.dropout(x, 0.2, generator=gen)
    keep = R.keep_mask(x.numel(), 0.2, 31337, 12345).view(x.shape).cuda()
    want = torch.where(keep, x.detach().float() * np.float32(1.25), torch.zeros((), device="cuda")).to(dtype)
    assert torch.equal(y, want)
    gy = torch.randn_like(y)
    y.backward(gy)
    want_g = torch.where(keep, gy.float() * np.float32(1.25), torch.zeros((), device="cuda")).to(dtype)
    assert torch.equal(x.grad, want_g)
    assert gen.counter == 12345 + (x.numel() + 3) // 4


@pytest.mark.gpu
def test_fused_swiglu_dropout_matches_unfused():
    from ferrotorch_b200.ops import functional as F

    torch.manual_seed(1)
    gu = (torch.randn(300, 2 * 1408, device="cuda")).to(torch.bfloat16).requires_grad_()
    gen = R.DevicePhilox(11, "cuda")
    y = R.swiglu_dropout(gu, 0.1, generator=gen)
    keep = R.keep_mask(300 * 1408, 0.1, 11, 0).view(300, 1408).cuda()
    g, u = gu.detach()[:, :1408].float(), gu.detach()[:, 1408:].float()
    want = torch.where(keep, torch.nn.functional.silu(g) * u / 0.9, torch.zeros((), device="cuda"))
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2)
    gy = torch.randn_like(y)
    y.backward(gy)
    ref = gu.detach().clone().requires_grad_()
    (F.swiglu(ref) * keep.to(torch.bfloat16) / 0.9).backward(gy)
    torch.testing.assert_close(gu.grad.float(), ref.grad.float(), rtol=3e-2, atol=3e-2)
    assert R.swiglu_dropout(gu, 0.0).shape == (300, 1408)
