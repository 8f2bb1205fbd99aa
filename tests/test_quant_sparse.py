"""Q4_0 dequant-GEMM and 2:4 sparse GEMM: packing round-trips on CPU, kernel numerics on GPU."""
import pytest
import torch

from ferrotorch_b200.ops import quant as Q
from ferrotorch_b200.ops import reference as R
from ferrotorch_b200.serialize.gguf import quantize_q4_0


def test_q4_planes_and_linear_cpu():
    torch.manual_seed(0)
    w = torch.randn(16, 128)
    blocks = quantize_q4_0(w)
    nib, sc = Q.q4_0_planes(blocks, 16, 128)
    assert nib.shape == (16, 64) and sc.shape == (16, 4) and sc.dtype == torch.float16
    deq = Q.dequant_q4_0_planes(nib, sc)
    assert torch.equal(deq, R.dequant_q4_0(blocks).view(16, 128))
    x = torch.randn(3, 128)
    assert torch.allclose(Q.q4_0_linear(x, nib, sc), x @ deq.t(), atol=1e-5)
    lin = torch.nn.Linear(128, 16)
    q = Q.Q4Linear.from_linear(lin)
    assert (q(x) - lin(x)).abs().max() < 0.5


def test_2_4_mask_pack_roundtrip_cpu():
    torch.manual_seed(1)
    w = torch.randn(8, 64)
    m = Q.apply_2_4_mask(w)
    assert ((m.view(-1, 4) != 0).sum(1) == 2).all()
    kept = m.view(-1, 4).abs().sum(1)
    assert torch.allclose(kept, w.view(-1, 4).abs().topk(2, dim=1).values.sum(1))
    v, meta = Q.pack_2_4(m)
    assert v.shape == (8, 32) and meta.shape == (8, 8) and meta.dtype == torch.uint8
    assert torch.equal(Q.unpack_2_4(v, meta), m)
    z = m.clone()
    z[0, :4] = 0                                     # an all-zero group still packs and unpacks
    assert torch.equal(Q.unpack_2_4(*Q.pack_2_4(z)), z)
    with pytest.raises(ValueError):
        Q.pack_2_4(w)
    x = torch.randn(5, 64)
    assert torch.allclose(Q.sparse24_linear(x, v, meta), x @ m.t(), atol=1e-5)
    q, s = Q.quantize_per_channel_int8(w)
    assert (Q.quantized_matmul_int8(x, q, s) - x @ w.t()).abs().max() < 0.6


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(64, 256, 512), (300, 520, 1024), (1024, 4096, 4096)])
def test_q4_0_gemm_gpu(M, N, K):
    from ferrotorch_b200 import _native

    torch.manual_seed(M)
    w = torch.randn(N, K) * 0.05
    nib, sc = Q.q4_0_planes(quantize_q4_0(w), N, K)
    deq = Q.dequant_q4_0_planes(nib, sc)
    x = (torch.randn(M, K)).to(torch.bfloat16).cuda()
    bias = torch.randn(N).to(torch.bfloat16).cuda()
    before = _native.launch_count()
    y = Q.q4_0_linear(x, nib.cuda(), sc.cuda(), bias)
    torch.cuda.synchronize()
    assert _native.launch_count() == before + 1 and _native.device_status(0) == 0
    want = x.float().cpu() @ deq.to(torch.bfloat16).float().t() + bias.float().cpu()
    err = (y.float().cpu() - want).abs().max().item()
    assert err < 0.02 * (K ** 0.5) * 0.05 * 4 + 0.05, err


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(64, 256, 512), (300, 520, 1024), (1024, 4096, 4096)])
def test_sparse24_gemm_gpu(M, N, K):
    from ferrotorch_b200 import _native

    torch.manual_seed(N)
    w = Q.apply_2_4_mask((torch.randn(N, K) * 0.05).to(torch.bfloat16))
    v, meta = Q.pack_2_4(w)
    x = torch.randn(M, K).to(torch.bfloat16).cuda()
    y = Q.sparse24_linear(x, v.cuda(), meta.cuda())
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    want = x.float().cpu() @ w.float().t()
    err = (y.float().cpu() - want).abs().max().item()
    assert err < 0.02 * (K ** 0.5) * 0.05 * 4 + 0.05, err
