"""Flash-attention kernels against the fp32 PyTorch attention of ops.reference."""
import pytest
import torch

from ferrotorch_b200 import _native
from ferrotorch_b200.ops import functional as F
from ferrotorch_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(got, want, atol, rtol, what):
    err = (got.float() - want.float()).abs()
    tol = atol + rtol * want.float().abs()
    assert not (err > tol).any(), "%s: max err %.4g" % (what, float(err.max()))


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,causal", [
    (1, 128, 128, 2, 2, 128, True),
    (2, 256, 256, 4, 2, 128, True),
    (1, 384, 384, 4, 1, 128, False),
    (2, 200, 200, 4, 2, 128, True),     # ragged: tile tails in q and kv
    (1, 100, 333, 2, 1, 128, True),     # query block is the tail of a longer key sequence
    (1, 1024, 1024, 8, 2, 128, True),
    (2, 256, 256, 4, 4, 64, True),
    (1, 130, 190, 2, 2, 64, False),
    (1, 2048, 2048, 4, 2, 128, True),   # many key blocks per CTA: lazy rescale, ring wrap-arounds
    (1, 640, 640, 2, 1, 128, True),     # odd number of query tiles: the last CTA has one tile only
    (2, 513, 513, 4, 2, 128, True),
    (1, 300, 700, 2, 2, 64, True),
    (1, 1024, 1024, 2, 2, 64, False),
])
def test_flash_fwd(B, Sq, Sk, Hq, Hkv, D, causal):
    torch.manual_seed(Sq + Sk + Hq)
    q, k, v = _rand(B, Sq, Hq, D), _rand(B, Sk, Hkv, D), _rand(B, Sk, Hkv, D)
    out, lse = F.flash_attn_fwd(q, k, v, causal)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    want, lse_w = R.attention(q, k, v, causal)
    _close(out, want, 2e-2, 2e-2, "attention out")
    _close(lse, lse_w, 2e-2, 1e-3, "attention lse")


def test_flash_fwd_large_scores_lazy_rescale():
    # row maxima that keep growing along the keys (by more and by less than the lazy-rescale
    # threshold) exercise both the rescale of O in TMEM and the stale-reference path
    torch.manual_seed(5)
    B, S, H, D = 1, 1024, 2, 128
    q, k, v = _rand(B, S, H, D), _rand(B, S, H, D), _rand(B, S, H, D)
    ramp = torch.linspace(0.2, 3.0, S, device=DEV).view(1, S, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    out, lse = F.flash_attn_fwd(q, k, v, False)
    want, lse_w = R.attention(q, k, v, False)
    _close(out, want, 2e-2, 2e-2, "attention out (growing maxima)")
    _close(lse, lse_w, 2e-2, 1e-3, "attention lse (growing maxima)")
    assert _native.device_status(0) == 0


def test_flash_fwd_packed_qkv():
    torch.manual_seed(0)
    B, S, Hq, Hkv, D = 2, 256, 8, 2, 128
    qkv = _rand(B, S, Hq + 2 * Hkv, D)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    out, _ = F.flash_attn_fwd(q, k, v, True)
    want, _ = R.attention(q, k, v, True)
    _close(out, want, 2e-2, 2e-2, "packed qkv")
    assert _native.device_status(0) == 0


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,causal", [
    (1, 128, 128, 2, 2, 128, True),
    (2, 256, 256, 4, 2, 128, True),
    (1, 320, 320, 4, 1, 128, False),
    (2, 200, 200, 4, 2, 128, True),
    (1, 100, 333, 2, 1, 128, True),
    (1, 1024, 1024, 8, 2, 128, True),
    (2, 256, 256, 4, 4, 64, True),
    (1, 130, 190, 2, 2, 64, False),
    (1, 2048, 2048, 8, 2, 128, True),    # many steps per CTA: ring and double-buffer wrap-arounds, GQA group of 4
    (2, 700, 700, 4, 4, 128, True),
    (1, 448, 448, 2, 1, 128, False),
])
@pytest.mark.parametrize("two_pass", [False, True])
def test_flash_bwd(B, Sq, Sk, Hq, Hkv, D, causal, two_pass):
    from ferrotorch_b200.ops import attention as A
    from ferrotorch_b200.ops.attention import flash_attention

    if two_pass and D != 128:
        pytest.skip("head_dim 64 always runs the two-pass kernels")
    prev = A.deterministic(two_pass)
    try:
        _flash_bwd_case(flash_attention, B, Sq, Sk, Hq, Hkv, D, causal)
    finally:
        A.deterministic(prev)


def _flash_bwd_case(flash_attention, B, Sq, Sk, Hq, Hkv, D, causal):

    torch.manual_seed(Sq * 3 + Sk + Hq)
    q, k, v = (_rand(B, Sq, Hq, D).requires_grad_(), _rand(B, Sk, Hkv, D).requires_grad_(),
               _rand(B, Sk, Hkv, D).requires_grad_())
    do = _rand(B, Sq, Hq, D, scale=0.5)
    out = flash_attention(q, k, v, causal=causal)
    out.backward(do)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    want, _ = R.attention(qr, kr, vr, causal)
    want.backward(do.float())
    _close(q.grad, qr.grad, 3e-2, 3e-2, "dq")
    _close(k.grad, kr.grad, 3e-2, 3e-2, "dk")
    _close(v.grad, vr.grad, 3e-2, 3e-2, "dv")


def test_flash_bwd_packed_qkv_grad_layout():
    from ferrotorch_b200.ops.attention import flash_attention

    torch.manual_seed(2)
    B, S, Hq, Hkv, D = 1, 256, 8, 2, 128
    qkv = _rand(B, S, Hq + 2 * Hkv, D).requires_grad_()
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    do = _rand(B, S, Hq, D, scale=0.5)
    flash_attention(q, k, v, causal=True).backward(do)
    ref_in = qkv.detach().float().requires_grad_()
    qr, kr, vr = ref_in[:, :, :Hq], ref_in[:, :, Hq:Hq + Hkv], ref_in[:, :, Hq + Hkv:]
    R.attention(qr, kr, vr, True)[0].backward(do.float())
    _close(qkv.grad, ref_in.grad, 3e-2, 3e-2, "packed dqkv")
