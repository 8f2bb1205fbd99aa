"""Numerics of every native kernel against a plain PyTorch fp32 reference of the same op.

Shapes cover tile-edge remainders (M, N, K not multiples of the tile) as well as the
Llama-3-8B shapes the benchmarks use.
"""
import math

import pytest
import torch

import ferrotorch_b200 as ft
from ferrotorch_b200 import _native
from ferrotorch_b200.ops import functional as F
from ferrotorch_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _assert_close(got, want, rtol=2e-2, atol=2e-2, what=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = err > tol
    assert not bad.any(), "%s: %d/%d mismatches, max err %.4g (ref max %.4g)" % (
        what, int(bad.sum()), bad.numel(), float(err.max()), float(want.abs().max()))


def test_library_loaded_and_status_clean():
    lib = _native.kernels()
    assert lib.ft_abi_version() == 1
    assert _native.device_status(0) == 0


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (304, 264, 200), (1000, 1032, 520),
                                   (64, 4096, 4096), (2048, 6144, 4096)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(M + N + K + 2 * a_mn + b_mn)
    a = _rand(K, M).t() if a_mn else _rand(M, K)
    b = _rand(K, N).t() if b_mn else _rand(N, K)
    before = _native.launch_count()
    c = F.gemm_nt(a, b)
    torch.cuda.synchronize()
    assert _native.launch_count() > before, "gemm did not run the native kernel"
    assert _native.device_status(0) == 0
    want = a.float() @ b.float().t()
    _assert_close(c, want, rtol=1e-2, atol=0.02 * math.sqrt(K), what="gemm %dx%dx%d" % (M, N, K))


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_gemm_tile_sizes(bn):
    torch.manual_seed(bn)
    M, N, K = 384, 520, 328
    a, b = _rand(M, K), _rand(N, K)
    c = F.gemm_nt(a, b, bn=bn)
    _assert_close(c, a.float() @ b.float().t(), rtol=1e-2, atol=0.4, what="bn=%d" % bn)
    assert _native.device_status(0) == 0


@pytest.mark.parametrize("bn", [-64, -128, -256])
def test_gemm_single_cta_kernel(bn):
    # a negative tile size selects the one-CTA kernel also for shapes the CTA-pair kernel would take
    torch.manual_seed(-bn)
    M, N, K = 640, 776, 328
    a, b = _rand(M, K), _rand(N, K)
    c = F.gemm_nt(a, b, bn=bn)
    _assert_close(c, a.float() @ b.float().t(), rtol=1e-2, atol=0.4, what="single bn=%d" % bn)
    assert _native.device_status(0) == 0


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (1, 1)])
def test_gemm_pair_kernel_long_run(a_mn, b_mn):
    # many tiles per CTA pair (both accumulators, several ring wrap-arounds), ragged M and N edges
    torch.manual_seed(7)
    M, N, K = 4096 + 136, 4096 + 72, 1024 + 40
    a = _rand(K, M).t() if a_mn else _rand(M, K)
    b = _rand(K, N).t() if b_mn else _rand(N, K)
    want = a.float() @ b.float().t()
    _assert_close(F.gemm_nt(a, b), want, rtol=1e-2, atol=0.02 * math.sqrt(K), what="pair long")
    c32 = torch.randn(M, N, device=DEV)
    c = c32.clone()
    F.gemm_nt(a, b, out=c, accumulate=True)
    _assert_close(c, want + c32, rtol=1e-3, atol=0.1, what="pair accumulate fp32")
    assert _native.device_status(0) == 0


@pytest.mark.parametrize("M,N,K,ksplit", [(64, 4096, 4096, 0), (64, 4096, 14336, 0), (64, 28672, 4096, 0), (17, 6144, 4096, 0),
                                          (128, 4096, 4096, 0), (100, 1032, 520, 1), (64, 4096, 4096, 1), (1, 2048, 1024, 4)])
def test_gemm_small_m(M, N, K, ksplit):
    # decode-sized batches: weight as the 128-row operand, transposed epilogue or split-K + finalize
    torch.manual_seed(M + N + K)
    x, w = _rand(M, K), _rand(N, K) * 0.05
    bias = _rand(N)
    want = x.float() @ w.float().t()
    before = _native.launch_count()
    y = F.gemm_small_m(x, w, ksplit=ksplit)
    torch.cuda.synchronize()
    assert _native.launch_count() > before and _native.device_status(0) == 0
    _assert_close(y, want, rtol=1e-2, atol=0.02 * math.sqrt(K) * 0.05, what="small-m %dx%dx%d" % (M, N, K))
    _assert_close(F.gemm_small_m(x, w, bias=bias, ksplit=ksplit), want + bias.float(), rtol=1e-2,
                  atol=0.02 * math.sqrt(K) * 0.05 + 0.02, what="small-m bias")
    if ksplit != 1:
        res = _rand(M, N)
        _assert_close(F.gemm_small_m(x, w, residual=res, ksplit=ksplit), want + res.float(), rtol=1e-2,
                      atol=0.02 * math.sqrt(K) * 0.05 + 0.02, what="small-m residual")
        # pieces are summed in a fixed order: a second call gives the same bits
        assert torch.equal(F.gemm_small_m(x, w, ksplit=ksplit), y)
    else:
        _assert_close(F.gemm_small_m(x, w, activation="silu", ksplit=1), torch.nn.functional.silu(want), rtol=1e-2,
                      atol=0.02 * math.sqrt(K) * 0.05 + 0.02, what="small-m silu")
    # gemm_nt routes decode shapes here
    n0 = F.stats["gemm_small_m"]
    _assert_close(F.gemm_nt(x, w), want, rtol=1e-2, atol=0.02 * math.sqrt(K) * 0.05, what="gemm_nt routed")
    assert (F.stats["gemm_small_m"] > n0) == (N >= 1024 and K >= 512)


def test_gemm_epilogues():
    torch.manual_seed(0)
    M, N, K = 520, 776, 392
    a, b = _rand(M, K), _rand(N, K)
    bias = _rand(N)
    want = a.float() @ b.float().t()
    _assert_close(F.gemm_nt(a, b, bias=bias), want + bias.float(), rtol=1e-2, atol=0.4, what="bias")
    _assert_close(F.gemm_nt(a, b, out_dtype=torch.float32), want, rtol=1e-3, atol=0.05, what="fp32 out")
    c0 = _rand(M, N)
    c = c0.clone()
    F.gemm_nt(a, b, out=c, accumulate=True)
    _assert_close(c, want + c0.float(), rtol=1e-2, atol=0.4, what="accumulate bf16")
    c32 = torch.randn(M, N, device=DEV)
    c = c32.clone()
    F.gemm_nt(a, b, out=c, accumulate=True)
    _assert_close(c, want + c32, rtol=1e-3, atol=0.05, what="accumulate fp32")
    _assert_close(F.gemm_nt(a, b, bias=bias, activation="relu"), torch.relu(want + bias.float()),
                  rtol=1e-2, atol=0.4, what="relu")
    _assert_close(F.gemm_nt(a, b, activation="gelu"), torch.nn.functional.gelu(want), rtol=1e-2, atol=0.4,
                  what="gelu")
    _assert_close(F.gemm_nt(a, b, activation="silu"), torch.nn.functional.silu(want), rtol=1e-2, atol=0.4,
                  what="silu")
    # strided output (a column slice of a wider buffer)
    wide = torch.zeros(M, 2 * N, device=DEV, dtype=torch.bfloat16)
    F.gemm_nt(a, b, out=wide[:, N:])
    _assert_close(wide[:, N:], want, rtol=1e-2, atol=0.4, what="strided out")
    assert float(wide[:, :N].abs().max()) == 0.0
    assert _native.device_status(0) == 0


def test_gemm_deterministic():
    a, b = _rand(1024, 1024), _rand(2048, 1024)
    c1 = F.gemm_nt(a, b).clone()
    c2 = F.gemm_nt(a, b)
    assert torch.equal(c1, c2)


def test_linear_autograd_matches_torch():
    torch.manual_seed(1)
    x = _rand(4, 96, 512, scale=0.5).requires_grad_()
    w = _rand(384, 512, scale=0.05).requires_grad_()
    b = _rand(384, scale=0.1).requires_grad_()
    y = F.linear(x, w, b)
    dy = _rand(4, 96, 384)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    _assert_close(y, yr, what="linear fwd")
    _assert_close(x.grad, xr.grad, what="linear dx")
    _assert_close(w.grad, wr.grad, rtol=2e-2, atol=0.15, what="linear dw")
    _assert_close(b.grad, br.grad, rtol=2e-2, atol=0.3, what="linear db")


@pytest.mark.parametrize("rows,H", [(7, 256), (333, 4096), (64, 8192), (1000, 1024)])
def test_rmsnorm_fwd_bwd(rows, H):
    torch.manual_seed(rows)
    x = _rand(rows, H).requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = F.rmsnorm(x, w, 1e-5)
    dy = _rand(rows, H)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = R.rmsnorm(xr, wr, 1e-5)
    yr.backward(dy.float())
    _assert_close(y, yr, what="rmsnorm fwd")
    _assert_close(x.grad, xr.grad, what="rmsnorm dx")
    _assert_close(w.grad, wr.grad, rtol=2e-2, atol=0.02 * math.sqrt(rows) + 0.05, what="rmsnorm dw")


def test_rmsnorm_residual():
    torch.manual_seed(3)
    x = _rand(130, 2048).requires_grad_()
    r = _rand(130, 2048).requires_grad_()
    w = _rand(2048).requires_grad_()
    y, s = F.rmsnorm(x, w, 1e-5, residual=r)
    dy, ds = _rand(130, 2048), _rand(130, 2048)
    torch.autograd.backward([y, s], [dy, ds])
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    sr = (xr + rr)
    yr = R.rmsnorm(sr.detach().to(torch.bfloat16).float() + (sr - sr.detach()), wr, 1e-5)
    torch.autograd.backward([yr, sr], [dy.float(), ds.float()])
    _assert_close(s, sr, what="residual sum")
    _assert_close(y, yr, what="rmsnorm(res) fwd")
    _assert_close(x.grad, xr.grad, what="rmsnorm(res) dx")
    _assert_close(r.grad, rr.grad, what="rmsnorm(res) dres")


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_fwd_bwd(interleaved):
    torch.manual_seed(5)
    B, S, Hq, Hkv, D = 2, 37, 8, 2, 128
    cos, sin = R.rope_tables(D, 64, 500000.0, device=DEV)
    qkv = _rand(B, S, Hq + 2 * Hkv, D)
    want = qkv.clone().view(B * S, Hq + 2 * Hkv, D)
    pos = torch.arange(S, device=DEV).repeat(B)
    want[:, : Hq + Hkv] = R.rope(want[:, : Hq + Hkv], cos, sin, pos, interleaved)
    x = qkv.clone().requires_grad_()
    y = F.rope_(x * 1.0, cos, sin, n_rot_heads=Hq + Hkv, seq_len=S, interleaved=interleaved)
    _assert_close(y.view(B * S, -1, D), want, what="rope fwd")
    g = _rand(B, S, Hq + 2 * Hkv, D)
    y.backward(g)
    gw = g.clone().view(B * S, Hq + 2 * Hkv, D)
    gw[:, : Hq + Hkv] = R.rope(gw[:, : Hq + Hkv], cos, sin, pos, interleaved, backward=True)
    _assert_close(x.grad.view(B * S, -1, D), gw, what="rope bwd")
    # explicit positions (decode: one token per sequence at arbitrary offsets)
    q1 = _rand(3, 1, 4, D)
    p = torch.tensor([5, 17, 63], device=DEV)
    got = F.rope_(q1.clone(), cos, sin, positions=p, interleaved=interleaved)
    _assert_close(got.view(3, 4, D), R.rope(q1.view(3, 4, D), cos, sin, p, interleaved), what="rope positions")


@pytest.mark.parametrize("act", ["silu", "relu", "gelu"])
def test_swiglu_fwd_bwd(act):
    torch.manual_seed(7)
    gu = _rand(257, 2 * 1416).requires_grad_()
    y = F.swiglu(gu, act)
    dy = _rand(257, 1416)
    y.backward(dy)
    gr = gu.detach().float().requires_grad_()
    yr = R.swiglu(gr, F._ACT_ID[act])
    yr.backward(dy.float())
    _assert_close(y, yr, what="swiglu fwd")
    _assert_close(gu.grad, gr.grad, rtol=2e-2, atol=3e-2, what="swiglu bwd")


def test_embedding_fwd_bwd():
    torch.manual_seed(9)
    V, H = 1000, 512
    w = _rand(V, H).requires_grad_()
    ids = torch.randint(0, V, (4, 33), device=DEV)
    y = F.embedding(ids, w)
    assert torch.equal(y, w.detach()[ids])
    dy = _rand(4, 33, H)
    y.backward(dy)
    wr = w.detach().float().requires_grad_()
    torch.nn.functional.embedding(ids, wr).backward(dy.float())
    _assert_close(w.grad, wr.grad, rtol=2e-2, atol=5e-2, what="embedding bwd")


@pytest.mark.parametrize("rows,V", [(5, 1000), (64, 128256), (33, 4099)])
def test_cross_entropy_fused(rows, V):
    torch.manual_seed(V)
    Vp = (V + 7) // 8 * 8
    buf = _rand(rows, Vp, scale=2.0)
    z = buf[:, :V]
    tgt = torch.randint(0, V, (rows,), device=DEV)
    tgt[0] = -100
    zr = z.detach().float().requires_grad_()
    lr = R.cross_entropy(zr, tgt)
    (lr.sum() * 0.25).backward()
    loss = F.cross_entropy_fwd_bwd_(z, tgt, 0.25)
    _assert_close(loss, lr, rtol=1e-3, atol=2e-2, what="ce loss")
    _assert_close(z, zr.grad, rtol=2e-2, atol=2e-3, what="ce grad")


def test_linear_cross_entropy_chunked():
    torch.manual_seed(11)
    T, H, V = 300, 256, 2048
    h = _rand(T, H, scale=0.5).requires_grad_()
    w = _rand(V, H, scale=0.05).requires_grad_()
    tgt = torch.randint(0, V, (T,), device=DEV)
    loss = F.linear_cross_entropy(h, w, tgt, chunk_rows=128)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = torch.nn.functional.cross_entropy(hr @ wr.t(), tgt)
    lr.backward()
    assert abs(float(loss) - float(lr)) < 2e-2
    _assert_close(h.grad, hr.grad, rtol=3e-2, atol=2e-4, what="lce dh")
    _assert_close(w.grad, wr.grad, rtol=3e-2, atol=2e-4, what="lce dw")


def test_adamw_flat_matches_reference():
    torch.manual_seed(13)
    n = 4096 * 33
    lib = _native.kernels()
    p = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    plp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    hp = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = _rand(n)
        rc = lib.ft_adamw_flat(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), plp.data_ptr(), n, 0,
                               None, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["weight_decay"], step,
                               0, 0, torch.cuda.current_stream().cuda_stream)
        _native.check(rc)
        R.adamw_step(pr, g, mr, vr, step=step, **hp)
    assert torch.allclose(p, pr, rtol=1e-5, atol=1e-6)
    assert torch.allclose(m, mr, rtol=1e-5, atol=1e-7)
    assert torch.allclose(v, vr, rtol=1e-5, atol=1e-9)
    assert torch.equal(plp, p.to(torch.bfloat16))
    # parity with torch.optim.AdamW on the same trajectory
    q = torch.nn.Parameter(torch.randn(1024, device=DEV))
    q0 = q.detach().clone()
    opt = torch.optim.AdamW([q], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    mm, vv = torch.zeros_like(q0), torch.zeros_like(q0)
    for step in range(1, 4):
        g = torch.randn(1024, device=DEV)
        q.grad = g.clone()
        opt.step()
        rc = lib.ft_adamw_flat(q0.data_ptr(), mm.data_ptr(), vv.data_ptr(), g.data_ptr(), None, 1024, 1, None,
                               1e-3, 0.9, 0.999, 1e-8, 0.01, step, 0, 0, torch.cuda.current_stream().cuda_stream)
        _native.check(rc)
    assert torch.allclose(q0, q.detach(), rtol=1e-5, atol=1e-6)


def test_sgd_flat_matches_torch():
    torch.manual_seed(15)
    lib = _native.kernels()
    n = 2048
    q = torch.nn.Parameter(torch.randn(n, device=DEV))
    p = q.detach().clone()
    buf = torch.zeros(n, device=DEV)
    opt = torch.optim.SGD([q], lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)
    for step in range(3):
        g = torch.randn(n, device=DEV)
        q.grad = g.clone()
        opt.step()
        rc = lib.ft_sgd_flat(p.data_ptr(), buf.data_ptr(), g.data_ptr(), None, n, 1, None, 0.1, 0.9, 0.0, 1e-4,
                             1, int(step == 0), 0, torch.cuda.current_stream().cuda_stream)
        _native.check(rc)
    assert torch.allclose(p, q.detach(), rtol=1e-5, atol=1e-6)


def test_grad_norm_and_clip_coef():
    lib = _native.kernels()
    n = 1 << 20
    g = _rand(n)
    part = torch.empty(lib.ft_grad_norm_scratch(0), device=DEV)
    out = torch.empty(3, device=DEV)
    _native.check(lib.ft_grad_norm(g.data_ptr(), n, 0, part.data_ptr(), None, 1.0, out.data_ptr(), 0,
                                   torch.cuda.current_stream().cuda_stream))
    nrm = float(g.float().norm())
    assert abs(float(out[0]) - nrm) / nrm < 1e-4
    assert abs(float(out[1]) - min(1.0, 1.0 / (nrm + 1e-6))) < 1e-6


@pytest.mark.gpu
def test_parity_sweep_on_gpu():
    """Every op of the sweep harness: native bf16 kernel against the fp32 oracle."""
    from ferrotorch_b200.utils import parity

    rows = parity.sweep(None, "cuda")
    bad = [r for r in rows if not r["ok"]]
    assert not bad, bad
