"""The autograd surface: implicit differentiation of fixed points, forward-mode pairs, the wrappers."""
import pytest
import torch

from ferrotorch_b200 import autograd as A


def test_fixed_point_scalar_cases():
    # x = a x + b  ->  x* = b / (1 - a),  dx*/da = b / (1 - a)^2,  dx*/db = 1 / (1 - a)
    a = torch.tensor(0.5, dtype=torch.float64, requires_grad=True)
    b = torch.tensor(3.0, dtype=torch.float64, requires_grad=True)
    x = A.fixed_point(lambda x, p: p[0] * x + p[1], torch.tensor(10.0, dtype=torch.float64), [a, b], 1000, 1e-12)
    assert x.item() == pytest.approx(6.0, abs=1e-9)
    x.backward()
    assert a.grad.item() == pytest.approx(12.0, abs=1e-6) and b.grad.item() == pytest.approx(2.0, abs=1e-6)
    # the reference's own example: f(x, a) = a x has the fixed point 0
    z = A.fixed_point(lambda x, p: p[0] * x, torch.tensor(10.0), [torch.tensor(0.5, requires_grad=True)], 1000, 1e-8)
    assert abs(z.item()) < 1e-6


def test_fixed_point_matches_unrolled_gradients_on_a_deq_layer():
    torch.manual_seed(0)
    W = (0.3 * torch.randn(6, 6, dtype=torch.float64) / 6 ** 0.5).requires_grad_()
    U = torch.randn(6, 4, dtype=torch.float64, requires_grad=True)
    inp = torch.randn(4, dtype=torch.float64)
    frozen = torch.randn(6, dtype=torch.float64)                        # a parameter that wants no gradient
    f = lambda x, p: torch.tanh(p[0] @ x + p[1] @ inp + p[2])          # noqa: E731
    x = A.fixed_point(f, torch.zeros(6, dtype=torch.float64), [W, U, frozen], 500, 1e-13)
    assert torch.allclose(x, f(x.detach(), [W, U, frozen]), atol=1e-10)
    (x ** 2).sum().backward()
    gW, gU = W.grad.clone(), U.grad.clone()
    W.grad = U.grad = None
    y = torch.zeros(6, dtype=torch.float64)
    for _ in range(200):                                                # the memory-hungry way: unroll everything
        y = f(y, [W, U, frozen])
    (y ** 2).sum().backward()
    assert torch.allclose(gW, W.grad, atol=1e-8) and torch.allclose(gU, U.grad, atol=1e-8)
    with torch.no_grad():
        assert not A.fixed_point(f, torch.zeros(6, dtype=torch.float64), [W, U, frozen], 500, 1e-10).requires_grad


def test_fixed_point_rejects_bad_runs():
    p = [torch.tensor(2.0, requires_grad=True)]
    with pytest.raises(RuntimeError, match="no convergence"):
        A.fixed_point(lambda x, q: q[0] * x * 0.5 + 1.0, torch.tensor(1.0), p, 20, 1e-9)      # slope 1: never settles
    with pytest.raises(ValueError, match="non-finite"):
        A.fixed_point(lambda x, q: x * 1e30, torch.tensor(1e30), p, 20, 1e-9)
    with pytest.raises(ValueError):
        A.fixed_point(lambda x, q: x, torch.tensor(1.0), p, 0, 1e-9)
    with pytest.raises(ValueError):
        A.fixed_point(lambda x, q: x, torch.tensor(1.0), p, 10, float("nan"))
    with pytest.raises(ValueError, match="shape"):
        A.fixed_point(lambda x, q: x.repeat(2), torch.ones(2), p, 10, 1e-9)


def test_dual_tensors_and_function_transforms():
    x = A.DualTensor(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 0.0]))
    y = (x * x + 3.0 * x).sin() / (x + 1.0)
    f = lambda t: torch.sin(t * t + 3.0 * t) / (t + 1.0)                # noqa: E731
    out, tan = A.jvp(f, x.primal, x.tangent)
    assert torch.allclose(y.primal, out) and torch.allclose(y.tangent, tan, atol=1e-6)
    m = A.DualTensor(torch.eye(2), torch.ones(2, 2)) @ A.DualTensor(torch.tensor([[1.0], [2.0]]))
    assert torch.allclose(m.tangent, torch.tensor([[3.0], [3.0]])) and (-x).sum().tangent.item() == -1.0
    with pytest.raises(ValueError):
        A.DualTensor(torch.zeros(2), torch.zeros(3))
    out, g = A.vjp(f, x.primal, torch.tensor([1.0, 1.0]))
    assert torch.allclose(g, torch.autograd.functional.jacobian(f, x.primal).sum(0), atol=1e-6)
    assert torch.allclose(A.jacfwd(f)(x.primal), A.jacobian(f, x.primal), atol=1e-6)
    assert A.hessian(lambda t: (t ** 3).sum())(torch.tensor([1.0, 2.0])).diag().tolist() == [6.0, 12.0]
    assert A.gradcheck(lambda t: (t * t).sum(), (torch.randn(3, dtype=torch.float64, requires_grad=True),))


def test_wrappers_penalties_and_control_flow():
    w = torch.tensor([3.0, 4.0], requires_grad=True)
    A.backward((w ** 2).sum())
    assert w.grad.tolist() == [6.0, 8.0]
    with pytest.raises(ValueError):
        A.backward(w * 2)
    w.grad = None
    A.backward_with_grad(w * 2, torch.ones(2))
    assert w.grad.tolist() == [2.0, 2.0]
    n = A.grad_norm((w ** 2).sum(), [w])
    assert n.item() == pytest.approx(10.0) and n.requires_grad
    x = torch.randn(5, 3, requires_grad=True)
    gp = A.gradient_penalty((2.0 * x).sum(1), x, target=1.0)
    assert gp.item() == pytest.approx((12 ** 0.5 - 1.0) ** 2, rel=1e-5)
    with A.no_grad():
        assert not A.is_grad_enabled()
    with A.inference_mode():
        assert A.is_inference_mode()
    lin = torch.nn.Linear(4, 4)
    inp = torch.randn(2, 4, requires_grad=True)
    torch.manual_seed(1)
    a = A.checkpoint(lambda t: torch.nn.functional.dropout(lin(t), 0.5, True), inp)
    a.sum().backward()                                                  # the recomputation draws the same mask
    g1 = inp.grad.clone()
    inp.grad = None
    torch.manual_seed(1)
    torch.nn.functional.dropout(lin(inp), 0.5, True).sum().backward()
    assert torch.allclose(g1, inp.grad)
    assert A.cond(torch.tensor(True), lambda t: t + 1, lambda t: t - 1, (torch.zeros(2),)).tolist() == [1.0, 1.0]
    assert A.cond(False, lambda t: t + 1, lambda t: t - 1, (torch.zeros(2),)).tolist() == [-1.0, -1.0]
    with pytest.raises(ValueError):
        A.cond(True, lambda t: t, lambda t: t.repeat(2), (torch.zeros(2),))
    carry, ys = A.scan(lambda c, v: (c + v, c * v), torch.tensor(0.0), torch.tensor([1.0, 2.0, 3.0]))
    assert carry.item() == 6.0 and ys.tolist() == [0.0, 2.0, 9.0]


def test_core_vocabulary():
    import ferrotorch_b200 as ft
    from ferrotorch_b200 import core as C

    assert ft.autograd is A and C.Device.Cpu.type == "cpu" and C.Device.Cuda(1) == torch.device("cuda", 1)
    with pytest.raises(NotImplementedError):
        C.Device.Mps()
    assert C.MemoryFormat.ChannelsLast.value is torch.channels_last
    z = C.ComplexTensor(torch.ones(2), torch.zeros(2))
    assert z.is_complex() and C.SparseTensor(torch.tensor([[0, 1], [1, 0]]), torch.ones(2), (2, 2)).to_dense().sum() == 2
    nt = C.NestedTensor([torch.zeros(2, 3), torch.zeros(4, 3)])
    assert nt.is_nested and C.NamedTensor(torch.zeros(2, 3), ("n", "c")).names == ("n", "c")
    q = C.QuantizedTensor(torch.tensor([0.0, 0.5, 1.0]), 0.5)
    assert q.dequantize().tolist() == [0.0, 0.5, 1.0] and q.int_repr().tolist() == [0, 1, 2]
    assert C.rearrange(torch.zeros(2, 3, 4), "a b c -> a (b c)").shape == (2, 12)
    mt = C.masked_tensor(torch.tensor([1.0, 2.0, 3.0]), torch.tensor([True, False, True]))
    assert mt.sum().get_data().item() == 4.0
    torch.manual_seed(0)
    qq, kk, vv = torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8)
    causal = C.flex_attention(qq, kk, vv, lambda s, b, h, i, j: s.masked_fill(j > i, float("-inf")))
    want = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
    assert torch.allclose(causal, want, atol=1e-5)
    alibi = C.flex_attention(qq, kk, vv, lambda s, b, h, i, j: s - (h + 1) * (i - j).abs())
    assert not torch.allclose(alibi, C.flex_attention(qq, kk, vv), atol=1e-3)


def test_autocast_policy_table_and_debug_events():
    assert A.autocast_category("matmul") == A.AutocastCategory.ReducedPrecision
    assert A.autocast_category("softmax") == A.AutocastCategory.FullPrecision
    assert A.autocast_category("relu") == A.AutocastCategory.Passthrough
    assert not A.should_cast_to_reduced("matmul") and not A.is_autocast_enabled()
    lin = torch.nn.Linear(4, 4)
    x = torch.randn(2, 4)
    A.set_autocast_debug(True)
    try:
        lin(x)                                           # outside autocast: nothing is logged
        assert A.drain_autocast_events() == []
        with A.autocast("cpu", dtype=torch.bfloat16):
            assert A.should_cast_to_reduced("linear") and A.should_keep_full_precision("layer_norm")
            y = lin(x)
            z = torch.softmax(y, -1)
        ev = A.drain_autocast_events()
    finally:
        A.set_autocast_debug(False)
    assert y.dtype == torch.bfloat16 and not A.is_autocast_debug()
    gemm = [e for e in ev if e["op"] in ("addmm", "mm", "linear")]
    assert gemm and gemm[0]["category"] == A.AutocastCategory.ReducedPrecision and set(gemm[0]["inputs"]) == {"bfloat16"}
    soft = [e for e in ev if e["op"] in ("_softmax", "softmax")]
    # the log shows what really ran: on CUDA the softmax is promoted to fp32, the CPU autocast leaves it
    assert soft and soft[0]["category"] == A.AutocastCategory.FullPrecision and soft[0]["output"] == str(z.dtype)[6:]
    assert A.drain_autocast_events() == []
    lin(x)
    assert A.drain_autocast_events() == []               # recorder is off again


def test_block_masks_and_einops_helpers():
    from ferrotorch_b200 import core as C

    torch.manual_seed(0)
    q, k, v = torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4)
    bm = C.BlockMask.from_fn(lambda i, j: j <= i, 8, 8, block=4)                 # causal: the upper-right block drops out
    assert bm.keep.tolist() == [[True, False], [True, True]] and bm.sparsity() == 0.25
    out = C.flex_attention(q, k, v, lambda s, b, h, i, j: s.masked_fill(j > i, float("-inf")), block_mask=bm)
    assert torch.allclose(out, torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True), atol=1e-5)
    window = C.BlockMask.from_fn(lambda i, j: (i - j).abs() < 4, 8, 8, block=4)
    assert window.keep.all() and window.dense().shape == (8, 8)
    with pytest.raises(ValueError):
        C.flex_attention(q[:, :, :4], k, v, block_mask=bm)
    x = torch.arange(12.0).view(3, 4)
    assert C.reduce(x, "a b -> a", "sum").tolist() == [6.0, 22.0, 38.0] and C.repeat(x, "a b -> a b c", c=2).shape == (3, 4, 2)
