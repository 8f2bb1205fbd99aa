"""Post-training quantisation against PyTorch's own quantisation (the conventions are shared) and
hand-worked values."""
import pytest
import torch

from ferrotorch_b200.ops import ptq as Q


def test_qparams_and_per_tensor_quantisation_match_torch():
    assert (Q.QuantDtype.Int4.qmin, Q.QuantDtype.Int4.qmax, Q.QuantDtype.Uint8.qmax) == (-8, 7, 255)
    p = Q.QParams.asymmetric(-1.0, 3.0, Q.QuantDtype.Uint8)
    assert p.scale.item() == pytest.approx(4 / 255) and p.zero_point.item() == 64          # round(0 - (-1 / s)) = 63.75 -> 64
    p = Q.QParams.asymmetric(0.5, 3.0, Q.QuantDtype.Int8)                                  # the range is widened to contain 0
    assert p.scale.item() == pytest.approx(3 / 255) and p.zero_point.item() == -128
    s = Q.QParams.symmetric(2.0, Q.QuantDtype.Int8)
    assert s.scale.item() == pytest.approx(2 / 127.5) and s.zero_point.item() == 0
    assert Q.QParams.symmetric(2.0, Q.QuantDtype.Uint8).zero_point.item() == 128
    e = Q.QParams.asymmetric(float("inf"), float("-inf"))                                  # nothing observed
    assert (e.scale.item(), e.zero_point.item()) == (1.0, 0)
    torch.manual_seed(0)
    x = torch.randn(64, 32) * 2
    q = Q.quantize(x, dtype=Q.QuantDtype.Uint8)
    ref = torch.quantize_per_tensor(x, q.scale.item(), int(q.zero_point.item()), torch.quint8)
    assert torch.equal(q.data, ref.int_repr()) and torch.allclose(q.dequantize(), ref.dequantize(), atol=1e-6)
    assert (q.dequantize() - x).abs().max() <= q.scale.item() / 2 + 1e-6 and q.shape == (64, 32) and q.numel() == 2048
    q4 = Q.quantize(x, dtype=Q.QuantDtype.Int4, symmetric=True)
    assert q4.data.min() >= -8 and q4.data.max() <= 7 and q4.data.dtype == torch.int8
    assert (Q.dequantize(q4) - x).abs().max() <= q4.scale.item() * 0.5 + x.abs().max() / 7.5 * 0.01 + 1e-5 + q4.scale.item() / 2
    with pytest.raises(ValueError):
        Q.quantize(torch.tensor([1.0, float("nan")]))
    with pytest.raises(ValueError):
        Q.quantize(x, Q.QuantScheme.per_channel(3))


def test_per_channel_and_integer_matmul():
    torch.manual_seed(1)
    w = torch.randn(16, 8) * torch.linspace(0.1, 3.0, 8)                # columns of very different scale
    qc = Q.quantize(w, Q.QuantScheme.per_channel(1), symmetric=True)
    ref = torch.quantize_per_channel(w, qc.scale, qc.zero_point.to(torch.int64), 1, torch.qint8)
    diff = (qc.data.int() - ref.int_repr().int()).abs()                  # torch divides in float64: a tie may fall the other way
    assert diff.max() <= 1 and (diff > 0).float().mean() < 0.02 and qc.scale.shape == (8,)
    qt = Q.quantize(w, symmetric=True)
    assert (qc.dequantize() - w).abs().mean() < (qt.dequantize() - w).abs().mean()      # per channel is tighter
    a = torch.randn(5, 16)
    qa = Q.quantize(a)
    for qb in (qc, qt):
        got = Q.quantized_matmul(qa, qb)
        assert torch.allclose(got, qa.dequantize() @ qb.dequantize(), atol=1e-4)          # integer path == dequantised product
        assert (got - a @ w).abs().max() < 0.25
    with pytest.raises(ValueError):
        Q.quantized_matmul(qa, Q.quantize(torch.randn(7, 3)))
    with pytest.raises(ValueError):
        Q.quantized_matmul(Q.quantize(a, Q.QuantScheme.per_channel(0)), qt)
    named = Q.quantize_named_tensors({"w": w, "steps": torch.tensor([3]), "b": torch.randn(8)}, Q.QuantScheme.per_channel(1))
    assert isinstance(named["w"], Q.QuantizedTensor) and named["w"].scheme.axis == 1 and named["b"].scheme.axis is None
    assert named["steps"].dtype == torch.int64


def test_observers():
    torch.manual_seed(2)
    mm = Q.MinMaxObserver()
    assert mm.calculate_qparams().scale.item() == 1.0
    for _ in range(3):
        mm.observe(torch.randn(100))
    mm.observe(torch.tensor([50.0]))                                     # one outlier
    hist = Q.HistogramObserver(512, coverage=0.99)
    data = torch.randn(20000)
    hist.observe(data[:10000])
    hist.observe(torch.cat([data[10000:], torch.tensor([50.0])]))       # the range grows: counts are re-binned
    lo, hi = hist.range()
    assert -4 < lo < -1.5 and 1.5 < hi < 4                               # the outlier does not stretch the range
    assert hist.calculate_qparams().scale.item() < mm.calculate_qparams().scale.item() / 5
    assert int(hist.hist.sum()) == 20001
    pc = Q.PerChannelMinMaxObserver(3, axis=1)
    pc.observe(torch.tensor([[1.0, -2.0, 0.0], [0.5, 4.0, 0.0]]))
    pc.observe(torch.tensor([[3.0, 0.0, -1.0]]))
    assert pc.min.tolist() == [0.5, -2.0, -1.0] and pc.max.tolist() == [3.0, 4.0, 0.0]
    assert pc.calculate_qparams(Q.QuantDtype.Int4).scale.shape == (3,)
    with pytest.raises(ValueError):
        pc.observe(torch.zeros(2, 4))
    with pytest.raises(ValueError):
        Q.HistogramObserver(0)
    for o in (mm, hist, pc):
        o.reset()
    assert hist.hist is None and mm.min == float("inf")
    hist.observe(data)
    q = Q.quantize(data, qparams=hist.calculate_qparams())             # calibrated range: the tails saturate
    assert q.qdtype is Q.QuantDtype.Int8 and int(q.data.max()) == 127 and int(q.data.min()) == -128
