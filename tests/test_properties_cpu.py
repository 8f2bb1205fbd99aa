"""Property-based checks (hypothesis) of host-side code: invariants that must hold for every input
of a family, not only for hand-picked cases."""
import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

FAST = settings(max_examples=40, deadline=None)


@FAST
@given(st.integers(1, 400), st.floats(0.05, 0.95), st.integers(0, 2 ** 31 - 1))
def test_nms_keeps_an_independent_dominating_set(n, thr, seed):
    # (1) kept boxes do not overlap each other above the threshold; (2) every dropped box overlaps a kept
    # box of a higher score above it; (3) native sweep and torch formulation agree
    from ferrotorch_b200.ops import det_ops as D

    g = torch.Generator().manual_seed(seed)
    xy, wh = torch.rand(n, 2, generator=g) * 60, torch.rand(n, 2, generator=g) * 40 + 0.5
    boxes, scores = torch.cat([xy, xy + wh], 1), torch.rand(n, generator=g)
    keep = D.nms(boxes, scores, thr)
    assert torch.equal(keep, D.nms_torch(boxes, scores, thr))
    assert (scores[keep][:-1] >= scores[keep][1:]).all()
    iou = D.box_iou(boxes, boxes)
    kk = iou[keep][:, keep].clone()
    kk.fill_diagonal_(0)
    assert (kk <= thr).all()
    dropped = torch.ones(n, dtype=torch.bool)
    dropped[keep] = False
    for i in torch.where(dropped)[0].tolist():
        better = keep[scores[keep] >= scores[i]]
        assert (iou[i, better] > thr).any()


@FAST
@given(st.integers(1, 6), st.integers(1, 8), st.integers(0, 2 ** 31 - 1))
def test_q4_0_round_trip_error_and_fixed_point(rows, blocks, seed):
    # |x - dq(q(x))| <= |d| / 2 except at the clamped top code (<= |d|); quantising the result again changes nothing
    from ferrotorch_b200.ops.quant import dequant_q4_0_planes, quantize_q4_0_planes

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, 32 * blocks, generator=g) * torch.rand(1, generator=g) * 10
    nib, sc = quantize_q4_0_planes(x)
    y = dequant_q4_0_planes(nib, sc)
    d = sc.float().abs().repeat_interleave(32, dim=1)
    assert ((x - y).abs() <= d * 1.001 + 1e-6).all()
    inner = (x - y).abs() <= d * 0.5 * 1.01 + 1e-3 * d + 1e-6          # fp16 scale rounding leaves a little slack
    assert inner.float().mean() > 0.9
    nib2, sc2 = quantize_q4_0_planes(y)
    y2 = dequant_q4_0_planes(nib2, sc2)
    nib3, sc3 = quantize_q4_0_planes(y2)
    assert torch.equal(nib2, nib3) and torch.equal(sc2, sc3)


@FAST
@given(st.integers(0, 2 ** 40), st.integers(0, 2 ** 63 - 1), st.lists(st.integers(0, 37), min_size=1, max_size=6))
def test_philox_stream_is_continuous_over_arbitrary_splits(counter, seed, cuts):
    # drawing n words at once equals drawing them in pieces: the generator's (counter, offset) state carries over
    from ferrotorch_b200.utils.philox import PhiloxGenerator, PhiloxState

    total = sum(cuts)
    a = PhiloxGenerator(seed)
    a.set_state(PhiloxState.from_parts(counter, seed, 0))
    whole = a.words(total)
    b = PhiloxGenerator(seed)
    b.set_state(PhiloxState.from_parts(counter, seed, 0))
    pieces = np.concatenate([b.words(c) for c in cuts]) if total else np.zeros(0, dtype=whole.dtype)
    assert np.array_equal(whole, pieces)
    assert a.get_state() == b.get_state()


@FAST
@given(st.integers(2, 5), st.integers(1, 3), st.integers(0, 2 ** 31 - 1), st.booleans())
def test_attention_over_key_blocks_merges_exactly(parts, heads_kv, seed, causal_first):
    # attention over the whole key set = merge of attention over any partition of the keys
    from ferrotorch_b200.ops import reference as R
    from ferrotorch_b200.parallel.context_parallel import merge_attention

    g = torch.Generator().manual_seed(seed)
    S, D = 4 * parts + 3, 8
    q = torch.randn(1, 6, 2 * heads_kv, D, generator=g)
    k, v = torch.randn(1, S, heads_kv, D, generator=g), torch.randn(1, S, heads_kv, D, generator=g)
    want, want_lse = R.attention(q, k, v, causal=False)
    cuts = sorted(set(torch.randint(1, S, (parts - 1,), generator=g).tolist()))
    bounds = [0] + cuts + [S]
    out = lse = None
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        o, l = R.attention(q, k[:, lo:hi], v[:, lo:hi], causal=False)
        out, lse = (o, l) if out is None else merge_attention(out, lse, o, l)
    assert torch.allclose(out, want, atol=1e-5) and torch.allclose(lse, want_lse, atol=1e-5)


@FAST
@given(st.lists(st.tuples(st.sampled_from(["float32", "float16", "bfloat16", "int64", "int32", "uint8", "bool"]),
                          st.lists(st.integers(0, 5), min_size=0, max_size=3)), min_size=1, max_size=5),
       st.integers(0, 2 ** 31 - 1))
def test_safetensors_round_trip_of_any_dtype_and_shape(specs, seed):
    import os
    import tempfile

    from ferrotorch_b200.serialize.state import load_safetensors, save_safetensors

    g = torch.Generator().manual_seed(seed)
    state = {}
    for i, (dt, shape) in enumerate(specs):
        dtype = getattr(torch, dt)
        if dtype.is_floating_point:
            t = torch.randn(shape, generator=g).to(dtype)
        elif dtype == torch.bool:
            t = torch.rand(shape, generator=g) > 0.5
        else:
            t = torch.randint(0, 100, shape, generator=g).to(dtype)
        state["t%d.weight" % i] = t
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "x.safetensors")
        save_safetensors(state, path, metadata={"format": "pt"})
        back = load_safetensors(path)
        assert set(back) == set(state)
        for k, t in state.items():
            assert back[k].dtype == t.dtype and back[k].shape == t.shape and torch.equal(back[k], t)


@FAST
@given(st.integers(1, 4), st.integers(2, 40), st.integers(2, 40), st.integers(1, 9), st.integers(0, 2 ** 31 - 1))
def test_roi_align_of_a_constant_map_is_that_constant_inside_the_map(c, h, w, k, seed):
    # bilinear samples of a constant are the constant; boxes that stay inside the map never touch the zero border
    from ferrotorch_b200.ops import det_ops as D

    g = torch.Generator().manual_seed(seed)
    val = torch.rand(c, generator=g) + 0.5
    feat = val.view(1, c, 1, 1).expand(1, c, h, w).contiguous()
    x1, y1 = torch.rand(k, generator=g) * (w - 1) * 0.5, torch.rand(k, generator=g) * (h - 1) * 0.5
    x2, y2 = x1 + torch.rand(k, generator=g) * (w - 1) * 0.5, y1 + torch.rand(k, generator=g) * (h - 1) * 0.5
    rois = torch.stack([torch.zeros(k), x1, y1, x2, y2], 1)
    for fn in (D.roi_align, D.roi_align_torch):
        out = fn(feat, rois, 3, 1.0, 2, True)
        assert torch.allclose(out, val.view(1, c, 1, 1).expand_as(out), atol=1e-5)
