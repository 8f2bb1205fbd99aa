"""The flat tensor API under the reference's names: spot checks against torch and closed forms."""
import math

import pytest
import torch

import ferrotorch_b200 as ft
from ferrotorch_b200 import tensor_ops as T


def test_root_resolves_reference_and_torch_names():
    x = ft.from_slice([1, 2, 3, 4, 5, 6], [2, 3])
    assert torch.equal(ft.sum_dim(x, 1, True), torch.tensor([[6.0], [15.0]])) and ft.zeros(2).shape == (2,)
    assert torch.equal(ft.cat([x, x]).sum_to_size(1, 3), 2 * x.sum(0, keepdim=True)) and ft.scalar(3.0).dim() == 0
    assert ft.DType is torch.dtype and issubclass(ft.FerrotorchError, RuntimeError) and ft.Device is ft.core.Device
    with pytest.raises(AttributeError):
        ft.no_such_name
    with pytest.raises(ft.FerrotorchError):
        ft.from_slice([1, 2], [3])
    d = ft.Dispatcher()                       # a priority table of Python-level kernels (dispatch.rs)
    d.register("relu", ft.DispatchKey.Cpu, lambda inputs, keys: torch.relu(inputs[0]))
    d.register("relu", ft.DispatchKey.Autocast, lambda inputs, keys: d.call("relu", [inputs[0].bfloat16()], keys.remove(ft.DispatchKey.Autocast)))
    keys = ft.DispatchKeySet.from_keys([ft.DispatchKey.Cpu, ft.DispatchKey.Autocast])
    assert d.call("relu", [torch.tensor([-1.0, 2.0])], keys).dtype == torch.bfloat16 and keys.highest() is ft.DispatchKey.Autocast
    assert d.call_direct("relu", ft.DispatchKey.Cpu, [torch.tensor([-1.0])]).tolist() == [0.0] and d.kernel_count() == 2
    assert [k.name for k in keys.insert(ft.DispatchKey.Tracer).iter_desc()] == ["Tracer", "Autocast", "Cpu"] and ft.DispatchKeySet.all().len() == 11
    with pytest.raises(ft.FerrotorchError):
        d.call("relu", [x], ft.DispatchKeySet())
    with pytest.raises(ft.FerrotorchError):
        d.call("gelu", [x], keys)
    with pytest.raises(ft.FerrotorchError):
        d.call_direct("relu", ft.DispatchKey.Cuda, [x])


def test_reductions_clamps_and_selection():
    torch.manual_seed(0)
    x = torch.randn(3, 4, 5)
    torch.testing.assert_close(T.mean_dims(x, [0, 2]), x.mean((0, 2)))
    torch.testing.assert_close(T.var_dim(x, 1), x.var(1))
    torch.testing.assert_close(T.logsumexp_dims(x, [1, 2], True), torch.logsumexp(x, (1, 2), True))
    v, i = T.max_with_dim(x, 2)
    assert torch.equal(v, x.amax(2)) and torch.equal(i, x.argmax(2))
    v, i = T.topk_dim(x, 2, 1, largest=False)
    assert torch.equal(v, x.topk(2, 1, largest=False).values)
    r = T.cummax(x, 1)
    assert torch.equal(r.values, x.cummax(1).values) and torch.equal(r.indices, r[1])
    y = x.clone()
    y[0, 0, 0] = float("nan")
    torch.testing.assert_close(T.nansum_dim(y, 2), y.nansum(2))
    torch.testing.assert_close(T.norm_with_dim(x, 2.0, 1), x.norm(2, 1))
    assert torch.equal(T.clamp_opt(x, None, 0.5), x.clamp(max=0.5))
    with pytest.raises(T.FerrotorchError):
        T.clamp_opt(x)
    flat = [bool(v) for v in (x > 0).flatten()]
    assert torch.equal(T.where_cond(flat, x, -x), x.abs())
    src = torch.arange(8.0).view(4, 2)
    assert torch.equal(T.scatter_add_segments(src, [0, 2, 0, 1], 3), torch.tensor([[4.0, 6.0], [6.0, 7.0], [2.0, 3.0]]))
    with pytest.raises(T.FerrotorchError):
        T.scatter_add_segments(src, [0, 3, 0, 1], 3)
    torch.testing.assert_close(T.gelu_with(x, T.GeluApproximate.Tanh), torch.nn.functional.gelu(x, approximate="tanh"))
    assert T.normalize_axis(-1, 3) == 2 and len(T.chunk_t(x, 2, 2)) == 2
    gx, gy = T.meshgrid(torch.arange(2), torch.arange(3), indexing=T.MeshIndexing.Xy)
    assert gx.shape == (3, 2)


def test_fft_special_masked_dual_sparse():
    torch.manual_seed(1)
    x = torch.randn(4, 8)
    torch.testing.assert_close(T.fft_norm(x, norm=T.FftNorm.Ortho), torch.fft.fft(x, norm="ortho"))
    torch.testing.assert_close(T.irfft2_norm(T.rfft2_norm(x, norm=T.FftNorm.Forward), norm=T.FftNorm.Forward), x)
    assert T.rfftn_differentiable is torch.fft.rfftn and T.fftshift is torch.fft.fftshift
    xr = x.clone().requires_grad_()
    T.rfft_differentiable(xr).abs().sum().backward()
    assert xr.grad is not None
    a, b = torch.tensor([2.0, 3.5]), torch.tensor([3.0, 0.5])
    torch.testing.assert_close(T.beta(a, b)[0], torch.tensor(math.gamma(2) * math.gamma(3) / math.gamma(5)))
    s = T.gammaln_sign(torch.tensor([2.5, -0.5, -1.5, -2.0]))
    assert s[:3].tolist() == [1.0, -1.0, 1.0] and math.isnan(s[3])
    assert T.zeta is torch.special.zeta and T.mvlgamma is torch.special.multigammaln
    d = torch.tensor([1.0, float("nan"), 3.0, float("inf"), 5.0])
    mt = T.masked_invalid(d)
    assert T.masked_sum(mt).item() == 9.0 and T.masked_count(mt).item() == 3.0 and T.masked_mean(mt).item() == 3.0
    assert T.masked_max(T.masked_equal(torch.tensor([1.0, 9.0, 2.0]), 9.0)).item() == 2.0
    assert T.masked_min(T.masked_where(torch.tensor([1.0, 9.0, 2.0]), [True, False, False])).item() == 2.0
    da = ft.autograd.DualTensor(torch.tensor([0.5, 1.0]), torch.ones(2))
    out = T.dual_mul(T.dual_sin(da), T.dual_sigmoid(da))
    ref_t = torch.func.jvp(lambda t: torch.sin(t) * torch.sigmoid(t), (da.primal,), (da.tangent,))[1]
    torch.testing.assert_close(out.tangent, ref_t)
    w = torch.randn(8, 16)
    p = T.magnitude_prune(w, 0.5)
    assert T.sparsity_ratio(p) == 0.5 and torch.equal(p[p != 0], w[p != 0])
    sp = T.to_sparse_semi_structured(w)
    dense = sp.to_dense()
    assert T.sparsity_ratio(dense) >= 0.5 and sp.shape == (8, 16)
    xin = torch.randn(3, 16)
    torch.testing.assert_close(T.sparse_matmul_24(xin, sp), xin @ dense.t(), rtol=1e-4, atol=1e-4)
    assert T.CsrTensor(torch.tensor([0, 1, 2]), torch.tensor([0, 1]), torch.ones(2), (2, 2)).to_dense().trace() == 2
    q = T.fake_quantize_differentiable(torch.tensor([0.26, 100.0]), 0.1, 0)
    torch.testing.assert_close(q, torch.tensor([0.3, 12.7]))
    assert T.QatLayer.__name__ == "QatLinear" and T.cuda_rng.PhiloxGenerator
    with T.AnomalyMode():
        assert T.AnomalyMode.is_enabled()
    with pytest.raises(T.FerrotorchError):
        T.check_gradient_anomaly(d)
    nq = torch.nested.nested_tensor([torch.randn(2, 3, 4), torch.randn(2, 5, 4)])
    assert T.nested_scaled_dot_product_attention(nq, nq, nq).unbind()[1].shape == (2, 5, 4)


def test_umbrella_aliases_and_prelude():
    import importlib

    ns = {}
    exec("from ferrotorch_b200.prelude import *", ns)
    for name in ("Linear", "Conv2d", "BatchNorm2d", "LayerNorm", "Dropout", "Module", "Parameter", "Sequential", "CrossEntropyLoss",
                 "MSELoss", "GELU", "ReLU", "SiLU", "Sigmoid", "Softmax", "Tanh", "GRU", "LSTM", "Adam", "AdamW", "Optimizer",
                 "Sgd", "zeros", "Tensor", "no_grad", "sum_dim", "Device"):
        assert name in ns, name
    assert ft.gpu is ft.cuda and ft.distributed is ft.parallel and ft.tokenize is importlib.import_module("ferrotorch_b200.utils.text")
    assert ft.llama.LlamaConfig is ft.models.LlamaConfig and callable(ft.llama.generate) and ft.llama.GptqQ4 and ft.llama.masked_decode_loop
    assert ft.llama.LlamaKvCache.empty().is_empty() and ft.llama.KVCache is ft.nn.KVCache and ft.grammar.JsonSchemaProcessor and ft.ml.accuracy_score
    assert ft.bert.BertModel and ft.whisper.WhisperEncoder and ft.graph.GcnConv and ft.rl.MlpPolicy and ft.diffusion.DDIMScheduler
    assert ft.jit_script.script is ft.jit.script
