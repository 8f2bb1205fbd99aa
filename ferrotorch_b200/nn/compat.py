"""Names of the reference's ``ferrotorch-nn`` surface that torch spells differently or keeps in
sub-modules (ferrotorch-nn/src/lib.rs re-exports): functional forms at package level, option
enums, score modifiers for ``flex_attention`` (flex_attention.rs:723-784), head reshapes
(attention.rs:606-660), packed sequences (rnn_utils.rs)."""
from __future__ import annotations

import enum
from typing import Callable, Dict

import torch
from torch import nn
from torch.nn.functional import (adaptive_avg_pool1d, adaptive_avg_pool2d, adaptive_avg_pool3d,  # noqa: F401
                                 adaptive_max_pool1d, adaptive_max_pool2d, adaptive_max_pool3d, affine_grid,
                                 avg_pool1d, avg_pool2d, avg_pool3d, fold, grid_sample, interpolate, lp_pool1d,
                                 lp_pool2d, max_pool1d, max_pool2d, max_pool3d, max_unpool2d, pixel_shuffle,
                                 pixel_unshuffle, unfold)
from torch.nn.utils.rnn import PackedSequence, pack_padded_sequence, pad_packed_sequence, pad_sequence  # noqa: F401

from .fake_quant import convert as _convert_qat, prepare_qat as _prepare_qat
from .paged import PagePool  # noqa: F401

HardSigmoid, HardSwish = nn.Hardsigmoid, nn.Hardswish
StateDict = Dict[str, torch.Tensor]
ForwardHook = Callable[[nn.Module, tuple, object], object]
ForwardPreHook = Callable[[nn.Module, tuple], object]
BackwardHook = Callable[[nn.Module, tuple, tuple], object]


class _StrEnum(str, enum.Enum):
    def __str__(self) -> str:          # usable wherever torch wants the option string
        return self.value


class Reduction(_StrEnum):
    Mean = "mean"; Sum = "sum"; NoReduction = "none"  # noqa: E702


class PaddingMode(_StrEnum):
    Zeros = "zeros"; Reflect = "reflect"; Replicate = "replicate"; Circular = "circular"  # noqa: E702


class StringPadding(_StrEnum):
    Valid = "valid"; Same = "same"  # noqa: E702


class InterpolateMode(_StrEnum):
    Nearest = "nearest"; Bilinear = "bilinear"; Bicubic = "bicubic"; Linear = "linear"; Trilinear = "trilinear"; Area = "area"  # noqa: E702


class GridSampleMode(_StrEnum):
    Bilinear = "bilinear"; Nearest = "nearest"; Bicubic = "bicubic"  # noqa: E702


class GridSamplePaddingMode(_StrEnum):
    Zeros = "zeros"; Border = "border"; Reflection = "reflection"  # noqa: E702


class GeluApproximate(_StrEnum):
    NoApproximation = "none"; Tanh = "tanh"  # noqa: E702


class EmbeddingBagMode(_StrEnum):
    Sum = "sum"; Mean = "mean"; Max = "max"  # noqa: E702


class RNNNonlinearity(_StrEnum):
    Tanh = "tanh"; ReLU = "relu"  # noqa: E702


class FanMode(_StrEnum):
    FanIn = "fan_in"; FanOut = "fan_out"  # noqa: E702


class NonLinearity(_StrEnum):
    Linear = "linear"; ReLU = "relu"; LeakyReLU = "leaky_relu"; Tanh = "tanh"; Sigmoid = "sigmoid"; SELU = "selu"  # noqa: E702

    def gain(self, param: float | None = None) -> float:
        return nn.init.calculate_gain(self.value, param)


class ObserverType(_StrEnum):
    MinMax = "minmax"; MovingAverage = "moving_average"  # noqa: E702


class RoPEConvention(_StrEnum):
    HalfRotation = "half"; Interleaved = "interleaved"  # noqa: E702


class RoPEScaling:
    """Constructors for the ``scaling`` dictionary of ``RotaryPositionEmbedding``
    (transformer.rs:227-278: None / Linear / NTK-aware / YaRN)."""

    NoScaling = None

    @staticmethod
    def Linear(factor: float) -> dict:
        return {"type": "linear", "factor": float(factor)}

    @staticmethod
    def NtkAware(factor: float) -> dict:
        return {"type": "ntk", "factor": float(factor)}

    @staticmethod
    def Yarn(factor: float, original_max_pos_embeddings: int, beta_fast: float = 32.0, beta_slow: float = 1.0) -> dict:
        return {"type": "yarn", "factor": float(factor), "original_max": int(original_max_pos_embeddings),
                "beta_fast": float(beta_fast), "beta_slow": float(beta_slow)}


# --------------------------------------------------------------------------- flex_attention score modifiers
# called with broadcastable index tensors, so each works on the whole score matrix at once
def causal_score_mod():
    return lambda score, b, h, q_idx, kv_idx: torch.where(q_idx >= kv_idx, score, torch.full_like(score, -1e30))


def alibi_score_mod(slope):
    """``score + slope * (q - k)``; ``slope`` a number or one value per head ``[H]``."""
    def mod(score, b, h, q_idx, kv_idx):
        s = slope[h] if isinstance(slope, torch.Tensor) and slope.dim() else slope
        return score + s * (q_idx - kv_idx).to(score.dtype)
    return mod


def relative_position_bias_score_mod(bias_table: torch.Tensor, max_dist: int):
    """``score + table[clamp(q - k, -max_dist, max_dist) + max_dist]``."""
    def mod(score, b, h, q_idx, kv_idx):
        idx = ((q_idx - kv_idx).clamp(-max_dist, max_dist) + max_dist).clamp(max=bias_table.numel() - 1)
        return score + bias_table.to(score.device, score.dtype)[idx.long()]
    return mod


# --------------------------------------------------------------------------- head reshapes
def reshape_to_heads(t: torch.Tensor, num_heads: int, seq_len: int, head_dim: int) -> torch.Tensor:
    """``[S, H*D] -> [H, S, D]``."""
    return t.reshape(seq_len, num_heads, head_dim).transpose(0, 1).contiguous()


def transpose_heads_to_2d(t: torch.Tensor, num_heads: int, seq_len: int, head_dim: int) -> torch.Tensor:
    """``[H, S, D] -> [S, H*D]``."""
    return t.reshape(num_heads, seq_len, head_dim).transpose(0, 1).reshape(seq_len, num_heads * head_dim).contiguous()


# --------------------------------------------------------------------------- QAT wrappers
class QatConfig:
    def __init__(self, weight_bits: int = 8, activation_bits: int = 8, observer: ObserverType = ObserverType.MinMax,
                 skip: tuple = ()):
        self.weight_bits, self.activation_bits, self.observer, self.skip = weight_bits, activation_bits, observer, tuple(skip)

    # presets (ferrotorch-nn/src/qat.rs ``impl QatConfig``)
    @classmethod
    def default_symmetric_int8(cls) -> "QatConfig":
        return cls(8, 8)

    @classmethod
    def per_channel_int8(cls) -> "QatConfig":
        """8-bit weights with one scale per output channel (what ``QatLinear`` always uses) and 8-bit activations."""
        return cls(8, 8, ObserverType.MinMax)

    @classmethod
    def int4_weight_int8_activation(cls) -> "QatConfig":
        return cls(4, 8)


class QuantizedModel:
    """Result of :meth:`QatModel.convert`: ``{layer name: (int8 weight, scale, zero point)}``."""

    def __init__(self, layers: dict, config: "QatConfig | None" = None):
        self.layers, self.config = layers, config or QatConfig()
        self.bits = self.config.weight_bits

    def __len__(self) -> int:
        return len(self.layers)

    # ---- qat.rs ``QuantizedModel`` accessors
    def weight_names(self) -> list:
        return sorted(self.layers)

    def num_weights(self) -> int:
        return len(self.layers)

    def weight(self, name: str) -> torch.Tensor:
        """The integer weight of layer ``name``."""
        return self._entry(name)[0]

    def weight_qparams(self, name: str):
        """``(scale, zero_point)`` of layer ``name``."""
        e = self._entry(name)
        return e[1], e[2]

    def dequantize_weight(self, name: str) -> torch.Tensor:
        return self.dequantized_state_dict()[name + ".weight"]

    def quantized_size_bytes(self) -> int:
        """Bytes of the integer weights at their nominal width plus fp32 scales."""
        total = 0
        for q, scale, _zp in (self._entry(n) for n in self.layers):
            total += (q.numel() * self.bits + 7) // 8 + scale.numel() * 4
        return total

    def compression_ratio(self) -> float:
        """fp32 bytes of the same weights over :meth:`quantized_size_bytes`."""
        dense = 0
        for n in self.layers:
            dense += self._entry(n)[0].numel() * 4
        return dense / self.quantized_size_bytes() if self.layers else 1.0

    def _entry(self, name: str):
        if name not in self.layers:
            raise KeyError("no quantised layer %r (have %s)" % (name, sorted(self.layers)))
        q, scale, zp = self.layers[name]
        return q, scale, (zp if torch.is_tensor(zp) and zp.dtype != q.dtype and zp.numel() == scale.numel() else torch.zeros_like(scale))

    def dequantized_state_dict(self) -> dict:
        out = {}
        for name, (q, scale, zp) in self.layers.items():
            s = scale.reshape(-1, *[1] * (q.dim() - 1)) if scale.numel() > 1 else scale
            z = zp.reshape(-1, *[1] * (q.dim() - 1)) if zp.numel() > 1 else zp
            out[name + ".weight"] = (q.float() - z.float()) * s.float()
        return out


class QatModel(nn.Module):
    """A model prepared for quantisation-aware training (qat.rs:182 ``prepare_qat``)."""

    def __init__(self, model: nn.Module, config: QatConfig | None = None):
        super().__init__()
        self.config = config or QatConfig()
        self.model = _prepare_qat(model, self.config.weight_bits, self.config.activation_bits, self.config.skip)

    def forward(self, *a, **kw):
        return self.model(*a, **kw)

    def convert(self) -> QuantizedModel:
        return QuantizedModel(_convert_qat(self.model), self.config)

    # ---- qat.rs ``QatModel``
    def _layers(self) -> dict:
        from .fake_quant import QatLinear

        return {n: m for n, m in self.model.named_modules() if isinstance(m, QatLinear)}

    def register_layer(self, name: str) -> None:
        """Swap the ``nn.Linear`` called ``name`` (a dotted path) for its fake-quantised form, e.g. one that
        was listed in ``skip`` when the model was prepared."""
        from .fake_quant import QatLinear

        parent, _, leaf = name.rpartition(".")
        owner = self.model.get_submodule(parent) if parent else self.model
        lin = getattr(owner, leaf)
        if isinstance(lin, QatLinear):
            return
        if not isinstance(lin, nn.Linear):
            raise TypeError("register_layer: %r is a %s, not a Linear" % (name, type(lin).__name__))
        setattr(owner, leaf, QatLinear.from_float(lin, self.config.weight_bits, self.config.activation_bits))

    def fake_quantize_weights(self, enabled: bool = True) -> "QatModel":
        for m in self._layers().values():
            m.weight_fq.enabled = bool(enabled)
        return self

    def fake_quantize_activations(self, enabled: bool = True) -> "QatModel":
        for m in self._layers().values():
            m.act_fq.enabled = bool(enabled)
        return self


KVPage = tuple      # (layer, page index): pages are slices of the pool's device tensors, addressed by index



# --------------------------------------------------------------------------- free functions of functional.rs / padding.rs / init.rs
def _mode(mode) -> str:
    m = str(getattr(mode, "value", mode)).lower()
    return {"zeros": "constant", "zero": "constant", "constant": "constant", "reflect": "reflect", "replicate": "replicate",
            "circular": "circular"}.get(m, m)


def functional_pad_1d(x, pad_left: int, pad_right: int, mode="constant", value: float = 0.0):
    """Pad the last dimension; ``mode``: constant / reflect / replicate / circular.  Negative amounts crop
    (the ``_signed`` spelling of the reference takes signed amounts; Python integers are signed anyway)."""
    m = _mode(mode)
    return nn.functional.pad(x, (pad_left, pad_right), m, value if m == "constant" else None)


def functional_pad_2d(x, pad_left: int, pad_right: int, pad_top: int, pad_bottom: int, mode="constant", value: float = 0.0):
    m = _mode(mode)
    return nn.functional.pad(x, (pad_left, pad_right, pad_top, pad_bottom), m, value if m == "constant" else None)


def functional_pad_3d(x, pad_left: int, pad_right: int, pad_top: int, pad_bottom: int, pad_front: int, pad_back: int,
                      mode="constant", value: float = 0.0):
    m = _mode(mode)
    return nn.functional.pad(x, (pad_left, pad_right, pad_top, pad_bottom, pad_front, pad_back), m, value if m == "constant" else None)


functional_pad_1d_signed, functional_pad_2d_signed, functional_pad_3d_signed = functional_pad_1d, functional_pad_2d, functional_pad_3d


def gelu_with(x, approximate="none"):
    return nn.functional.gelu(x, approximate=str(getattr(approximate, "value", approximate)).lower())


def elu_with(x, alpha: float = 1.0):
    return nn.functional.elu(x, alpha)


def softplus_with(x, beta: float = 1.0, threshold: float = 20.0):
    return nn.functional.softplus(x, beta, threshold)


def hardtanh_with(x, min_val: float = -1.0, max_val: float = 1.0):
    return nn.functional.hardtanh(x, min_val, max_val)


def log_sigmoid(x):
    return nn.functional.logsigmoid(x)


def sum(x):  # noqa: A001 - the reference's functional module exports the full reductions under these names
    return x.sum()


def mean(x):
    return x.mean()


def zeros(param):
    """Initialiser: fill with zeros (init.rs:93)."""
    return nn.init.zeros_(param)


def ones(param):
    return nn.init.ones_(param)


def _fan(param, mode) -> int:
    fan_in, fan_out = nn.init._calculate_fan_in_and_fan_out(param)
    return fan_in if str(getattr(mode, "value", mode)).lower() in ("fan_in", "fanin") else fan_out


def _gain(nonlinearity, a: float = 0.0) -> float:
    return nn.init.calculate_gain(str(getattr(nonlinearity, "value", nonlinearity)).lower(), a)


def kaiming_normal_with_fan_mode_and_generator(param, nonlinearity="relu", mode="fan_in", generator=None, a: float = 0.0):
    with torch.no_grad():
        return param.normal_(0.0, _gain(nonlinearity, a) / _fan(param, mode) ** 0.5, generator=generator)


def kaiming_uniform_with_fan_mode_and_generator(param, nonlinearity="relu", mode="fan_in", generator=None, a: float = 0.0):
    bound = 3.0 ** 0.5 * _gain(nonlinearity, a) / _fan(param, mode) ** 0.5
    with torch.no_grad():
        return param.uniform_(-bound, bound, generator=generator)


def kaiming_normal_with_fan_mode(param, nonlinearity="relu", mode="fan_in"):
    return kaiming_normal_with_fan_mode_and_generator(param, nonlinearity, mode)


def kaiming_uniform_with_fan_mode(param, nonlinearity="relu", mode="fan_in"):
    return kaiming_uniform_with_fan_mode_and_generator(param, nonlinearity, mode)


def kaiming_normal_with_generator(param, nonlinearity="relu", generator=None):
    return kaiming_normal_with_fan_mode_and_generator(param, nonlinearity, "fan_in", generator)


def kaiming_uniform_with_generator(param, nonlinearity="relu", generator=None):
    return kaiming_uniform_with_fan_mode_and_generator(param, nonlinearity, "fan_in", generator)


def xavier_normal_with_generator(param, gain: float = 1.0, generator=None):
    return nn.init.xavier_normal_(param, gain, generator=generator)


def xavier_uniform_with_generator(param, gain: float = 1.0, generator=None):
    return nn.init.xavier_uniform_(param, gain, generator=generator)


def normal_with_generator(param, mean: float = 0.0, std: float = 1.0, generator=None):
    return nn.init.normal_(param, mean, std, generator=generator)


def uniform_with_generator(param, a: float = 0.0, b: float = 1.0, generator=None):
    return nn.init.uniform_(param, a, b, generator=generator)


def trunc_normal_with_generator(param, mean: float = 0.0, std: float = 1.0, a: float = -2.0, b: float = 2.0, generator=None):
    return nn.init.trunc_normal_(param, mean, std, a, b, generator=generator)


def orthogonal_with_generator(param, gain: float = 1.0, generator=None):
    return nn.init.orthogonal_(param, gain, generator=generator)


def sparse_with_generator(param, sparsity: float, std: float = 0.01, generator=None):
    return nn.init.sparse_(param, sparsity, std, generator=generator)


__all__ = [_n for _n, _o in list(globals().items())
           if not _n.startswith("_") and type(_o).__name__ != "module" and _n not in ("annotations", "Callable", "Dict", "Any", "Hashable")]
