"""Configuration objects and the reference's spellings for optimizers and schedulers
(ferrotorch-optim/src/lib.rs re-exports: ``AdamWConfig``, ``SgdConfig``, ..., ``LrScheduler``,
``SequentialLr``, the option enums).  A config holds exactly the keyword arguments of its
optimizer with the optimizer's own defaults (which are torch's, as in the reference:
adamw.rs:68-79, sgd.rs:44-86, rmsprop.rs:61-70), so ``AdamWConfig(lr=3e-4).build(params)`` is
``AdamW(params, lr=3e-4)``.  Where the reference's default differs from torch's (L-BFGS keeps 10
curvature pairs, lbfgs.rs:92, torch 100) torch's value stands: pass ``history_size=10`` for the other."""
from __future__ import annotations

import dataclasses
import enum
import inspect
from typing import Any, Dict, Hashable

import torch
from torch.optim import (ASGD, LBFGS, SGD, Adadelta, Adagrad, Adam, Adamax, AdamW, NAdam, RAdam, RMSprop, Rprop,
                         SparseAdam, lr_scheduler)
from torch.optim.swa_utils import SWALR

from .extra import Adafactor, Kfac, Muon, NaturalGradient, WarmupLR


# the reference's setter names that do not spell a keyword of the optimizer here: name -> (field, how the
# field's new value follows from the config and the argument)
_BUILDER_ALIASES = {
    "AdafactorConfig": {"eps_sq": ("eps", lambda c, v: (v, c.eps[1])), "eps_rms": ("eps", lambda c, v: (c.eps[0], v)),
                        "decay_rate": ("beta2_decay", lambda c, v: -abs(v))},
    "RpropConfig": {"cpu_fallback": ("foreach", lambda c, v: None if v else c.foreach)},
}


def _config_for(opt_cls, name: str):
    fields = []
    for p in list(inspect.signature(opt_cls.__init__).parameters.values())[2:]:      # skip self, params
        if p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        default = p.default if p.default is not inspect.Parameter.empty else None
        if isinstance(default, (list, dict, set)):
            fields.append((p.name, Any, dataclasses.field(default_factory=lambda d=default: type(d)(d))))
        else:
            fields.append((p.name, Any, dataclasses.field(default=default)))

    def build(self, params):
        """The optimizer over ``params`` (an iterable of tensors or of parameter-group dicts)."""
        return opt_cls(params, **dataclasses.asdict(self))

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    ns = {"build": build, "to_dict": to_dict, "optimizer": opt_cls}
    # builder-style setters, ``AdamWConfig().with_lr(3e-4).with_betas((0.9, 0.95))``, as the reference's
    # configs are written (adamw.rs ``with_lr`` ...); each returns a changed copy
    for fname, _t, _f in fields:
        ns["with_" + fname] = (lambda f: lambda self, value: dataclasses.replace(self, **{f: value}))(fname)
    for alias, target in _BUILDER_ALIASES.get(name, {}).items():
        if any(f[0] == target[0] for f in fields):
            ns["with_" + alias] = (lambda t: lambda self, value=True: dataclasses.replace(self, **{t[0]: t[1](self, value)}))(target)
    cls = dataclasses.make_dataclass(name, fields, namespace=ns)
    cls.__doc__ = "Keyword arguments of :class:`%s` with its defaults." % opt_cls.__name__
    cls.__module__ = __name__
    return cls


SgdConfig = _config_for(SGD, "SgdConfig")
AdamConfig = _config_for(Adam, "AdamConfig")
AdamWConfig = _config_for(AdamW, "AdamWConfig")
AdamaxConfig = _config_for(Adamax, "AdamaxConfig")
NAdamConfig = _config_for(NAdam, "NAdamConfig")
RAdamConfig = _config_for(RAdam, "RAdamConfig")
AdagradConfig = _config_for(Adagrad, "AdagradConfig")
AdadeltaConfig = _config_for(Adadelta, "AdadeltaConfig")
AdafactorConfig = _config_for(Adafactor, "AdafactorConfig")
RmspropConfig = _config_for(RMSprop, "RmspropConfig")
RpropConfig = _config_for(Rprop, "RpropConfig")
AsgdConfig = _config_for(ASGD, "AsgdConfig")
SparseAdamConfig = _config_for(SparseAdam, "SparseAdamConfig")
LbfgsConfig = _config_for(LBFGS, "LbfgsConfig")
MuonConfig = _config_for(Muon, "MuonConfig")
KfacConfig = _config_for(Kfac, "KfacConfig")
NaturalGradientConfig = _config_for(NaturalGradient, "NaturalGradientConfig")

Sgd, Asgd, Lbfgs, Rmsprop = SGD, ASGD, LBFGS, RMSprop
LrScheduler = lr_scheduler.LRScheduler
SequentialLr = lr_scheduler.SequentialLR
MetricScheduler = lr_scheduler.ReduceLROnPlateau      # the schedulers that step on a metric
Swalr = SWALR
LinearWarmup = WarmupLR

ParamKey = Hashable
ParamGroup = Dict[str, Any]
OptimizerState = Dict[str, Any]


class _StrEnum(str, enum.Enum):
    def __str__(self) -> str:
        return self.value


class AnnealStrategy(_StrEnum):
    Cos = "cos"; Linear = "linear"  # noqa: E702


class CyclicMode(_StrEnum):
    Triangular = "triangular"; Triangular2 = "triangular2"; ExpRange = "exp_range"  # noqa: E702


class PlateauMode(_StrEnum):
    Min = "min"; Max = "max"  # noqa: E702


class ThresholdMode(_StrEnum):
    Rel = "rel"; Abs = "abs"  # noqa: E702


class LineSearchFn(_StrEnum):
    StrongWolfe = "strong_wolfe"


class AveragingStrategy(enum.Enum):
    """How an averaged model folds in new weights (swa.rs): equal-weight running mean or an
    exponential moving average with ``decay``."""
    Swa = "swa"
    Ema = "ema"

    def avg_fn(self, decay: float = 0.999):
        from torch.optim.swa_utils import get_ema_multi_avg_fn, get_swa_multi_avg_fn

        return get_swa_multi_avg_fn() if self is AveragingStrategy.Swa else get_ema_multi_avg_fn(decay)


@dataclasses.dataclass
class GradScalerConfig:
    init_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    enabled: bool = True

    def build(self, device: str = "cuda"):
        from torch.amp import GradScaler

        return GradScaler(device, **dataclasses.asdict(self))


for _f in dataclasses.fields(GradScalerConfig):
    setattr(GradScalerConfig, "with_" + _f.name, (lambda f: lambda self, value: dataclasses.replace(self, **{f: value}))(_f.name))


@dataclasses.dataclass
class GradScalerState:
    scale: float
    growth_tracker: int

    @classmethod
    def of(cls, scaler) -> "GradScalerState":
        sd = scaler.state_dict()
        return cls(float(sd.get("scale", 1.0)), int(sd.get("_growth_tracker", 0)))

    def restore(self, scaler) -> None:
        sd = scaler.state_dict()
        if sd:                                              # a disabled scaler has no state
            sd.update(scale=self.scale, _growth_tracker=self.growth_tracker)
            scaler.load_state_dict(sd)

__all__ = [_n for _n, _o in list(globals().items())
           if not _n.startswith("_") and type(_o).__name__ != "module" and _n not in ("annotations", "Callable", "Dict", "Any", "Hashable")]
