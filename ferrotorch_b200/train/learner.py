"""``Learner``: fit / evaluate loop with AMP, clipping, EMA, schedulers, callbacks, metrics,
history and per-epoch checkpoints (ferrotorch-train/src/learner.rs:479-790, callback.rs:41-220,
metric.rs:36-301, history.rs:34-203, amp.rs:86-130).

Differences from the reference's loop: the loss is read back once per ``log_every`` batches
instead of every step (learner.rs:581 synchronises each step), EMA stays on the device, and a
:class:`ferrotorch_b200.parallel.host_ddp.DDP` wrapper or a ``FlatTrainer`` plugs in directly
(the reference leaves DDP to the user, ddp.rs:43-54).
"""
from __future__ import annotations

import contextlib
import math
import os
from dataclasses import dataclass, field

from typing import Callable

import torch
from torch import nn

from ..serialize import load_checkpoint, save_checkpoint


# --------------------------------------------------------------------------- metrics
class Metric:
    name = "metric"

    def reset(self): ...
    def update(self, output, target, loss): ...
    def compute(self) -> float: ...


class LossMetric(Metric):
    name = "loss"

    def reset(self):
        self.total, self.n = 0.0, 0

    def update(self, output, target, loss):
        b = target.shape[0] if hasattr(target, "shape") and target.dim() else 1
        self.total += float(loss) * b
        self.n += b

    def compute(self):
        return self.total / max(self.n, 1)


class TopKAccuracy(Metric):
    def __init__(self, k: int = 1):
        self.k, self.name = k, "accuracy" if k == 1 else "top%d_accuracy" % k
        self.reset()

    def reset(self):
        self.correct, self.n = 0, 0

    def update(self, output, target, loss):
        top = output.detach().topk(self.k, dim=-1).indices
        self.correct += int((top == target.unsqueeze(-1)).any(-1).sum())
        self.n += target.numel()

    def compute(self):
        return self.correct / max(self.n, 1)


def AccuracyMetric():
    return TopKAccuracy(1)


class RunningAverage(Metric):
    def __init__(self, momentum: float = 0.98, name: str = "running_loss"):
        self.momentum, self.name = momentum, name
        self.reset()

    def reset(self):
        self.value = None

    def update(self, output, target, loss):
        v = float(loss)
        self.value = v if self.value is None else self.momentum * self.value + (1 - self.momentum) * v

    def compute(self):
        return self.value if self.value is not None else float("nan")

    def window_size(self) -> int:
        """The number of recent values that carry most of the weight: ``1 / (1 - momentum)`` (the
        reference's metric is a plain window of that many values, metric.rs ``RunningAverage``)."""
        return max(1, round(1.0 / max(1e-12, 1.0 - self.momentum)))


# --------------------------------------------------------------------------- history / callbacks
@dataclass
class EpochResult:
    epoch: int
    train: dict
    val: dict | None = None
    lr: float | None = None

    @classmethod
    def new_with_defaults(cls, epoch: int, train_loss: float, val_loss: float | None = None, lr: float | None = None) -> "EpochResult":
        return cls(epoch, {"loss": float(train_loss)}, {"loss": float(val_loss)} if val_loss is not None else None, lr)


@dataclass
class EvalResult:
    """What ``Learner.evaluate`` measured (history.rs ``EvalResult``)."""
    metrics: dict
    num_batches: int = 0

    def get(self, key: str, default=None):
        return self.metrics.get(key, default)

    @classmethod
    def new_with_defaults(cls, loss: float) -> "EvalResult":
        return cls({"loss": float(loss)})


@dataclass
class TrainingHistory:
    epochs: list[EpochResult] = field(default_factory=list)

    def append(self, r: EpochResult):
        self.epochs.append(r)

    def best(self, key: str = "loss", split: str = "val", mode: str = "min"):
        vals = [(getattr(e, split) or {}).get(key) for e in self.epochs]
        vals = [(v, i) for i, v in enumerate(vals) if v is not None]
        if not vals:
            return None
        v, i = (min if mode == "min" else max)(vals)
        return self.epochs[i]

    def series(self, key: str, split: str = "train") -> list:
        return [(getattr(e, split) or {}).get(key) for e in self.epochs]

    # ---- the reference's accessors (ferrotorch-train/src/history.rs:158-210)
    def push(self, result: EpochResult) -> None:
        self.epochs.append(result)

    def __len__(self) -> int:
        return len(self.epochs)

    def len(self) -> int:
        return len(self.epochs)

    def is_empty(self) -> bool:
        return not self.epochs

    def train_losses(self) -> list:
        return self.series("loss", "train")

    def val_losses(self) -> list:
        """One entry per epoch; ``None`` where an epoch had no validation pass."""
        return self.series("loss", "val")

    def _best_loss(self, split: str):
        vals = [(v, i) for i, v in enumerate(self.series("loss", split)) if v is not None]
        if not vals:
            return None
        v, i = min(vals)
        return i, v

    def best_train_loss(self):
        """``(epoch index, loss)`` of the lowest training loss, or ``None`` for an empty history."""
        return self._best_loss("train")

    def best_val_loss(self):
        return self._best_loss("val")


class Callback:
    def on_train_start(self, learner): ...
    def on_epoch_start(self, learner, epoch): ...
    def on_batch_end(self, learner, epoch, batch_idx, loss): ...
    def on_epoch_end(self, learner, result: EpochResult): ...
    def on_train_end(self, learner): ...


class EarlyStopping(Callback):
    def __init__(self, monitor: str = "loss", patience: int = 3, mode: str = "min", min_delta: float = 0.0):
        self.monitor, self.patience, self.mode, self.min_delta = monitor, patience, mode, min_delta
        self.best, self.bad = None, 0

    def on_epoch_end(self, learner, result):
        v = (result.val or result.train).get(self.monitor)
        if v is None:
            return
        better = self.best is None or (v < self.best - self.min_delta if self.mode == "min" else v > self.best + self.min_delta)
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                learner.should_stop = True

    def best_loss(self):
        """The best monitored value so far (``None`` before the first epoch)."""
        return self.best

    def wait(self) -> int:
        """Epochs since the monitored value last improved."""
        return self.bad


class ProgressLogger(Callback):
    def __init__(self, every: int = 50, sink=print):
        self.every, self.sink = every, sink

    def on_batch_end(self, learner, epoch, batch_idx, loss):
        if (batch_idx + 1) % self.every == 0:
            self.sink("epoch %d batch %d loss %.4f" % (epoch, batch_idx + 1, float(loss)))

    def on_epoch_end(self, learner, result):
        self.sink("epoch %d train %s val %s" % (result.epoch, result.train, result.val))


class EMACallback(Callback):
    def __init__(self, decay: float = 0.999):
        self.decay, self.ema = decay, None

    def on_train_start(self, learner):
        from ..optim import EMA

        self.ema = EMA(learner.model, self.decay)

    def on_batch_end(self, learner, epoch, batch_idx, loss):
        self.ema.update()

    # ---- the reference's accessors (callback.rs ``EmaCallback``): usable without a Learner
    def init_from_params(self, params) -> None:
        from ..optim import EMA

        self.ema = EMA(list(params), self.decay)

    def is_initialized(self) -> bool:
        return self.ema is not None

    def update_from_params(self, params=None) -> None:
        if self.ema is None:
            self.init_from_params(params)
        self.ema.update(params)

    def num_updates(self) -> int:
        return self.ema.num_updates() if self.ema is not None else 0

    def shadow_params(self) -> list:
        return self.ema.shadow_params() if self.ema is not None else []


class TensorBoardCallback(Callback):
    def __init__(self, log_dir: str):
        from .tensorboard import TensorBoardWriter

        self.w = TensorBoardWriter(log_dir)

    def on_epoch_end(self, learner, result):
        self.w.add_scalars("train", result.train, result.epoch)
        if result.val:
            self.w.add_scalars("val", result.val, result.epoch)
        self.w.flush()

    def on_train_end(self, learner):
        self.w.close()


# --------------------------------------------------------------------------- AMP
class AmpContext:
    """Autocast + GradScaler in one object (amp.rs:86-130): ``backward_step`` = scale -> backward
    -> unscale -> (clip) -> step (skipped on inf/nan) -> update."""

    def __init__(self, dtype=torch.bfloat16, device_type: str = "cuda", use_scaler: bool | None = None):
        self.dtype, self.device_type = dtype, device_type
        use = (dtype == torch.float16) if use_scaler is None else use_scaler
        self.scaler = torch.amp.GradScaler(device_type, enabled=use and device_type == "cuda")

    def autocast(self):
        return torch.autocast(self.device_type, dtype=self.dtype)

    def backward_step(self, loss, optimizer, params=None, max_grad_norm: float | None = None):
        self.scaler.scale(loss).backward()
        if max_grad_norm is not None and params is not None:
            self.scaler.unscale_(optimizer)
            nn.utils.clip_grad_norm_(params, max_grad_norm)
        self.scaler.step(optimizer)
        self.scaler.update()

    # ---- amp.rs:86-200
    def is_enabled(self) -> bool:
        """Whether reduced-precision autocast is in effect on this device type."""
        return self.dtype in (torch.bfloat16, torch.float16)

    def autocast_forward(self, fn, *args, **kwargs):
        """Run ``fn`` under autocast and return its result."""
        with self.autocast():
            return fn(*args, **kwargs)

    def get_scale(self) -> float:
        return float(self.scaler.get_scale()) if self.scaler.is_enabled() else 1.0

    def scaler_mut(self):
        return self.scaler

    def scaler_state_dict(self) -> dict:
        return self.scaler.state_dict()

    def load_scaler_state_dict(self, state: dict) -> None:
        if state:
            self.scaler.load_state_dict(state)


# --------------------------------------------------------------------------- Learner
class Learner:
    def __init__(self, model: nn.Module, optimizer, loss_fn, *, scheduler=None, metrics=None, callbacks=None,
                 amp: AmpContext | None = None, max_grad_norm: float | None = None, ddp=None, device=None,
                 checkpoint_dir: str | None = None, log_every: int = 10, trainer=None):
        """``trainer``: a :class:`~ferrotorch_b200.train.engine.FlatTrainer` (plain, data-parallel,
        tensor-parallel or hybrid) that owns forward, backward, clipping and the fused update; the
        Learner then drives epochs, callbacks, metrics on the loss, schedules and checkpoints around
        ``trainer.step`` and ``optimizer`` / ``loss_fn`` may be ``None``."""
        self.trainer = trainer
        self.model, self.optimizer, self.loss_fn = model, optimizer, loss_fn
        self.scheduler, self.amp, self.max_grad_norm, self.ddp = scheduler, amp, max_grad_norm, ddp
        self.metrics = metrics if metrics is not None else [LossMetric()]
        self.callbacks = callbacks or []
        self.device = device
        self.checkpoint_dir, self.log_every = checkpoint_dir, log_every
        self.history = TrainingHistory()
        self.epoch, self.global_step, self.should_stop = 0, 0, False

    def with_checkpointing(self, directory: str) -> "Learner":
        self.checkpoint_dir = directory
        return self

    def _to_device(self, t):
        return t.to(self.device, non_blocking=True) if self.device is not None and hasattr(t, "to") else t

    def _forward(self, x, y):
        ctx = self.amp.autocast() if self.amp is not None else contextlib.nullcontext()
        with ctx:
            out = self.model(x)
            loss = self.loss_fn(out, y)
        return out, loss

    def _run_epoch(self, data, train: bool) -> dict:
        for m in self.metrics:
            m.reset()
        self.model.train(train)
        params = [p for p in self.model.parameters() if p.requires_grad]
        for bi, (x, y) in enumerate(data):
            x, y = self._to_device(x), self._to_device(y)
            self.last_batch_size = int(x.shape[0]) if hasattr(x, "shape") and x.dim() else 1
            if train and self.trainer is not None:
                loss = self.trainer.step(x, y)
                out = None
                self.global_step += 1
                for cb in self.callbacks:
                    cb.on_batch_end(self, self.epoch, bi, loss.detach())
            elif train:
                self.optimizer.zero_grad(set_to_none=True)
                out, loss = self._forward(x, y)
                if self.amp is not None and self.ddp is None:
                    self.amp.backward_step(loss, self.optimizer, params, self.max_grad_norm)
                else:
                    loss.backward()
                    if self.ddp is not None:
                        self.ddp.sync_gradients()
                    if self.max_grad_norm is not None:
                        nn.utils.clip_grad_norm_(params, self.max_grad_norm)
                    self.optimizer.step()
                self.global_step += 1
                for cb in self.callbacks:
                    cb.on_batch_end(self, self.epoch, bi, loss.detach())
            elif self.trainer is not None:
                with torch.no_grad():
                    out, loss = None, self.trainer.evaluate(x, y) if hasattr(self.trainer, "evaluate") else self._trainer_loss(x, y)
            else:
                with torch.no_grad():
                    out, loss = self._forward(x, y)
            for m in self.metrics:
                if out is not None or isinstance(m, (LossMetric, RunningAverage)):
                    m.update(out, y, loss.detach())
        return {m.name: m.compute() for m in self.metrics}

    def _trainer_loss(self, x, y):
        """Evaluation loss through the trainer's model: ``model(x, labels=y)`` convention of the
        language models, else ``loss_fn(model(x), y)``."""
        out = self.model(x)
        if self.loss_fn is not None:
            return self.loss_fn(out, y)
        return nn.functional.cross_entropy(out.float().reshape(-1, out.shape[-1]), y.reshape(-1))

    def _lr(self):
        if self.trainer is not None:
            return float(getattr(self.trainer, "lr", 0.0))
        return self.optimizer.param_groups[0]["lr"]

    def fit(self, train_data, val_data=None, epochs: int = 1) -> TrainingHistory:
        for cb in self.callbacks:
            cb.on_train_start(self)
        start = self.epoch
        for epoch in range(start, start + epochs):
            self.epoch = epoch
            for cb in self.callbacks:
                cb.on_epoch_start(self, epoch)
            tr = self._run_epoch(train_data() if callable(train_data) else train_data, True)
            va = self._run_epoch(val_data() if callable(val_data) else val_data, False) if val_data is not None else None
            if self.scheduler is not None:
                if isinstance(self.scheduler, torch.optim.lr_scheduler.ReduceLROnPlateau):
                    self.scheduler.step((va or tr)["loss"])
                else:
                    self.scheduler.step()
            res = EpochResult(epoch, tr, va, self._lr())
            self.history.append(res)
            if self.checkpoint_dir:
                os.makedirs(self.checkpoint_dir, exist_ok=True)
                self.save_checkpoint(os.path.join(self.checkpoint_dir, "checkpoint_epoch_%d.ftc" % epoch))
            for cb in self.callbacks:
                cb.on_epoch_end(self, res)
            self.epoch = epoch + 1
            if self.should_stop:
                break
        for cb in self.callbacks:
            cb.on_train_end(self)
        return self.history

    def evaluate(self, data) -> dict:
        return self._run_epoch(data() if callable(data) else data, False)

    def save_checkpoint(self, path: str) -> None:
        extra = {"rng": torch.get_rng_state().tolist()}
        if self.amp is not None:
            extra["scaler"] = self.amp.scaler.state_dict()
        opt_state = self.trainer.state_dict() if self.trainer is not None else self.optimizer.state_dict()
        save_checkpoint(path, self.model.state_dict(), opt_state, epoch=self.epoch, step=self.global_step, extra=extra)

    def load_checkpoint(self, path: str) -> None:
        ck = load_checkpoint(path)
        self.model.load_state_dict(ck["model"])
        if self.trainer is not None:
            self.trainer.load_state_dict(ck["optimizer"])
        else:
            self.optimizer.load_state_dict(ck["optimizer"])
        self.epoch, self.global_step = ck["epoch"] + 1, ck["step"]
        if "rng" in ck["extra"]:
            torch.set_rng_state(torch.tensor(ck["extra"]["rng"], dtype=torch.uint8))
        if self.amp is not None and ck["extra"].get("scaler"):
            self.amp.scaler.load_state_dict(ck["extra"]["scaler"])


def checkpoint_sequential(functions, segments: int, x: torch.Tensor) -> torch.Tensor:
    """Activation checkpointing over a list of layers in ``segments`` chunks
    (ferrotorch-train/src/checkpoint.rs:113)."""
    from torch.utils.checkpoint import checkpoint

    fns = list(functions)
    per = math.ceil(len(fns) / segments)
    for s in range(0, len(fns), per):
        chunk = fns[s:s + per]

        def run(inp, chunk=chunk):
            for f in chunk:
                inp = f(inp)
            return inp

        x = checkpoint(run, x, use_reentrant=False) if s + per < len(fns) else run(x)
    return x


LossFn = Callable[[torch.Tensor, torch.Tensor], torch.Tensor]      # (prediction, target) -> scalar loss
