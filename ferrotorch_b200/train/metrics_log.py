"""Run metrics: device-timed step durations, throughput, exposed-communication share and model
FLOP utilisation, written as one JSON line per report per rank and (optionally) as TensorBoard
scalars.

The reference keeps per-epoch metrics in ``TrainingHistory`` (ferrotorch-train/src/history.rs:34-203),
logs every N batches (callback.rs:163) and writes scalars with its own event writer
(tensorboard.rs:314-409); it has no monitor that spans ranks.  Here a step is timed on the device
(a pair of CUDA events on the launching stream; the host clock on CPU), a report takes the
**maximum over ranks** of the window's mean step time (the slowest rank sets the pace of a
synchronous job), and the line carries what a throughput number needs to be read: items per second
for the whole job, the share of the step during which the communication stream ran alone, and the
achieved fraction of a stated FLOP peak.

Events are resolved lazily: ``end_step`` records and returns, the elapsed time is read when a report
is due, so the hot loop never synchronises the device.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field

import torch

from .learner import Callback


class StepTimer:
    """``begin()`` / ``end()`` bracket one step; ``drain()`` returns the milliseconds of every finished
    step since the last drain.  On a CUDA device the brackets are events on the current stream and
    ``drain`` waits for the last one only."""

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self._open = None
        self._pending: list = []

    def begin(self) -> None:
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            self._open = ev
        else:
            self._open = time.perf_counter()

    def end(self) -> None:
        if self._open is None:
            raise RuntimeError("StepTimer.end() without begin()")
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            self._pending.append((self._open, ev))
        else:
            self._pending.append((time.perf_counter() - self._open) * 1e3)
        self._open = None

    def drain(self) -> list[float]:
        out, self._pending = self._pending, []
        if self.cuda and out:
            out[-1][1].synchronize()
            out = [a.elapsed_time(b) for a, b in out]
        return out


@dataclass
class Report:
    step: int
    steps_in_window: int
    ms_per_step: float
    ms_per_step_max_over_ranks: float
    items_per_s: float
    unit: str
    loss: float | None = None
    exposed_comm_frac: float | None = None
    flop_utilisation: float | None = None
    extra: dict = field(default_factory=dict)

    def as_dict(self) -> dict:
        d = {k: v for k, v in self.__dict__.items() if v is not None and k != "extra"}
        d.update(self.extra)
        return d


class MetricsLogger:
    """``step(items, loss=…, exposed_comm_ms=…)`` after every optimiser step; every ``every`` steps
    one :class:`Report` goes to ``<directory>/metrics_rank<r>.jsonl`` and to the TensorBoard writer.

    ``items`` counts what this rank processed in the step (tokens, images); the reported rate is
    the whole job's: the sum over ranks of the window's items divided by the slowest rank's time.
    ``flops_per_item`` and ``peak_flops`` (per device) turn the rate into a utilisation."""

    def __init__(self, directory: str | None = None, *, group=None, device="cpu", unit: str = "tokens", every: int = 10,
                 flops_per_item: float | None = None, peak_flops: float | None = None, tensorboard=None, sink=None):
        self.group, self.unit, self.every = group, unit, max(1, int(every))
        self.rank = group.rank if group is not None else 0
        self.world = group.world_size if group is not None else 1
        self.flops_per_item, self.peak_flops = flops_per_item, peak_flops
        self.timer = StepTimer(device)
        self.tensorboard, self.sink = tensorboard, sink
        self._file = None
        if directory is not None:
            os.makedirs(directory, exist_ok=True)
            self.path = os.path.join(directory, "metrics_rank%d.jsonl" % self.rank)
            self._file = open(self.path, "a", buffering=1)
        self._n = 0
        self._items = 0
        self._comm_ms = 0.0
        self._have_comm = False
        self._loss = None
        self.reports: list[Report] = []

    # ------------------------------------------------------------------ hot loop
    def begin_step(self) -> None:
        self.timer.begin()

    def end_step(self, items: int, loss=None, exposed_comm_ms: float | None = None, **extra) -> Report | None:
        """``loss`` may be a device tensor: it is read only when a report is written."""
        self.timer.end()
        self._n += 1
        self._items += int(items)
        self._loss = loss
        if exposed_comm_ms is not None:
            self._comm_ms += float(exposed_comm_ms)
            self._have_comm = True
        if self._n % self.every == 0:
            return self.report(**extra)
        return None

    # ------------------------------------------------------------------ reporting
    def report(self, **extra) -> Report | None:
        ms = self.timer.drain()
        if not ms:
            return None
        mean_ms = sum(ms) / len(ms)
        stats = torch.tensor([mean_ms, float(self._items)], dtype=torch.float64)
        if self.world > 1:
            allr = self.group.all_gather(stats[None].clone()).reshape(self.world, 2)
            max_ms, items = float(allr[:, 0].max()), float(allr[:, 1].sum())
        else:
            max_ms, items = mean_ms, float(self._items)
        rate = items / (max_ms * len(ms) / 1e3) if max_ms > 0 else 0.0
        loss = self._loss
        if isinstance(loss, torch.Tensor):
            loss = float(loss.detach().float().mean())
        util = None
        if self.flops_per_item and self.peak_flops:
            util = rate * self.flops_per_item / (self.peak_flops * self.world)
        rep = Report(step=self._n, steps_in_window=len(ms), ms_per_step=mean_ms, ms_per_step_max_over_ranks=max_ms,
                     items_per_s=rate, unit=self.unit + "/s", loss=loss,
                     exposed_comm_frac=(self._comm_ms / sum(ms)) if self._have_comm and sum(ms) > 0 else None,
                     flop_utilisation=util, extra=dict(extra, rank=self.rank, world_size=self.world, time=time.time()))
        self._items, self._comm_ms, self._have_comm = 0, 0.0, False
        self.reports.append(rep)
        line = json.dumps(rep.as_dict(), sort_keys=True)
        if self._file is not None:
            self._file.write(line + "\n")
        if self.sink is not None and self.rank == 0:
            self.sink(line)
        if self.tensorboard is not None and self.rank == 0:
            self.tensorboard.add_scalar("throughput/" + self.unit + "_per_s", rep.items_per_s, rep.step)
            self.tensorboard.add_scalar("time/ms_per_step_max_over_ranks", rep.ms_per_step_max_over_ranks, rep.step)
            if rep.loss is not None:
                self.tensorboard.add_scalar("train/loss", rep.loss, rep.step)
            if rep.exposed_comm_frac is not None:
                self.tensorboard.add_scalar("time/exposed_comm_frac", rep.exposed_comm_frac, rep.step)
            if rep.flop_utilisation is not None:
                self.tensorboard.add_scalar("throughput/flop_utilisation", rep.flop_utilisation, rep.step)
        return rep

    def close(self) -> None:
        if self.timer._pending:
            self.report()
        if self._file is not None:
            self._file.close()
            self._file = None


def read_metrics(path: str) -> list[dict]:
    """The reports of one ``metrics_rank<r>.jsonl`` file."""
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


class MetricsCallback(Callback):
    """Feeds a :class:`MetricsLogger` from ``Learner.fit``: a step runs from the end of the previous
    batch to the end of this one (data loading included, which is what a user waits for);
    ``items_of(learner)`` says how many items the last batch held (default: ``learner.last_batch_size``
    when the learner has it, else 1)."""

    def __init__(self, logger: MetricsLogger, items_of=None):
        self.logger, self.items_of = logger, items_of

    def on_train_start(self, learner):
        self.logger.begin_step()

    def on_batch_end(self, learner, epoch, batch_idx, loss):
        n = self.items_of(learner) if self.items_of is not None else getattr(learner, "last_batch_size", 1)
        self.logger.end_step(n, loss=loss, epoch=epoch)
        self.logger.begin_step()

    def on_train_end(self, learner):
        self.logger.timer._open = None
        self.logger.close()
