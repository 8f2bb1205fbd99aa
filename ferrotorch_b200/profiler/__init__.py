"""Profiler: op / kernel ranges timed with CUDA events, a wait-warmup-active schedule, memory
records, FLOP estimates, table / Chrome-trace / TensorBoard output.

Reference: ``with_profiler`` (ferrotorch-profiler/src/profiler.rs:459), CUDA-event kernel scopes
flushed after a synchronise (cuda_timing.rs:71-119, profiler.rs:302-329), ``ProfileSchedule``
(schedule.rs:74-200), reports (report.rs:259, 446-478, 524), ``flops::estimate`` (flops.rs:53).
"""
from __future__ import annotations

import contextlib
import json
import time
import enum
from dataclasses import dataclass, field

import torch


@dataclass
class ProfileEvent:
    name: str
    category: str
    start_us: float
    dur_us: float
    device: str = "cpu"
    shapes: tuple = ()
    flops: float | None = None
    bytes: int | None = None


@dataclass
class ProfileConfig:
    record_shapes: bool = True
    record_memory: bool = False
    with_flops: bool = True
    cuda_events: bool = True
    nvtx: bool = False          # also open an NVTX range per scope (shows up in Nsight timelines)


class ProfileSchedule:
    """``wait`` steps idle, ``warmup`` steps running but discarded, ``active`` steps recorded,
    repeated ``repeat`` times (0 = forever); ``on_trace_ready(profiler)`` fires after each cycle."""

    def __init__(self, wait: int = 0, warmup: int = 0, active: int = 1, repeat: int = 1, on_trace_ready=None):
        self.wait, self.warmup, self.active, self.repeat, self.on_trace_ready = wait, warmup, active, repeat, on_trace_ready
        self.step_num = 0

    def state(self) -> str:
        cycle = self.wait + self.warmup + self.active
        if self.repeat and self.step_num >= cycle * self.repeat:
            return "done"
        pos = self.step_num % cycle
        return "wait" if pos < self.wait else "warmup" if pos < self.wait + self.warmup else "active"

    def cycle_finished(self) -> bool:
        cycle = self.wait + self.warmup + self.active
        return self.step_num > 0 and self.step_num % cycle == 0

    # ---- the reference's accessors (schedule.rs:163-240)
    def set_on_trace_ready(self, callback) -> None:
        """``callback(cycle_number)`` after the last active step of every cycle (zero-based)."""
        self._cycle_cb = callback

    def phase(self) -> str:
        return self.state()

    def is_active(self) -> bool:
        return self.state() == "active"

    def current_step(self) -> int:
        return self.step_num

    def current_cycle(self) -> int:
        return self.step_num // (self.wait + self.warmup + self.active)

    def step(self) -> str:
        """Advance one step; returns the phase the schedule is in afterwards."""
        self.step_num += 1
        cycle = self.wait + self.warmup + self.active
        cb = getattr(self, "_cycle_cb", None)
        if cb is not None and self.cycle_finished() and (not self.repeat or self.step_num <= cycle * self.repeat):
            cb(self.step_num // cycle - 1)
        return self.state()


def estimate_flops(op: str, shapes) -> float | None:
    """FLOPs from shapes for the common ops (flops.rs:53)."""
    try:
        if op in ("matmul", "mm", "linear", "gemm"):
            a, b = shapes[0], shapes[1]
            m = 1
            for d in a[:-1]:
                m *= d
            n = b[0] if op == "linear" else b[-1]
            return 2.0 * m * a[-1] * n
        if op == "attention":
            b, s, h, d = shapes[0]
            sk = shapes[1][1]
            return 4.0 * b * h * s * sk * d
        if op in ("add", "mul", "relu", "sub", "div"):
            n = 1
            for d in shapes[0]:
                n *= d
            return float(n)
    except Exception:  # noqa: BLE001
        return None
    return None


def estimate(op_name: str, input_shapes):
    """FLOPs of an op from its input shapes as an integer, ``None`` for an op without a formula (flops.rs:53)."""
    v = estimate_flops(op_name, [tuple(s) for s in input_shapes])
    return None if v is None else int(v)


class Profiler:
    _current: "Profiler | None" = None

    def __init__(self, config: ProfileConfig | None = None, schedule: ProfileSchedule | None = None):
        self.cfg, self.schedule = config or ProfileConfig(), schedule
        self.events: list[ProfileEvent] = []
        self.memory: list[tuple[float, str, int]] = []
        self.memory_categories: list[tuple[str, int]] = []
        self._pending: list = []
        self._t0 = time.perf_counter()
        self._stopped = False

    # ---- recording
    def _recording(self) -> bool:
        return not self._stopped and (self.schedule is None or self.schedule.state() == "active")

    def is_active(self) -> bool:
        return self._recording()

    def stop(self) -> None:
        """Later ``scope`` / ``record*`` calls record nothing; what was recorded stays (profiler.rs:263)."""
        self._stopped = True

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    @contextlib.contextmanager
    def scope(self, name: str, category: str = "op", shapes=(), op: str | None = None, nbytes: int | None = None):
        """Time a region.  On CUDA the region is bracketed by events on the current stream; the
        elapsed time is read at :meth:`flush` (no synchronisation inside the region)."""
        if not self._recording():
            yield
            return
        use_cuda = self.cfg.cuda_events and torch.cuda.is_available() and category in ("kernel", "cuda", "op")
        start = self._now_us()
        if use_cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        nvtx = self.cfg.nvtx and torch.cuda.is_available()
        if nvtx:
            torch.cuda.nvtx.range_push("%s:%s" % (category, name))
        try:
            yield
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()
            flops = estimate_flops(op or name, shapes) if self.cfg.with_flops and shapes else None
            ev = ProfileEvent(name, category, start, self._now_us() - start, "cpu",
                              tuple(shapes) if self.cfg.record_shapes else (), flops, nbytes)
            self.events.append(ev)
            if use_cuda:
                e1.record()
                self._pending.append((ev, e0, e1))
            if self.cfg.record_memory and torch.cuda.is_available():
                self.record_memory(name, torch.cuda.memory_allocated())

    def record(self, name: str, dur_us: float, category: str = "manual") -> None:
        if self._recording():
            self.events.append(ProfileEvent(name, category, self._now_us(), dur_us))

    def record_with_duration(self, name: str, category: str, duration_us: float) -> None:
        """The reference's argument order (profiler.rs:155)."""
        self.record(name, duration_us, category)

    def record_memory_categorized(self, name: str, nbytes: int, category: str = "other") -> None:
        """A memory event (positive = allocation, negative = free) filed under a
        :class:`MemoryCategory`; :meth:`ProfileReport.memory_by_category` nets them per category."""
        if self._recording():
            self.memory.append((self._now_us(), name, int(nbytes)))
            self.memory_categories.append((str(category), int(nbytes)))

    def flush_cuda_kernels(self) -> None:
        self.flush()

    def pending_cuda_count(self) -> int:
        """Device scopes recorded but not yet read back (read by :meth:`flush`)."""
        return len(self._pending)

    def push_gpu_event(self, name: str, timing: "GpuTimingPair", category: str = "kernel") -> None:
        """Add a device interval measured elsewhere (profiler.rs:200): duration = end - start, never negative."""
        self.events.append(ProfileEvent(name, category, float(timing.start_us), float(timing.duration_us()), str(DeviceType.Cuda)))

    def record_memory(self, tag: str, nbytes: int) -> None:
        self.memory.append((self._now_us(), tag, int(nbytes)))

    def flush(self) -> None:
        """Synchronise and convert pending CUDA event pairs into device durations."""
        if self._pending:
            torch.cuda.synchronize()
            for ev, e0, e1 in self._pending:
                self.events.append(ProfileEvent(ev.name, ev.category, ev.start_us, e0.elapsed_time(e1) * 1e3, "cuda",
                                                ev.shapes, ev.flops, ev.bytes))
            self._pending.clear()

    def step(self) -> None:
        if self.schedule is None:
            return
        self.schedule.step()
        if self.schedule.cycle_finished():
            self.flush()
            if self.schedule.on_trace_ready is not None:
                self.schedule.on_trace_ready(self)

    # ---- reports
    def summary(self) -> dict:
        self.flush()
        agg: dict = {}
        for e in self.events:
            k = (e.name, e.device)
            a = agg.setdefault(k, {"name": e.name, "device": e.device, "count": 0, "total_us": 0.0, "flops": 0.0})
            a["count"] += 1
            a["total_us"] += e.dur_us
            a["flops"] += e.flops or 0.0
        return agg

    def report(self) -> "ProfileReport":
        return ProfileReport(self)

    def table(self, sort_by: str = "total_us") -> str:
        rows = sorted(self.summary().values(), key=lambda a: -a[sort_by])
        out = ["%-32s %-5s %8s %12s %12s %10s" % ("name", "dev", "calls", "total us", "avg us", "TFLOP/s")]
        for a in rows:
            tf = a["flops"] / a["total_us"] / 1e6 if a["flops"] and a["total_us"] else 0.0
            out.append("%-32s %-5s %8d %12.1f %12.1f %10.2f" % (a["name"][:32], a["device"], a["count"], a["total_us"],
                                                                  a["total_us"] / a["count"], tf))
        return "\n".join(out)

    def chrome_trace_json(self) -> str:
        self.flush()
        ev = [{"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": e.dur_us,
               "pid": 0, "tid": 1 if e.device == "cuda" else 0, "args": {"shapes": list(e.shapes), "flops": e.flops}}
              for e in self.events]
        ev += [{"name": "memory", "ph": "C", "ts": t, "pid": 0, "args": {tag: b}} for t, tag, b in self.memory]
        return json.dumps({"traceEvents": ev, "displayTimeUnit": "ms"})

    def export_chrome_trace(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.chrome_trace_json())

    def export_tensorboard(self, log_dir: str, step: int = 0) -> None:
        from ..train.tensorboard import TensorBoardWriter

        w = TensorBoardWriter(log_dir)
        for a in self.summary().values():
            w.add_scalar("profile/%s/%s_us" % (a["device"], a["name"]), a["total_us"], step)
        w.close()


# --------------------------------------------------------------------------- report objects
class SchedulePhase:
    """The states :meth:`ProfileSchedule.state` returns (schedule.rs ``SchedulePhase``)."""
    WAIT, WARMUP, ACTIVE, DONE = "wait", "warmup", "active", "done"


class MemoryCategory:
    """Tags for :meth:`Profiler.record_memory` (event.rs ``MemoryCategory``)."""
    PARAMETERS, GRADIENTS, OPTIMIZER_STATE, ACTIVATIONS, TEMPORARY, OTHER = (
        "parameters", "gradients", "optimizer_state", "activations", "temporary", "other")


@dataclass
class OpSummary:
    name: str
    device: str
    count: int
    total_us: float
    flops: float = 0.0

    @property
    def avg_us(self) -> float:
        return self.total_us / self.count if self.count else 0.0

    @property
    def tflops(self) -> float:
        return self.flops / self.total_us / 1e6 if self.flops and self.total_us else 0.0


class ProfileReport:
    """The events of a run and their per-op totals, detached from the profiler that took them
    (report.rs ``ProfileReport``): ``ops()``, ``top(n)``, ``total_us()``, ``table()``,
    ``chrome_trace_json()``, ``save_chrome_trace(path)``."""

    def __init__(self, profiler: "Profiler"):
        profiler.flush()
        self.events = list(profiler.events)
        self.memory = list(profiler.memory)
        self._memory_categories = list(profiler.memory_categories)
        self._ops = [OpSummary(a["name"], a["device"], a["count"], a["total_us"], a["flops"])
                     for a in profiler.summary().values()]
        self._table, self._trace = profiler.table(), profiler.chrome_trace_json()

    def ops(self) -> list[OpSummary]:
        return sorted(self._ops, key=lambda o: -o.total_us)

    def top(self, n: int = 10) -> list[OpSummary]:
        return self.ops()[:n]

    def total_us(self, device: str | None = None) -> float:
        return sum(o.total_us for o in self._ops if device is None or o.device == device)

    def table(self) -> str:
        return self._table

    def chrome_trace_json(self) -> str:
        return self._trace

    def save_chrome_trace(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self._trace)

    # ---- the reference's accessors (report.rs:94-560)
    def top_ops(self, n: int = 10) -> list[OpSummary]:
        return self.top(n)

    def total_time_us(self) -> float:
        return self.total_us()

    def has_gpu_events(self) -> bool:
        return any(e.device == "cuda" for e in self.events)

    def has_stack_traces(self) -> bool:
        return False                      # ranges are named by the caller; no stacks are collected

    def total_flops(self) -> float:
        """FLOPs of the recorded ranges; a range timed on both clocks is counted once."""
        seen_dev = {(e.name, e.start_us) for e in self.events if e.device == "cuda"}
        return float(sum(e.flops or 0.0 for e in self.events if e.device == "cuda" or (e.name, e.start_us) not in seen_dev))

    def flops_per_second(self) -> float:
        """Total FLOPs over the time of the ranges that carry a FLOP count (device time where there is one)."""
        seen_dev = {(e.name, e.start_us) for e in self.events if e.device == "cuda"}
        us = sum(e.dur_us for e in self.events if e.flops and (e.device == "cuda" or (e.name, e.start_us) not in seen_dev))
        return self.total_flops() / (us * 1e-6) if us > 0 else 0.0

    def memory_by_category(self) -> list[tuple[str, int]]:
        """Net bytes per category, largest magnitude first."""
        net: dict = {}
        for cat, b in self._memory_categories:
            net[cat] = net.get(cat, 0) + b
        return sorted(net.items(), key=lambda kv: -abs(kv[1]))

    def save_tensorboard_trace(self, logdir: str, run_id: str | None = None, hostname: str | None = None) -> str:
        """Write the Chrome trace where TensorBoard's profile plugin looks for it:
        ``<logdir>/plugins/profile/<run_id>/<hostname>.pt.trace.json``; returns that path."""
        import os
        import socket

        target = os.path.join(logdir, "plugins", "profile", run_id or "run0")
        os.makedirs(target, exist_ok=True)
        path = os.path.join(target, "%s.pt.trace.json" % (hostname or socket.gethostname() or "localhost"))
        with open(path, "w") as f:
            f.write(self._trace)
        return os.path.abspath(path)


class CudaKernelScope:
    """Times a region on the device with a pair of CUDA events on the current stream; ``stop()``
    queues the pair, the profiler's ``flush()`` turns it into an event after one synchronise
    (cuda_timing.rs:71-119).  On a machine without CUDA it falls back to the host clock."""

    def __init__(self, profiler: "Profiler", name: str, category: str = "kernel"):
        self.p, self.name, self.category = profiler, name, category
        self._cm = profiler.scope(name, category)
        self._cm.__enter__()
        self._open = True

    def stop(self) -> None:
        if self._open:
            self._cm.__exit__(None, None, None)
            self._open = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()


@contextlib.contextmanager
def profile_op_scope(name: str, category: str = "op", shapes=(), op: str | None = None):
    """Hook used by instrumented ops: a no-op unless a profiler is installed
    (ferrotorch-core/src/profiler_hook.rs:49-97)."""
    p = Profiler._current
    if p is None:
        yield
    else:
        with p.scope(name, category, shapes, op):
            yield


def with_profiler(fn, config: ProfileConfig | None = None, schedule: ProfileSchedule | None = None):
    """Run ``fn(profiler)`` with a profiler installed; returns ``(result, profiler)``."""
    p = Profiler(config, schedule)
    prev, Profiler._current = Profiler._current, p
    try:
        r = fn(p)
    finally:
        Profiler._current = prev
        p.flush()
    return r, p


class DeviceType(str, enum.Enum):
    """Where an event ran (event.rs:21)."""
    Cpu = "cpu"
    Cuda = "cuda"

    def __str__(self) -> str:
        return self.value


@dataclass
class GpuTimingPair:
    """Start and end of a device interval in microseconds (event.rs:116)."""
    start_us: int
    end_us: int

    def duration_us(self) -> int:
        return max(0, int(self.end_us) - int(self.start_us))
