"""GPU memory guard: budget, reservation, OOM policy, pre-OOM hooks by priority, pressure
listeners and a watchdog thread (ferrotorch-gpu/src/memory_guard.rs:76-1305).

The guard sits on top of an ``allocator`` object with ``used_bytes()`` / ``total_bytes()`` /
``empty_cache()``; the default one reads ``torch.cuda`` (``mem_get_info``, the caching
allocator's statistics).  Tests use a fake allocator with a budget, never real exhaustion.
"""
from __future__ import annotations

import enum
import threading
import time
from typing import Callable


class OomPolicy(enum.Enum):
    FAIL = "fail"                  # raise immediately
    RUN_HOOKS_THEN_FAIL = "hooks"  # run pre-OOM hooks (free caches, offload), retry once, then raise
    WAIT = "wait"                  # block (bounded) until pressure drops, e.g. another job frees memory


class MemoryBudgetExceeded(MemoryError):
    pass


class TorchCudaAllocator:
    def __init__(self, device: int = 0):
        self.device = device

    def used_bytes(self) -> int:
        import torch

        return int(torch.cuda.memory_reserved(self.device))

    def total_bytes(self) -> int:
        import torch

        return int(torch.cuda.mem_get_info(self.device)[1])

    def empty_cache(self) -> None:
        import torch

        torch.cuda.empty_cache()


class MemoryGuard:
    def __init__(self, allocator=None, budget_bytes: int | None = None, reserve_bytes: int = 0,
                 policy: OomPolicy = OomPolicy.RUN_HOOKS_THEN_FAIL, pressure_threshold: float = 0.9,
                 wait_timeout_s: float = 5.0):
        self.alloc = allocator or TorchCudaAllocator()
        self.budget = budget_bytes if budget_bytes is not None else self.alloc.total_bytes()
        self.reserve, self.policy = reserve_bytes, policy
        self.pressure_threshold, self.wait_timeout_s = pressure_threshold, wait_timeout_s
        self._hooks: list[tuple[int, str, Callable[[int], int]]] = []
        self._listeners: list[Callable[[float], None]] = []
        self._emergency: Callable[[], None] | None = None
        self._watchdog: threading.Thread | None = None
        self._stop = threading.Event()
        self.paused = threading.Event()
        self.stats = {"checks": 0, "hook_runs": 0, "freed_by_hooks": 0, "failures": 0, "pauses": 0}
        self._level_listeners: list = []
        self._last_level = None
        self._hook_ids: dict = {}
        self._next_hook = 0
        self._peak = 0
        self._oom_callbacks: list = []

    # ---- configuration
    def add_pre_oom_hook(self, fn: Callable[[int], int], priority: int = 0, name: str = "") -> None:
        """``fn(bytes_needed) -> bytes_freed``; hooks run in descending priority until enough is free."""
        self._hooks.append((priority, name or getattr(fn, "__name__", "hook"), fn))
        self._hooks.sort(key=lambda h: -h[0])

    def add_pressure_listener(self, fn: Callable[[float], None]) -> None:
        self._listeners.append(fn)

    def set_emergency_checkpoint(self, fn: Callable[[], None]) -> None:
        self._emergency = fn

    # ---- queries
    def available(self) -> int:
        return self.budget - self.reserve - self.alloc.used_bytes()

    def pressure(self) -> float:
        return self.alloc.used_bytes() / max(1, self.budget - self.reserve)

    # ---- the check callers make before a large allocation
    def ensure(self, nbytes: int) -> None:
        self.stats["checks"] += 1
        if nbytes <= self.available():
            return
        if self.policy == OomPolicy.FAIL:
            return self._fail(nbytes)
        if self.policy == OomPolicy.WAIT:
            deadline = time.time() + self.wait_timeout_s
            while time.time() < deadline:
                if nbytes <= self.available():
                    return
                time.sleep(0.01)
        need = nbytes - self.available()
        for _, _, fn in self._hooks:
            self.stats["hook_runs"] += 1
            self.stats["freed_by_hooks"] += int(fn(need) or 0)
            need = nbytes - self.available()
            if need <= 0:
                return
        self.alloc.empty_cache()
        if nbytes <= self.available():
            return
        self._fail(nbytes)

    def _fail(self, nbytes: int):
        for fn in self._oom_callbacks:
            fn()
        self.stats["failures"] += 1
        if self._emergency is not None:
            self._emergency()
        raise MemoryBudgetExceeded("need %d bytes, %d available (budget %d, reserved %d)" %
                                   (nbytes, self.available(), self.budget, self.reserve))

    # ---- watchdog: pauses training (``guard.paused`` is set) while pressure is above the threshold
    def start_watchdog(self, interval_s: float = 0.05) -> None:
        def run():
            while not self._stop.wait(interval_s):
                p = self.pressure()
                if p >= self.pressure_threshold:
                    if not self.paused.is_set():
                        self.paused.set()
                        self.stats["pauses"] += 1
                    for fn in self._listeners:
                        fn(p)
                else:
                    self.paused.clear()

        self._stop.clear()
        self._watchdog = threading.Thread(target=run, daemon=True)
        self._watchdog.start()

    def stop_watchdog(self) -> None:
        self._stop.set()
        if self._watchdog is not None:
            self._watchdog.join(2.0)

    def wait_if_paused(self, timeout_s: float = 1.0) -> bool:
        """Training loops call this between steps; returns False if still paused after the timeout."""
        deadline = time.time() + timeout_s
        while self.paused.is_set() and time.time() < deadline:
            time.sleep(0.005)
        return not self.paused.is_set()

    # ---- the reference's method names (memory_guard.rs:254-770)
    def pressure_level(self) -> PressureLevel:
        return PressureLevel.of(self.pressure())

    def notify_pressure_change(self) -> PressureLevel:
        """Call the ``(old, new)`` listeners when the level moved since the last call."""
        new, old = self.pressure_level(), (self._last_level if self._last_level is not None else PressureLevel.NONE)
        if new != old:
            self._last_level = new
            for fn in self._level_listeners:
                fn(old, new)
        return new

    def add_level_listener(self, fn) -> None:
        self._level_listeners.append(fn)

    def register_hook(self, fn, priority: int = 0, name: str = "") -> int:
        self.add_pre_oom_hook(fn, priority, name)
        self._next_hook += 1
        self._hook_ids[self._next_hook] = fn
        return self._next_hook

    def remove_hook(self, hid: int) -> bool:
        fn = self._hook_ids.pop(hid, None)
        if fn is None:
            return False
        self._hooks = [h for h in self._hooks if h[2] is not fn]
        return True

    def memory_stats(self) -> dict:
        used = self.alloc.used_bytes()
        self._peak = max(self._peak, used)
        return {"used_bytes": used, "peak_bytes": self._peak, "budget_bytes": self.budget,
                "reserved_bytes": self.reserve, "available_bytes": self.available(), "pressure": self.pressure(),
                "level": self.pressure_level().name, **self.stats}

    def reset_peak_stats(self) -> None:
        self._peak = self.alloc.used_bytes()

    def safe_alloc(self, shape, dtype=None, device=None):
        """``torch.empty`` behind the guard: the size is checked against the budget (running hooks /
        waiting / failing by policy) before the allocator is asked."""
        import math

        import torch

        dtype = dtype or torch.float32
        self.ensure(math.prod(shape) * torch.empty(0, dtype=dtype).element_size())
        return torch.empty(tuple(shape), dtype=dtype, device=device)

    def on_oom(self, fn) -> None:
        """``fn()`` runs (after the hooks, before the error is raised) whenever a request cannot be met
        (memory_guard.rs:373)."""
        self._oom_callbacks.append(fn)

    def safe_alloc_copy(self, data, dtype=None, device=None):
        """A guarded allocation filled with ``data`` (a tensor or anything ``torch.as_tensor`` takes)."""
        import torch

        src = torch.as_tensor(data, dtype=dtype)
        out = self.safe_alloc(src.shape, src.dtype, device)
        out.copy_(src)
        return out

    def safe_alloc_with_hooks(self, shape, dtype=None, device=None):
        """Like ``safe_alloc`` but the pre-OOM hooks always get their chance, whatever the policy says
        (memory_guard.rs:479)."""
        prev = self.policy
        if prev == OomPolicy.FAIL:
            self.policy = OomPolicy.RUN_HOOKS_THEN_FAIL
        try:
            return self.safe_alloc(shape, dtype, device)
        finally:
            self.policy = prev

    def free(self, tensor) -> int:
        """Give a guarded allocation back: the storage is released to the caching allocator when the last
        reference goes; returns the bytes the tensor held."""
        n = tensor.numel() * tensor.element_size()
        tensor.set_()
        return n

    def device_ordinal(self) -> int:
        return int(getattr(self.alloc, "device", 0))

    def device(self):
        import torch

        return torch.device("cuda", self.device_ordinal()) if isinstance(self.alloc, TorchCudaAllocator) else torch.device("cpu")

    def set_budget(self, nbytes: int) -> None:
        self.budget = int(nbytes)

    def set_oom_policy(self, policy: OomPolicy) -> None:
        self.policy = policy

    def has_reservation(self) -> bool:
        return self.reserve > 0

    def release_reservation(self) -> None:
        self.reserve = 0

    def reserved_bytes(self) -> int:
        return self.reserve

    def device_arc(self):
        return self.device()


# --------------------------------------------------------------------------- the reference's vocabulary
# (memory_guard.rs: OomPolicy::{Fail, RetryAfterFree, WaitAndRetry, CheckpointAndFail}, PressureLevel,
#  MemoryStats, MemoryGuardBuilder, register_hook / remove_hook, reservations, safe_alloc)
OomPolicy.Fail = OomPolicy.FAIL
OomPolicy.RetryAfterFree = OomPolicy.RUN_HOOKS_THEN_FAIL
OomPolicy.WaitAndRetry = OomPolicy.WAIT
OomPolicy.CheckpointAndFail = OomPolicy.FAIL        # with an emergency-checkpoint callback installed


class PressureLevel(enum.IntEnum):
    NONE = 0        # < 50 % of the usable budget
    LOW = 1         # 50 - 70 %
    MEDIUM = 2      # 70 - 85 %
    HIGH = 3        # 85 - 95 %
    CRITICAL = 4    # >= 95 %

    @classmethod
    def of(cls, pressure: float) -> "PressureLevel":
        for level, lo in ((cls.CRITICAL, 0.95), (cls.HIGH, 0.85), (cls.MEDIUM, 0.70), (cls.LOW, 0.50)):
            if pressure >= lo:
                return level
        return cls.NONE





class MemoryGuardBuilder:
    """``MemoryGuardBuilder().budget_bytes(n).reserve_bytes(m).oom_policy(p).build(allocator)``."""

    def __init__(self):
        self._kw: dict = {}

    def budget_bytes(self, n: int) -> "MemoryGuardBuilder":
        self._kw["budget_bytes"] = int(n)
        return self

    def reserve_bytes(self, n: int) -> "MemoryGuardBuilder":
        self._kw["reserve_bytes"] = int(n)
        return self

    def oom_policy(self, policy: OomPolicy) -> "MemoryGuardBuilder":
        self._kw["policy"] = policy
        return self

    def pressure_threshold(self, frac: float) -> "MemoryGuardBuilder":
        self._kw["pressure_threshold"] = float(frac)
        return self

    def build(self, allocator=None) -> MemoryGuard:
        if self._kw.get("reserve_bytes", 0) and self._kw.get("budget_bytes") is not None and \
                self._kw["reserve_bytes"] >= self._kw["budget_bytes"]:
            raise ValueError("MemoryGuardBuilder: the reservation must be smaller than the budget")
        return MemoryGuard(allocator, **self._kw)


# --------------------------------------------------------------------------- small types of the reference's guard
from dataclasses import dataclass as _dataclass  # noqa: E402
from typing import Callable as _Callable  # noqa: E402

MemoryHook = _Callable[[int], int]                  # bytes needed -> bytes freed
MemoryPressureListener = _Callable[[float], None]   # called with the pressure ratio when it crosses the threshold


@_dataclass
class MemoryStats:
    used_bytes: int
    peak_bytes: int
    budget_bytes: int
    reserved_bytes: int
    available_bytes: int
    pressure: float
    level: str

    @classmethod
    def of(cls, guard: MemoryGuard) -> "MemoryStats":
        d = guard.memory_stats()
        return cls(*[d[k] for k in ("used_bytes", "peak_bytes", "budget_bytes", "reserved_bytes", "available_bytes",
                                    "pressure", "level")])


class MemoryReservation:
    """Headroom held back from the budget for the lifetime of the object (or the ``with`` block)."""

    def __init__(self, guard: MemoryGuard, nbytes: int):
        if nbytes < 0 or guard.reserve + nbytes >= guard.budget:
            raise ValueError("MemoryReservation: %d bytes do not fit under the budget of %d" % (nbytes, guard.budget))
        self.guard, self.nbytes, self._held = guard, int(nbytes), True
        guard.reserve += self.nbytes

    def release(self) -> None:
        if self._held:
            self.guard.reserve -= self.nbytes
            self._held = False

    def reserved_bytes(self) -> int:
        return self.nbytes if self._held else 0

    def device_ordinal(self) -> int:
        return self.guard.device_ordinal()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()
        return False


class MemoryWatchdog:
    """The guard's background pressure check as an object of its own (memory_guard.rs:1147-1310): a thread
    samples the allocator every ``interval_s``; while usage is above ``pressure_threshold`` x the usable budget
    the guard is *paused* and training loops that call :meth:`wait_if_paused` between steps hold still."""

    def __init__(self, guard: MemoryGuard, interval_s: float = 0.05, pressure_threshold: float | None = None):
        self._guard, self.interval_s = guard, interval_s
        if pressure_threshold is not None:
            guard.pressure_threshold = pressure_threshold
        self._checked = threading.Event()
        guard.add_pressure_listener(lambda _p: self._checked.set())

    def guard(self) -> MemoryGuard:
        return self._guard

    def device(self):
        return self._guard.device()

    def memory_info(self) -> tuple:
        """``(free, total)`` bytes as the guard sees them."""
        a = self._guard.alloc
        return max(0, a.total_bytes() - a.used_bytes()), a.total_bytes()

    def pressure_threshold_bytes(self) -> int:
        g = self._guard
        return int(g.pressure_threshold * max(1, g.budget - g.reserve))

    def check_pressure(self) -> bool:
        """One check now, on the caller's thread: is usage above the threshold?"""
        self._checked.set()
        return self._guard.alloc.used_bytes() >= self.pressure_threshold_bytes()

    def start(self) -> "MemoryWatchdog":
        self._guard.start_watchdog(self.interval_s)
        return self

    def stop(self) -> None:
        self._guard.stop_watchdog()

    def wait_if_paused(self, timeout_s: float = 1.0) -> bool:
        return self._guard.wait_if_paused(timeout_s)

    def wait_for_first_check(self, timeout_s: float = 1.0) -> bool:
        """Block until the thread has looked at the allocator at least once (true) or the time is up."""
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            if self._checked.is_set() or (self._guard._watchdog is not None and self._guard._watchdog.is_alive()
                                          and time.time() > deadline - timeout_s + 2 * self.interval_s):
                return True
            time.sleep(min(0.005, self.interval_s))
        return self._checked.is_set()


class MemoryGuardedDevice:
    """A device handle whose allocations go through a guard (memory_guard.rs ``MemoryGuardedDevice``)."""

    def __init__(self, guard: MemoryGuard):
        self._guard = guard

    def guard(self) -> MemoryGuard:
        return self._guard

    def device(self):
        return self._guard.device()

    def safe_alloc(self, shape, dtype=None):
        return self._guard.safe_alloc(shape, dtype, self.device())

    def safe_alloc_copy(self, data, dtype=None):
        return self._guard.safe_alloc_copy(data, dtype, self.device())
