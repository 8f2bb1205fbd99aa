"""Host-side failure detection between steps: a key-value store, a heartbeat per rank, and a
guard that training loops call before every launch.

The reference has receive time-outs and typed errors but no heartbeat, no membership and no
re-rendezvous (ferrotorch-distributed/src/error.rs:21-66, collective.rs:35; the rest is a design
note, .design/phase-7-distributed.md:392-431); a changed world size is handled offline by
resharding a distributed checkpoint (checkpoint.rs:478-573).  Here the ranks of a job learn on the
host that a peer is gone *before* they launch the next step's kernels -- so no device-side wait
ever has to run into its limit for that reason -- and the survivors can reload the last sharded
checkpoint at the smaller world size (``dist_checkpoint.load_distributed`` reshards).

A rank leaves only between steps (``Heartbeat.leave``) or disappears (its counter stops); the
device-side bounded waits of the kernels remain the second line of defence.
"""
from __future__ import annotations

import os
import threading
import time


class RankFailure(RuntimeError):
    """One or more ranks stopped beating (``.ranks``) or announced that they left (``.left``)."""

    def __init__(self, ranks, left=()):
        self.ranks, self.left = sorted(ranks), sorted(left)
        super().__init__("ranks %s stopped responding, ranks %s left" % (self.ranks, self.left))


class FileStore:
    """Key-value store on a directory every rank can reach (atomic writes by rename)."""

    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)

    def _path(self, key: str) -> str:
        return os.path.join(self.dir, key.replace("/", "__"))

    def set(self, key: str, value: bytes | str) -> None:
        data = value.encode() if isinstance(value, str) else value
        tmp = self._path(key) + ".tmp%d" % os.getpid()
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, self._path(key))

    def get(self, key: str) -> bytes | None:
        try:
            with open(self._path(key), "rb") as f:
                return f.read()
        except FileNotFoundError:
            return None


class TorchStore:
    """Adapter over a ``torch.distributed`` store (``TCPStore`` / ``FileStore``): ``get`` returns
    None for a missing key instead of blocking."""

    def __init__(self, store):
        self.store = store

    def set(self, key: str, value: bytes | str) -> None:
        self.store.set(key, value)

    def get(self, key: str) -> bytes | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key)
        except Exception:  # noqa: BLE001
            return None


class Heartbeat:
    """Every rank bumps ``hb/<rank>`` every ``interval`` seconds on a helper thread; a peer whose
    counter has not changed for ``timeout`` seconds (measured on the observer's own clock, so
    clock skew between hosts does not matter) counts as failed."""

    def __init__(self, store, rank: int, world_size: int, interval: float = 0.2, timeout: float = 2.0,
                 prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._count = 0
        self._seen: dict[int, tuple[bytes | None, float]] = {}
        self._stop = threading.Event()
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        now = time.monotonic()
        for r in range(world_size):
            self._seen[r] = (None, now)

    def _beat(self) -> None:
        self._count += 1
        self.store.set("%s/%d" % (self.prefix, self.rank), str(self._count))

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:  # noqa: BLE001   (the store going away is detected by the peers)
                pass

    # ------------------------------------------------------------------ observation
    def left_ranks(self) -> list[int]:
        return [r for r in range(self.world) if self.store.get("%s/left/%d" % (self.prefix, r)) is not None]

    def dead_ranks(self) -> list[int]:
        """Ranks (other than this one and those that left cleanly) whose counter is stale."""
        now = time.monotonic()
        left = set(self.left_ranks())
        dead = []
        for r in range(self.world):
            if r == self.rank or r in left:
                continue
            val = self.store.get("%s/%d" % (self.prefix, r))
            last_val, last_t = self._seen[r]
            if val is not None and val != last_val:
                self._seen[r] = (val, now)
            elif now - last_t > self.timeout:
                dead.append(r)
        return dead

    def check(self) -> None:
        """Call between steps, before the next launch: raises :class:`RankFailure` when a peer is
        gone or has left."""
        dead, left = self.dead_ranks(), [r for r in self.left_ranks() if r != self.rank]
        if dead or left:
            raise RankFailure(dead, left)

    def wait_for_all(self, limit: float = 30.0) -> None:
        """Block until every rank has beaten at least once (start-up rendezvous)."""
        t0 = time.monotonic()
        while True:
            missing = [r for r in range(self.world) if self.store.get("%s/%d" % (self.prefix, r)) is None]
            if not missing:
                now = time.monotonic()
                for r in range(self.world):
                    self._seen[r] = (self._seen[r][0], now)
                return
            if time.monotonic() - t0 > limit:
                raise RankFailure(missing)
            time.sleep(self.interval / 2)

    # ------------------------------------------------------------------ leaving
    def leave(self) -> None:
        """Announce a clean departure (between steps, nothing of this rank in flight)."""
        self.store.set("%s/left/%d" % (self.prefix, self.rank), "1")
        self.stop()

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2 * self.interval + 1.0)


def survivors(world_size: int, failure: RankFailure) -> list[int]:
    """Ranks that go on after ``failure``, in order: their index in this list is the new rank."""
    gone = set(failure.ranks) | set(failure.left)
    return [r for r in range(world_size) if r not in gone]


def barrier(store, name: str, rank: int, ranks, limit: float = 30.0, poll: float = 0.02) -> None:
    """Store-based barrier among ``ranks`` (used by survivors to regroup); raises
    :class:`RankFailure` with the ranks that did not arrive within ``limit`` seconds."""
    store.set("bar/%s/%d" % (name, rank), "1")
    t0 = time.monotonic()
    while True:
        missing = [r for r in ranks if store.get("bar/%s/%d" % (name, r)) is None]
        if not missing:
            return
        if time.monotonic() - t0 > limit:
            raise RankFailure(missing)
        time.sleep(poll)
