"""Counter-based Philox-4x32-10 generator on the host with the reference's stream layout
(ferrotorch-gpu/src/rng.rs:94-300: ``PhiloxState``, ``PhiloxGenerator``; :399-540: the per-device
manager).

One 64-bit counter value yields four 32-bit words (counter in the low two counter words, the other
two zero, the seed as the key); ``next_u32`` walks the words of one counter before moving to the
next, ``next_f32`` keeps the top 24 bits.  Device-side random numbers of this framework come from
torch's CUDA generator (itself Philox-4x32-10, addressed by seed and offset); this host generator
is for reproducible streams that do not depend on a device -- data order, dropout masks in CPU
oracles.  The word stream is filled by the C++ host library (``csrc/host/philox.cpp``), with a
vectorised numpy form of the same rounds as the fallback and as the test oracle.
"""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass

import numpy as np

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox_4x32_10(counter, key, counter_hi=0) -> np.ndarray:
    """Four output words per counter: ``counter`` (scalar or array, 64-bit, the low two counter
    words; ``counter_hi`` the high two) under the 64-bit ``key``.  Returns uint32 ``[..., 4]``."""
    c = np.asarray(counter, dtype=np.uint64)
    ch = np.broadcast_to(np.asarray(counter_hi, dtype=np.uint64), c.shape)
    c0, c1, c2, c3 = c & _MASK, c >> np.uint64(32), ch & _MASK, ch >> np.uint64(32)
    k0, k1 = int(key) & 0xFFFFFFFF, (int(key) >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = np.uint64(M0) * c0, np.uint64(M1) * c2           # 32 x 32 -> 64 bits: no overflow in uint64
        c0, c1, c2, c3 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0), p1 & _MASK,
                          (p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1), p0 & _MASK)
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


_fill = False          # False = not looked up yet, None = unavailable


def _native_fill():
    global _fill
    if _fill is False:
        try:
            import ctypes

            from .. import _native

            lib = _native.host()
            lib.ftp_fill_words.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p]
            lib.ftp_fill_words.restype = ctypes.c_int
            _fill = lib.ftp_fill_words
        except Exception:  # noqa: BLE001 - no compiler / library: the numpy path serves
            _fill = None
    return _fill


@dataclass(frozen=True)
class PhiloxState:
    counter: int
    seed: int
    offset: int = 0

    def __post_init__(self):
        if not 0 <= self.offset < 4:
            raise ValueError("invalid Philox offset %d; must be < 4" % self.offset)

    @classmethod
    def from_parts(cls, counter: int, seed: int, offset: int) -> "PhiloxState":
        return cls(counter, seed, offset)


class PhiloxGenerator:
    def __init__(self, seed: int = 0):
        self.set_seed(seed)

    def set_seed(self, seed: int) -> None:
        self.seed, self.counter, self.offset = int(seed) & (2 ** 64 - 1), 0, 0

    def get_state(self) -> PhiloxState:
        return PhiloxState(self.counter, self.seed, self.offset)

    def set_state(self, state: PhiloxState) -> None:
        self.seed, self.counter, self.offset = state.seed, state.counter, state.offset

    def advance(self, n_counters: int) -> None:
        """Skip ``n_counters`` counter values (four words each); a partly used counter is dropped."""
        self.counter, self.offset = (self.counter + int(n_counters)) & (2 ** 64 - 1), 0

    def words(self, n: int) -> np.ndarray:
        """The next ``n`` 32-bit words of the stream (the C++ host library fills them when it is
        built; the numpy form of the same rounds otherwise)."""
        if n <= 0:
            return np.empty(0, np.uint32)
        fill = _native_fill()
        if fill is not None:
            out = np.empty(n, np.uint32)
            if fill(self.counter, self.seed, self.offset, n, out.ctypes.data) != 0:
                raise RuntimeError("ftp_fill_words failed")
        else:
            blocks = (self.offset + n + 3) // 4
            ctr = (np.arange(blocks, dtype=np.uint64) + np.uint64(self.counter))
            out = philox_4x32_10(ctr, self.seed).reshape(-1)[self.offset:self.offset + n]
        end = self.offset + n
        self.counter, self.offset = (self.counter + end // 4) & (2 ** 64 - 1), end % 4
        return out

    def next_u32(self) -> int:
        return int(self.words(1)[0])

    def next_f32(self) -> float:
        return float(np.float32(self.next_u32() >> 8) * np.float32(1.0 / 16777216.0))

    def generate_uniform(self, n: int) -> np.ndarray:
        """``n`` float32 values in [0, 1) on a 2^-24 grid."""
        return (self.words(n) >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)

    def generate_normal(self, n: int) -> np.ndarray:
        """Box-Muller over consecutive pairs (u1, u2): ``sqrt(-2 ln u1) * (cos, sin)(2 pi u2)``;
        a zero u1 is re-drawn, as the reference does."""
        pairs = (n + 1) // 2
        saved = self.get_state()
        u = self.generate_uniform(2 * pairs).reshape(pairs, 2)
        if (u[:, 0] == 0).any():                                  # one in 2^24 per pair: redo element-wise
            self.set_state(saved)
            u = np.empty((pairs, 2), np.float32)
            for i in range(pairs):
                u1 = self.next_f32()
                while u1 == 0.0:
                    u1 = self.next_f32()
                u[i] = (u1, self.next_f32())
        r = np.sqrt(np.float32(-2.0) * np.log(u[:, 0]))
        theta = np.float32(2.0 * math.pi) * u[:, 1]
        return np.stack([r * np.cos(theta), r * np.sin(theta)], axis=1).reshape(-1)[:n].astype(np.float32)

    def __repr__(self) -> str:
        return "PhiloxGenerator(counter=%d, seed=%d, offset=%d)" % (self.counter, self.seed, self.offset)


class CudaRngManager:
    """One generator per device ordinal, created on first use with the default seed."""

    DEFAULT_SEED = 0

    def __init__(self):
        self.generators: dict = {}
        self._default = self.DEFAULT_SEED

    def generator(self, device: int) -> PhiloxGenerator:
        if device not in self.generators:
            self.generators[device] = PhiloxGenerator(self._default)
        return self.generators[device]

    def manual_seed(self, device: int, seed: int) -> None:
        self.generator(device).set_seed(seed)

    def manual_seed_all(self, seed: int) -> None:
        self._default = seed                                     # devices met later start from it too
        for g in self.generators.values():
            g.set_seed(seed)

    def get_rng_state(self, device: int) -> PhiloxState:
        return self.generator(device).get_state()

    def set_rng_state(self, device: int, state: PhiloxState) -> None:
        self.generator(device).set_state(state)


_manager = CudaRngManager()
_manager_lock = threading.Lock()


def cuda_rng_manager() -> CudaRngManager:
    return _manager


def fork_rng(devices) -> list:
    """Snapshot the generators of ``devices`` (restore with :func:`join_rng`)."""
    with _manager_lock:
        return [_manager.get_rng_state(d) for d in devices]


def join_rng(devices, states) -> None:
    if len(devices) != len(states):
        raise ValueError("join_rng: %d devices but %d states" % (len(devices), len(states)))
    with _manager_lock:
        for d, s in zip(devices, states):
            _manager.set_rng_state(d, s)
