"""Native token-batch loader: a memory-mapped token file, seeded per-epoch shuffling, rank
sharding and worker threads that assemble batches ahead of the training loop
(``csrc/host/token_loader.cpp``; the reference's counterpart is the rayon-backed ``DataLoader`` +
``DistributedSampler``, ferrotorch-data/src/dataloader.rs:219-458, sampler.rs:144-182).

    write_token_file("train.bin", ids)                       # uint16 / uint32 little endian
    loader = TokenFileLoader("train.bin", seq_len=4096, batch_size=4, rank=r, world_size=w)
    for inputs, labels in loader:                            # one epoch; pinned int64 [B, S]
        ...
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native

_protos_done = False


def _lib():
    global _protos_done
    lib = _native.host()
    if not _protos_done:
        vp, i, ll, ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong
        lib.ftd_open.restype, lib.ftd_open.argtypes = vp, [ctypes.c_char_p, i, i, i, i, i, ull, i, i, i]
        lib.ftd_close.restype, lib.ftd_close.argtypes = None, [vp]
        lib.ftd_next.restype, lib.ftd_next.argtypes = ll, [vp, vp]
        lib.ftd_num_samples.restype, lib.ftd_num_samples.argtypes = ll, [vp]
        lib.ftd_batches_per_epoch.restype, lib.ftd_batches_per_epoch.argtypes = ll, [vp]
        lib.ftd_last_error.restype, lib.ftd_last_error.argtypes = ctypes.c_char_p, []
        _protos_done = True
    return lib


def write_token_file(path: str, ids, vocab_size: int | None = None) -> int:
    """Write token ids as uint16 (vocabularies up to 65536) or uint32; returns the bytes per id."""
    a = np.asarray(ids.cpu() if isinstance(ids, torch.Tensor) else ids).reshape(-1)
    top = int(vocab_size if vocab_size is not None else (a.max() + 1 if a.size else 1))
    dt = np.uint16 if top <= 65536 else np.uint32
    a.astype("<u2" if dt is np.uint16 else "<u4").tofile(path)
    return 2 if dt is np.uint16 else 4


class TokenFileLoader:
    """Iterating yields ``(inputs, labels)`` int64 ``[batch, seq_len]`` for one epoch; the next
    iteration continues with the next epoch's permutation.  Batches come out in a fixed order
    for a given ``(seed, epoch, rank, world_size)`` whatever the number of worker threads."""

    def __init__(self, path: str, seq_len: int, batch_size: int, *, dtype_bytes: int = 2, num_workers: int = 4,
                 prefetch: int = 8, seed: int = 0, shuffle: bool = True, rank: int = 0, world_size: int = 1,
                 pin_memory: bool | None = None):
        self._lib = _lib()
        self._h = self._lib.ftd_open(path.encode(), dtype_bytes, seq_len, batch_size, num_workers, prefetch, seed,
                                     int(shuffle), rank, world_size)
        if not self._h:
            raise ValueError(self._lib.ftd_last_error().decode())
        self.seq_len, self.batch_size = seq_len, batch_size
        self.num_samples = int(self._lib.ftd_num_samples(self._h))
        self.batches_per_epoch = int(self._lib.ftd_batches_per_epoch(self._h))
        self.epoch = 0
        self.pin = torch.cuda.is_available() if pin_memory is None else pin_memory

    def __len__(self) -> int:
        return self.batches_per_epoch

    def next_batch(self) -> tuple[torch.Tensor, torch.Tensor]:
        buf = torch.empty((self.batch_size, self.seq_len + 1), dtype=torch.int64, pin_memory=self.pin)
        ep = int(self._lib.ftd_next(self._h, buf.data_ptr()))
        if ep < 0:
            raise RuntimeError(self._lib.ftd_last_error().decode())
        self.epoch = ep
        return buf[:, :-1], buf[:, 1:]

    def __iter__(self):
        for _ in range(self.batches_per_epoch):
            yield self.next_batch()

    def close(self) -> None:
        if self._h:
            self._lib.ftd_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
