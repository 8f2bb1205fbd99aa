"""The rest of the reference's ``ferrotorch-data`` surface under its names (ferrotorch-data/src/
lib.rs): small dataset combinators (dataset.rs:73-400), tensor transforms (transforms.rs),
collation (collate.rs), the iterator kinds of its loader (dataloader.rs:58-700) and the seed
function.  The loader itself is ``torch.utils.data.DataLoader``; the iterator classes here are
thin, explicit forms of its sync / prefetch / multi-worker modes for code written against them."""
from __future__ import annotations

import enum
import queue
import threading
from dataclasses import dataclass
from typing import Callable, Iterable, Sequence

import torch
from torch.utils.data import ChainDataset, ConcatDataset, DataLoader, Dataset, default_collate, get_worker_info  # noqa: F401


def manual_seed(seed: int) -> None:
    """Seed every generator the data pipeline draws from (torch CPU / CUDA, Python, numpy)."""
    import random

    import numpy as np

    torch.manual_seed(seed)
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))


@dataclass(frozen=True)
class WorkerInfo:
    worker_id: int
    num_workers: int

    @classmethod
    def current(cls) -> "WorkerInfo | None":
        """Inside a DataLoader worker: that worker's info; in the main process: None."""
        w = get_worker_info()
        return None if w is None else cls(w.id, w.num_workers)

    def shard(self, n: int) -> range:
        """The contiguous slice of ``range(n)`` this worker owns (remainder to the leading workers)."""
        base, extra = divmod(n, self.num_workers)
        lo = self.worker_id * base + min(self.worker_id, extra)
        return range(lo, lo + base + (1 if self.worker_id < extra else 0))


class WorkerMode(enum.Enum):
    IntraBatch = "intra_batch"     # workers split the samples of one batch
    CrossBatch = "cross_batch"     # workers build whole batches ahead (what torch's DataLoader does)


class VecDataset(Dataset):
    def __init__(self, samples: Sequence):
        self.samples = list(samples)

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, i: int):
        if not -len(self.samples) <= i < len(self.samples):
            raise IndexError("VecDataset: index %d out of range for %d samples" % (i, len(self.samples)))
        return self.samples[i]


class MappedDataset(Dataset):
    def __init__(self, dataset: Dataset, fn: Callable):
        self.dataset, self.fn = dataset, fn

    def __len__(self) -> int:
        return len(self.dataset)

    def __getitem__(self, i: int):
        return self.fn(self.dataset[i])


# --------------------------------------------------------------------------- transforms
class Transform:
    """``transform(sample) -> sample``."""

    def __call__(self, x):
        raise NotImplementedError


class Compose(Transform):
    def __init__(self, transforms: Iterable[Callable]):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class ToTensor(Transform):
    """Arrays / nested lists -> float tensor; uint8 image data ``[H, W, C]`` -> ``[C, H, W]`` in [0, 1]."""

    def __call__(self, x):
        t = torch.as_tensor(x)
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
            if t.dim() == 3:
                t = t.permute(2, 0, 1).contiguous()
        return t if t.is_floating_point() else t.float()


class Normalize(Transform):
    def __init__(self, mean, std):
        self.mean, self.std = torch.as_tensor(mean, dtype=torch.float32), torch.as_tensor(std, dtype=torch.float32)
        if bool((self.std == 0).any()):
            raise ValueError("Normalize: std must be non-zero")

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = (-1,) + (1,) * (x.dim() - 1 - (x.dim() == 4))
        m, s = self.mean.view(shape).to(x), self.std.view(shape).to(x)
        return (x - m) / s


class RandomHorizontalFlip(Transform):
    def __init__(self, p: float = 0.5, generator: torch.Generator | None = None):
        self.p, self.g = p, generator

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return x.flip(-1) if float(torch.rand((), generator=self.g)) < self.p else x


class RandomCrop(Transform):
    def __init__(self, size, padding: int = 0, generator: torch.Generator | None = None):
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.padding, self.g = padding, generator

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.padding:
            x = torch.nn.functional.pad(x, [self.padding] * 4)
        H, W = x.shape[-2:]
        th, tw = self.size
        if th > H or tw > W:
            raise ValueError("RandomCrop: crop %s larger than input %s" % (self.size, (H, W)))
        i = int(torch.randint(0, H - th + 1, (), generator=self.g))
        j = int(torch.randint(0, W - tw + 1, (), generator=self.g))
        return x[..., i:i + th, j:j + tw]


class ToDevice(Transform):
    """Move every tensor of a (nested) sample; ``pinned`` stages host tensors through pinned
    memory so that the copy can overlap compute."""

    def __init__(self, device, pinned: bool = False):
        self.device, self.pinned = torch.device(device), pinned

    def __call__(self, x):
        if isinstance(x, torch.Tensor):
            if self.pinned and self.device.type == "cuda" and not x.is_cuda:
                x = x.pin_memory()
            return x.to(self.device, non_blocking=self.pinned)
        if isinstance(x, (list, tuple)):
            return type(x)(self(v) for v in x)
        if isinstance(x, dict):
            return {k: self(v) for k, v in x.items()}
        return x


def default_collate_pair(samples):
    """``[(x, y), ...] -> (stack(x), stack(y))``."""
    xs, ys = zip(*samples)
    return default_collate(list(xs)), default_collate(list(ys))


# --------------------------------------------------------------------------- iterator kinds
class BatchIter:
    """Synchronous batches of sample lists over explicit indices."""

    def __init__(self, dataset: Dataset, indices: Sequence[int], batch_size: int, drop_last: bool = False):
        self.dataset, self.indices, self.bs, self.drop_last, self.pos = dataset, list(indices), batch_size, drop_last, 0

    def __len__(self) -> int:
        n = len(self.indices)
        return n // self.bs if self.drop_last else (n + self.bs - 1) // self.bs

    def __iter__(self):
        return self

    def __next__(self):
        idx = self.indices[self.pos:self.pos + self.bs]
        if not idx or (self.drop_last and len(idx) < self.bs):
            raise StopIteration
        self.pos += self.bs
        return [self.dataset[i] for i in idx]


class CollatedIter:
    def __init__(self, inner: Iterable, collate_fn: Callable = default_collate):
        self.inner, self.collate_fn = iter(inner), collate_fn

    def __iter__(self):
        return self

    def __next__(self):
        return self.collate_fn(next(self.inner))


class PrefetchIter:
    """Runs ``inner`` on a background thread, ``depth`` items ahead; an exception in the
    producer is re-raised at the consumer."""

    _END = object()

    def __init__(self, inner: Iterable, depth: int = 2):
        self.q: queue.Queue = queue.Queue(maxsize=max(1, depth))
        self._stop = threading.Event()

        def work():
            try:
                for item in inner:
                    while not self._stop.is_set():
                        try:
                            self.q.put(item, timeout=0.1)
                            break
                        except queue.Full:
                            continue
                    if self._stop.is_set():
                        return
                self.q.put(self._END)
            except BaseException as e:  # noqa: BLE001
                self.q.put(e)

        self.thread = threading.Thread(target=work, daemon=True)
        self.thread.start()

    def __iter__(self):
        return self

    def __next__(self):
        item = self.q.get()
        if item is self._END:
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        return item

    def close(self) -> None:
        self._stop.set()


def MultiWorkerIter(dataset: Dataset, batch_size: int, num_workers: int, shuffle: bool = False, collate_fn=None, **kw):
    """Whole batches built by ``num_workers`` processes, delivered in order: torch's loader iterator."""
    return iter(DataLoader(dataset, batch_size=batch_size, num_workers=num_workers, shuffle=shuffle, collate_fn=collate_fn, **kw))
