"""Datasets, loaders and samplers.

``torch.utils.data`` is re-exported (the reference's ``ferrotorch-data`` mirrors it: ``Dataset``,
``IterableDataset``, ``DataLoader`` with workers / prefetch / pin-memory / collate,
``Sequential`` / ``Random`` / ``Distributed`` / ``Weighted`` / ``Batch`` samplers,
ferrotorch-data/src/dataloader.rs:219-458, sampler.rs:74-182), plus the synthetic datasets of
the benchmark configs and a pinned-memory prefetcher that overlaps the host-to-device copy of
batch i+1 with the step on batch i.
"""
from __future__ import annotations

import torch
from torch.utils.data import (BatchSampler, DataLoader, Dataset, IterableDataset, RandomSampler, Sampler,  # noqa: F401
                              SequentialSampler, Subset, TensorDataset, WeightedRandomSampler, random_split)
from torch.utils.data.distributed import DistributedSampler  # noqa: F401


class SyntheticTokens(Dataset):
    """Uniform-random token ids ``[seq_len + 1]`` per item (inputs = ``[:-1]``, labels = ``[1:]``),
    deterministic per (seed, index)."""

    def __init__(self, vocab_size: int, seq_len: int, length: int, seed: int = 0):
        self.vocab_size, self.seq_len, self.length, self.seed = vocab_size, seq_len, length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        t = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g)
        return t[:-1], t[1:]


class SyntheticImages(Dataset):
    """N(0,1) images ``[3, H, W]`` with uniform labels (the ResNet-50 benchmark data)."""

    def __init__(self, length: int, num_classes: int = 1000, size: int = 224, seed: int = 0):
        self.length, self.num_classes, self.size, self.seed = length, num_classes, size, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        return torch.randn(3, self.size, self.size, generator=g), int(torch.randint(0, self.num_classes, (1,), generator=g))


def shuffle_with_seed(n: int, seed: int) -> list[int]:
    """Deterministic permutation of ``range(n)`` (sampler.rs:74)."""
    return torch.randperm(n, generator=torch.Generator().manual_seed(seed)).tolist()


class DevicePrefetcher:
    """Iterate a loader of (possibly nested) CPU tensors; batch i+1 is copied from pinned memory
    on a side stream while the caller works on batch i."""

    def __init__(self, loader, device):
        self.loader, self.device = loader, torch.device(device)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def _move(self, obj):
        if isinstance(obj, torch.Tensor):
            if self.stream is not None and not obj.is_pinned():
                obj = obj.pin_memory()
            return obj.to(self.device, non_blocking=True)
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._move(o) for o in obj)
        if isinstance(obj, dict):
            return {k: self._move(v) for k, v in obj.items()}
        return obj

    def __iter__(self):
        it = iter(self.loader)
        nxt = None

        def fetch():
            try:
                b = next(it)
            except StopIteration:
                return None
            if self.stream is None:
                return self._move(b)
            with torch.cuda.stream(self.stream):
                return self._move(b)

        nxt = fetch()
        while nxt is not None:
            if self.stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.stream)
            cur, nxt = nxt, fetch()
            yield cur

    def __len__(self):
        return len(self.loader)

from .token_loader import TokenFileLoader, write_token_file  # noqa: F401,E402

from .interop import (dataframe_to_tensor, record_batch_to_tensor, tensor_from_arrow_array,  # noqa: F401,E402
                      tensor_to_arrow_array, tensor_to_arrow_arrayref)


from .compat import (BatchIter, ChainDataset, CollatedIter, Compose, ConcatDataset, MappedDataset, MultiWorkerIter,  # noqa: F401,E402
                     Normalize, PrefetchIter, RandomCrop, RandomHorizontalFlip, ToDevice, ToTensor, Transform, VecDataset,
                     WorkerInfo, WorkerMode, default_collate, default_collate_pair, manual_seed)
