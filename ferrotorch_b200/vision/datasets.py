"""Dataset readers written out: MNIST (IDX files), CIFAR-10 / CIFAR-100 (binary batches) and an
image-folder dataset, each with a synthetic variant for tests and examples.

The reference reads the same on-disk formats (ferrotorch-vision/src/datasets/mnist.rs
``Mnist::from_dir`` / ``synthetic``; cifar.rs ``Cifar10::from_dir`` with ``data_batch_{1..5}.bin`` /
``test_batch.bin``, ``Cifar100::from_dir`` with ``train.bin`` / ``test.bin`` and the fine label in the
second header byte; folder.rs ``ImageFolder``).  A sample is ``(image float32 [C, H, W] in [0, 1],
label int)``; ``transform`` is applied to the image, ``target_transform`` to the label.  The whole
split is decoded once into one uint8 tensor; ``__getitem__`` converts a single image.
"""
from __future__ import annotations

import gzip
import os
import struct
from typing import Callable

import numpy as np
import torch
from torch.utils.data import Dataset


class DatasetFormatError(ValueError):
    """A dataset file does not have the layout its format prescribes."""


def _split_name(split) -> str:
    name = getattr(split, "value", split)
    if isinstance(name, bool):
        name = "train" if name else "test"
    if name not in ("train", "test"):
        raise ValueError("split must be 'train' or 'test', got %r" % (split,))
    return name


def _read_maybe_gz(path: str) -> bytes:
    if os.path.exists(path):
        with open(path, "rb") as f:
            return f.read()
    if os.path.exists(path + ".gz"):
        with gzip.open(path + ".gz", "rb") as f:
            return f.read()
    raise FileNotFoundError(path)


class _ArrayDataset(Dataset):
    """``images uint8 [N, C, H, W]`` + ``labels int64 [N]`` behind the Dataset protocol."""

    num_classes = 0
    split = "train"                 # which part of the dataset an instance holds ("train" / "test")

    def __init__(self, images: torch.Tensor, labels: torch.Tensor, split: str, transform: Callable | None = None,
                 target_transform: Callable | None = None):
        if images.shape[0] != labels.shape[0]:
            raise DatasetFormatError("%d images but %d labels" % (images.shape[0], labels.shape[0]))
        if len(labels) and (int(labels.min()) < 0 or int(labels.max()) >= self.num_classes):
            raise DatasetFormatError("label outside [0, %d)" % self.num_classes)
        self.images, self.labels, self.split = images, labels, split
        self.transform, self.target_transform = transform, target_transform

    def __len__(self) -> int:
        return self.images.shape[0]

    def __getitem__(self, i: int):
        if not -len(self) <= i < len(self):
            raise IndexError("sample %d of %d" % (i, len(self)))
        img, lab = self.images[i].to(torch.float32) / 255.0, int(self.labels[i])
        if self.transform is not None:
            img = self.transform(img)
        if self.target_transform is not None:
            lab = self.target_transform(lab)
        return img, lab

    @classmethod
    def _synthetic_arrays(cls, split: str, n: int, shape: tuple[int, int, int]):
        """Class-dependent patterns plus noise, reproducible per split: a small model can learn them."""
        g = torch.Generator().manual_seed(0x5EED + (0 if split == "train" else 1) + 7 * cls.num_classes)
        labels = torch.randint(0, cls.num_classes, (n,), generator=g)
        c, h, w = shape
        yy, xx = torch.meshgrid(torch.arange(h), torch.arange(w), indexing="ij")
        base = torch.stack([((xx * (k % 5 + 1) + yy * (k // 5 + 1)) % 16).float() / 15.0 for k in range(cls.num_classes)])
        img = base[labels][:, None].expand(-1, c, -1, -1) * 0.7 + torch.rand((n, c, h, w), generator=g) * 0.3
        return (img * 255).round().to(torch.uint8), labels


# --------------------------------------------------------------------------- MNIST
def read_idx(data: bytes) -> np.ndarray:
    """One IDX file: two zero bytes, a type code, the number of dimensions, big-endian extents, data."""
    if len(data) < 4 or data[0] != 0 or data[1] != 0:
        raise DatasetFormatError("not an IDX file (bad magic)")
    codes = {0x08: np.uint8, 0x09: np.int8, 0x0B: ">i2", 0x0C: ">i4", 0x0D: ">f4", 0x0E: ">f8"}
    if data[2] not in codes:
        raise DatasetFormatError("IDX type code 0x%02x" % data[2])
    nd = data[3]
    if len(data) < 4 + 4 * nd:
        raise DatasetFormatError("IDX header truncated")
    dims = struct.unpack(">" + "I" * nd, data[4:4 + 4 * nd])
    dt = np.dtype(codes[data[2]])
    want = int(np.prod(dims, dtype=np.int64)) * dt.itemsize
    body = data[4 + 4 * nd:]
    if len(body) != want:
        raise DatasetFormatError("IDX body has %d bytes, header says %d" % (len(body), want))
    return np.frombuffer(body, dtype=dt).reshape(dims)


def write_idx(array: np.ndarray) -> bytes:
    """The inverse of :func:`read_idx` for uint8 arrays (fixtures, exports)."""
    a = np.ascontiguousarray(array, dtype=np.uint8)
    return bytes([0, 0, 0x08, a.ndim]) + struct.pack(">" + "I" * a.ndim, *a.shape) + a.tobytes()


class Mnist(_ArrayDataset):
    num_classes = 10
    FILES = {"train": ("train-images-idx3-ubyte", "train-labels-idx1-ubyte"), "test": ("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")}

    @classmethod
    def from_dir(cls, root: str, split="train", **kw) -> "Mnist":
        """The four canonical files (plain or ``.gz``) directly in ``root`` or in ``root/MNIST/raw``."""
        split = _split_name(split)
        for base in (root, os.path.join(root, "MNIST", "raw")):
            try:
                img = read_idx(_read_maybe_gz(os.path.join(base, cls.FILES[split][0])))
                lab = read_idx(_read_maybe_gz(os.path.join(base, cls.FILES[split][1])))
                break
            except FileNotFoundError:
                continue
        else:
            raise FileNotFoundError("no %s under %s" % (cls.FILES[split][0], root))
        if img.ndim != 3 or lab.ndim != 1 or img.dtype != np.uint8 or lab.dtype != np.uint8:
            raise DatasetFormatError("MNIST: images must be uint8 [N, H, W] and labels uint8 [N]")
        return cls(torch.from_numpy(img.copy())[:, None], torch.from_numpy(lab.astype(np.int64)), split, **kw)

    @classmethod
    def synthetic(cls, split="train", num_samples: int = 256, **kw) -> "Mnist":
        split = _split_name(split)
        return cls(*cls._synthetic_arrays(split, num_samples, (1, 28, 28)), split, **kw)


# --------------------------------------------------------------------------- CIFAR
def read_cifar_batches(blobs: list[bytes], label_bytes: int, label_index: int) -> tuple[torch.Tensor, torch.Tensor]:
    """CIFAR binary batches: records of ``label_bytes`` label bytes + 3072 pixel bytes (R, G, B planes
    of 32 x 32, row-major).  ``label_index`` picks the header byte that is the label."""
    rec = label_bytes + 3072
    imgs, labs = [], []
    for blob in blobs:
        if len(blob) == 0 or len(blob) % rec:
            raise DatasetFormatError("CIFAR batch of %d bytes is not a multiple of %d" % (len(blob), rec))
        a = np.frombuffer(blob, dtype=np.uint8).reshape(-1, rec)
        labs.append(a[:, label_index].astype(np.int64))
        imgs.append(a[:, label_bytes:].reshape(-1, 3, 32, 32))
    return torch.from_numpy(np.concatenate(imgs).copy()), torch.from_numpy(np.concatenate(labs))


class Cifar10(_ArrayDataset):
    num_classes = 10

    @classmethod
    def from_dir(cls, root: str, split="train", **kw) -> "Cifar10":
        split = _split_name(split)
        names = ["data_batch_%d.bin" % i for i in range(1, 6)] if split == "train" else ["test_batch.bin"]
        base = root if os.path.exists(os.path.join(root, names[0])) else os.path.join(root, "cifar-10-batches-bin")
        blobs = [_read_maybe_gz(os.path.join(base, n)) for n in names]
        return cls(*read_cifar_batches(blobs, 1, 0), split, **kw)

    @classmethod
    def synthetic(cls, split="train", num_samples: int = 256, **kw) -> "Cifar10":
        split = _split_name(split)
        return cls(*cls._synthetic_arrays(split, num_samples, (3, 32, 32)), split, **kw)


class Cifar100(_ArrayDataset):
    num_classes = 100

    @classmethod
    def from_dir(cls, root: str, split="train", **kw) -> "Cifar100":
        split = _split_name(split)
        name = "train.bin" if split == "train" else "test.bin"
        base = root if os.path.exists(os.path.join(root, name)) else os.path.join(root, "cifar-100-binary")
        return cls(*read_cifar_batches([_read_maybe_gz(os.path.join(base, name))], 2, 1), split, **kw)     # coarse, fine

    @classmethod
    def synthetic(cls, split="train", num_samples: int = 256, **kw) -> "Cifar100":
        split = _split_name(split)
        return cls(*cls._synthetic_arrays(split, num_samples, (3, 32, 32)), split, **kw)


# --------------------------------------------------------------------------- image folder
IMG_EXTENSIONS = (".jpg", ".jpeg", ".png", ".ppm", ".bmp", ".pgm", ".tif", ".tiff", ".webp")


class ImageFolder(Dataset):
    """``root/<class name>/**/<image>``: classes are the sorted sub-directory names, samples the
    image files below them in sorted order; images are decoded on access."""

    def __init__(self, root: str, transform: Callable | None = None, target_transform: Callable | None = None,
                 extensions: tuple[str, ...] = IMG_EXTENSIONS):
        self.root, self.transform, self.target_transform = root, transform, target_transform
        self.classes = sorted(d.name for d in os.scandir(root) if d.is_dir())
        if not self.classes:
            raise FileNotFoundError("no class folders in %s" % root)
        self.class_to_idx = {c: i for i, c in enumerate(self.classes)}
        self.samples = []
        for c in self.classes:
            for base, _dirs, files in sorted(os.walk(os.path.join(root, c), followlinks=True)):
                for f in sorted(files):
                    if f.lower().endswith(extensions):
                        self.samples.append((os.path.join(base, f), self.class_to_idx[c]))
        if not self.samples:
            raise FileNotFoundError("no image files below %s" % root)

    def __len__(self) -> int:
        return len(self.samples)

    # ---- folder.rs constructors
    @classmethod
    def from_dir(cls, root: str, **kw) -> "ImageFolder":
        return cls(root, **kw)

    @classmethod
    def from_dir_with_extensions(cls, root: str, extensions, **kw) -> "ImageFolder":
        exts = tuple(e.lower() if e.startswith(".") else "." + e.lower() for e in extensions)
        return cls(root, extensions=exts, **kw)

    @classmethod
    def from_dir_with_filter(cls, root: str, keep, **kw) -> "ImageFolder":
        """Only the files for which ``keep(path)`` is true."""
        ds = cls(root, **kw)
        ds.samples = [(p, c) for p, c in ds.samples if keep(p)]
        if not ds.samples:
            raise FileNotFoundError("the filter left no image below %s" % root)
        return ds

    def num_classes(self) -> int:
        return len(self.classes)

    def __getitem__(self, i: int):
        from .io import read_image_as_tensor

        path, lab = self.samples[i]
        img = read_image_as_tensor(path)
        if self.transform is not None:
            img = self.transform(img)
        if self.target_transform is not None:
            lab = self.target_transform(lab)
        return img, lab
