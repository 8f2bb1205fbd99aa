"""Own dataset readers (IDX, CIFAR binary, image folder) and tensor transforms: file formats
round-trip through fixtures written here, malformed files are typed errors, the deterministic
transform kernels equal ``torchvision.transforms.functional`` on tensors, random pipelines are
reproducible from a seed."""
import gzip
import os

import numpy as np
import pytest
import torch

from ferrotorch_b200 import vision as V
from ferrotorch_b200.vision import datasets as DS
from ferrotorch_b200.vision import own_transforms as O


def test_mnist_idx_files_plain_and_gz(tmp_path):
    rng = np.random.default_rng(0)
    img, lab = rng.integers(0, 256, (5, 28, 28), dtype=np.uint8), rng.integers(0, 10, (5,), dtype=np.uint8)
    (tmp_path / "train-images-idx3-ubyte").write_bytes(DS.write_idx(img))
    (tmp_path / "train-labels-idx1-ubyte").write_bytes(DS.write_idx(lab))
    raw = tmp_path / "MNIST" / "raw"
    raw.mkdir(parents=True)
    with gzip.open(raw / "t10k-images-idx3-ubyte.gz", "wb") as f:
        f.write(DS.write_idx(img[:2]))
    with gzip.open(raw / "t10k-labels-idx1-ubyte.gz", "wb") as f:
        f.write(DS.write_idx(lab[:2]))
    tr = V.Mnist.from_dir(str(tmp_path), V.Split.Train)
    te = V.Mnist.from_dir(str(tmp_path), "test", transform=lambda t: t * 2)
    assert len(tr) == 5 and len(te) == 2 and tr.split == "train"
    x, y = tr[3]
    assert x.shape == (1, 28, 28) and x.dtype == torch.float32 and y == int(lab[3])
    assert torch.equal(x[0], torch.from_numpy(img[3]).float() / 255)
    assert torch.equal(te[1][0], tr[1][0] * 2)
    with pytest.raises(IndexError):
        tr[5]
    # malformed files: bad magic, truncated body, label out of range, count mismatch
    with pytest.raises(DS.DatasetFormatError):
        DS.read_idx(b"\x01\x00\x08\x01" + b"\x00" * 8)
    with pytest.raises(DS.DatasetFormatError):
        DS.read_idx(DS.write_idx(img)[:-3])
    (tmp_path / "train-labels-idx1-ubyte").write_bytes(DS.write_idx(np.array([1, 2, 3, 4, 11], dtype=np.uint8)))
    with pytest.raises(DS.DatasetFormatError):
        V.Mnist.from_dir(str(tmp_path), "train")
    (tmp_path / "train-labels-idx1-ubyte").write_bytes(DS.write_idx(lab[:4]))
    with pytest.raises(DS.DatasetFormatError):
        V.Mnist.from_dir(str(tmp_path), "train")
    with pytest.raises(FileNotFoundError):
        V.Mnist.from_dir(str(tmp_path / "nowhere"), "train")


def test_cifar_binary_batches(tmp_path):
    rng = np.random.default_rng(1)

    def records(n, label_bytes, classes):
        head = rng.integers(0, classes, (n, label_bytes), dtype=np.uint8)
        px = rng.integers(0, 256, (n, 3072), dtype=np.uint8)
        return head, px, np.concatenate([head, px], 1).tobytes()

    d10 = tmp_path / "cifar-10-batches-bin"
    d10.mkdir()
    heads, pixels = [], []
    for i in range(1, 6):
        h, p, blob = records(3, 1, 10)
        heads.append(h), pixels.append(p)
        (d10 / ("data_batch_%d.bin" % i)).write_bytes(blob)
    h, p, blob = records(2, 1, 10)
    (d10 / "test_batch.bin").write_bytes(blob)
    tr, te = V.Cifar10.from_dir(str(tmp_path), "train"), V.Cifar10.from_dir(str(d10), "test")
    assert len(tr) == 15 and len(te) == 2 and V.Cifar10.num_classes == 10
    x, y = tr[4]                                   # second record of the second batch
    assert y == int(heads[1][1, 0]) and x.shape == (3, 32, 32)
    assert torch.equal(x, torch.from_numpy(pixels[1][1].reshape(3, 32, 32).copy()).float() / 255)   # R, G, B planes
    d100 = tmp_path / "c100"
    d100.mkdir()
    h, p, blob = records(4, 2, 20)
    (d100 / "train.bin").write_bytes(blob)
    c100 = V.Cifar100.from_dir(str(d100), "train")
    assert [c100[i][1] for i in range(4)] == [int(v) for v in h[:, 1]], "the fine label is the second header byte"
    (d100 / "test.bin").write_bytes(blob[:-1])
    with pytest.raises(DS.DatasetFormatError):
        V.Cifar100.from_dir(str(d100), "test")


def test_synthetic_sets_are_reproducible_and_learnable():
    a, b = V.Mnist.synthetic("train", 64), V.Mnist.synthetic("train", 64)
    c = V.Mnist.synthetic("test", 64)
    assert torch.equal(a.images, b.images) and not torch.equal(a.images, c.images)
    ds = V.Cifar10.synthetic("train", 256)
    x = torch.stack([ds[i][0] for i in range(256)]).flatten(1)
    y = torch.tensor([ds[i][1] for i in range(256)])
    torch.manual_seed(0)
    lin = torch.nn.Linear(x.shape[1], 10)
    opt = torch.optim.Adam(lin.parameters(), 1e-2)
    first = last = None
    for _ in range(30):
        loss = torch.nn.functional.cross_entropy(lin(x), y)
        opt.zero_grad(), loss.backward(), opt.step()
        first, last = (float(loss.detach()) if first is None else first), float(loss.detach())
    assert last < 0.5 * first


def test_image_folder_reads_own_image_files(tmp_path):
    for cls, val in (("cats", 0.2), ("dogs", 0.8)):
        (tmp_path / cls / "nested").mkdir(parents=True)
        V.write_tensor_as_image(str(tmp_path / cls / "a.png"), torch.full((3, 6, 5), val))
        V.write_tensor_as_image(str(tmp_path / cls / "nested" / "b.png"), torch.full((3, 6, 5), val))
    (tmp_path / "cats" / "notes.txt").write_text("not an image")
    ds = DS.ImageFolder(str(tmp_path), transform=O.Resize((4, 4)))
    assert ds.classes == ["cats", "dogs"] and len(ds) == 4 and [s[1] for s in ds.samples] == [0, 0, 1, 1]
    x, y = ds[3]
    assert x.shape == (3, 4, 4) and y == 1 and abs(float(x.mean()) - 0.8) < 0.01
    with pytest.raises(FileNotFoundError):
        DS.ImageFolder(str(tmp_path / "cats" / "nested"))


def test_deterministic_transforms_equal_torchvision_functional():
    TF = pytest.importorskip("torchvision.transforms.functional")
    from torchvision.transforms import InterpolationMode as IM

    torch.manual_seed(0)
    x, xb = torch.rand(3, 37, 45), torch.rand(2, 3, 32, 40)

    def close(a, b, tol=1e-5):
        assert a.shape == b.shape and torch.allclose(a, b, atol=tol), (a - b).abs().max()

    close(O.center_crop(x, (20, 30)), TF.center_crop(x, [20, 30]))
    close(O.center_crop(x, (50, 60)), TF.center_crop(x, [50, 60]))                       # larger than the image: padded
    close(O.resize(x, 24), TF.resize(x, [24], antialias=True))
    close(O.resize(x, (50, 20)), TF.resize(x, [50, 20], antialias=True))
    close(O.resize(xb, (16, 16), antialias=False), TF.resize(xb, [16, 16], antialias=False))
    for ang in (30.0, -75.0, 135.0):
        close(O.rotate(x, ang), TF.rotate(x, ang))
        close(O.rotate(x, ang, fill=0.5, mode="bilinear"), TF.rotate(x, ang, interpolation=IM.BILINEAR, fill=[0.5]), 1e-4)
    close(O.affine(x, 20.0, (3, -4), 1.2, (10.0, 5.0)), TF.affine(x, 20.0, [3, -4], 1.2, [10.0, 5.0]))
    close(O.affine(xb, 0.0, (5, 0), 1.0, (0.0, 0.0), 0.3, "bilinear"),
          TF.affine(xb, 0.0, [5, 0], 1.0, [0.0, 0.0], interpolation=IM.BILINEAR, fill=[0.3]), 1e-4)
    close(O.adjust_brightness(x, 1.3), TF.adjust_brightness(x, 1.3))
    close(O.adjust_contrast(x, 0.6), TF.adjust_contrast(x, 0.6))
    close(O.adjust_saturation(x, 1.7), TF.adjust_saturation(x, 1.7))
    for h in (-0.3, 0.1, 0.5):
        close(O.adjust_hue(x, h), TF.adjust_hue(x, h), 1e-4)
    close(O.posterize(x, 3), TF.posterize((x * 255).to(torch.uint8), 3).float() / 255)
    close(O.solarize(x, 0.4), TF.solarize(x, 0.4))
    close(O.autocontrast(x), TF.autocontrast(x))
    close(O.adjust_sharpness(x, 1.8), TF.adjust_sharpness(x, 1.8))
    xq = (x * 255).round() / 255
    close(O.equalize(xq), TF.equalize((xq * 255).to(torch.uint8)).float() / 255)
    close(O.hflip(x), TF.hflip(x)), close(O.vflip(x), TF.vflip(x))


def test_random_pipelines_are_reproducible_and_keep_their_contracts():
    pipe = O.Compose([O.RandomResizedCrop(24, scale=(0.3, 1.0)), O.RandomHorizontalFlip(), O.RandomVerticalFlip(0.3),
                      O.RandomRotation(25, mode="bilinear"), O.ColorJitter(0.4, 0.4, 0.4, 0.1),
                      O.RandomApply([O.ElasticTransform(8.0, 3.0)], p=0.7),
                      O.RandomChoice([O.RandomCrop(20, padding=2), O.CenterCrop(20)]), O.TrivialAugmentWide()])
    x = torch.rand(3, 40, 52)
    V.vision_manual_seed(123)
    a = [pipe(x) for _ in range(6)]
    V.vision_manual_seed(123)
    b = [pipe(x) for _ in range(6)]
    V.vision_manual_seed(124)
    c = [pipe(x) for _ in range(6)]
    assert all(torch.equal(p, q) for p, q in zip(a, b)) and not all(torch.equal(p, q) for p, q in zip(a, c))
    for t in a:
        assert t.shape == (3, 20, 20) and torch.isfinite(t).all() and t.min() >= -1e-6 and t.max() <= 1 + 1e-6
    # every TrivialAugmentWide operation keeps shape and range; batched input works too
    taw = O.TrivialAugmentWide()
    for name, (mags, _signed) in taw._space().items():
        y = taw.apply_op(x, name, float(mags[-1]) if mags is not None else 0.0)
        assert y.shape == x.shape and torch.isfinite(y).all(), name
    assert O.ElasticTransform(5.0, 2.0)(torch.rand(2, 3, 16, 16)).shape == (2, 3, 16, 16)
    crops = {tuple(O.RandomResizedCrop(8).get_params(30, 50)) for _ in range(20)}
    assert len(crops) > 5 and all(0 <= t and 0 <= l and t + h <= 30 and l + w <= 50 for t, l, h, w in crops)
    with pytest.raises(ValueError):
        O.RandomCrop(64)(x)
    with pytest.raises(ValueError):
        O.ColorJitter(hue=0.7)
