"""Input pipelines on small on-disk fixtures (CPU only): image folders with the ImageNet augmentations and
the CIFAR-10 batches with crop and flip, read by worker processes and sharded over ranks."""
import os
import pickle

import numpy as np
import pytest
import torch

from gcow_b200.data import Cifar10U8, EpochLoader, ImageFolderU8, make_loaders


@pytest.fixture(scope="module")
def image_tree(tmp_path_factory):
    from PIL import Image
    root = tmp_path_factory.mktemp("imgs")
    rng = np.random.default_rng(0)
    for split, per_class in (("train", 16), ("val", 8)):
        for ci, cname in enumerate(("apple", "bird", "cat", "dog")):
            d = root / split / cname
            d.mkdir(parents=True)
            for i in range(per_class):
                h, w = int(rng.integers(40, 90)), int(rng.integers(40, 90))
                a = np.full((h, w, 3), 60 * ci, dtype=np.uint8)
                a[:, :, 0] = i                                  # red channel = index within the class
                Image.fromarray(a).save(d / f"{i:03d}.png")
    return str(root)


@pytest.fixture(scope="module")
def cifar_tree(tmp_path_factory):
    root = tmp_path_factory.mktemp("cifar") / "cifar-10-batches-py"
    root.mkdir()
    rng = np.random.default_rng(1)
    for name, n in (("data_batch_1", 40), ("data_batch_2", 24), ("test_batch", 16)):
        rec = {"data": rng.integers(0, 256, (n, 3072), dtype=np.uint8), "labels": [int(v) for v in rng.integers(0, 10, n)]}
        with open(root / name, "wb") as f:
            pickle.dump(rec, f)
    return str(root.parent)


def test_image_folder_batches_are_uint8_nhwc_and_sharded(image_tree):
    seen = []
    for rank in range(2):
        tr, va = make_loaders(image_tree, False, 8, rank, 2, workers=2, seed=3, image=32)
        assert tr.classes == 4 and len(tr) == 4                 # 64 images / 2 ranks / batch 8
        got = []
        for x, y in tr:
            assert x.dtype == torch.uint8 and x.shape == (8, 32, 32, 3) and y.dtype == torch.int64
            got += [(int(t[0, 0, 0]), int(c)) for t, c in zip(x, y)]   # (index within class, class)
        seen.append(set(got))
        vx, vy = next(iter(va))
        assert vx.shape[1:] == (32, 32, 3) and len(va) == 2     # 32 validation images over 2 ranks
    assert not (seen[0] & seen[1]) and len(seen[0] | seen[1]) == 64   # the ranks see disjoint halves of the epoch


def test_image_folder_epochs_reshuffle(image_tree):
    tr, _ = make_loaders(image_tree, False, 8, 0, 1, workers=0, seed=3, image=32)
    first = torch.cat([y for _, y in tr])
    second = torch.cat([y for _, y in tr])
    assert first.numel() == 64 and not torch.equal(first, second)
    assert torch.equal(first.sort().values, second.sort().values)


def test_validation_transform_is_resize_and_centre_crop(image_tree):
    ds = ImageFolderU8(os.path.join(image_tree, "val"), train=False, size=32)
    x, y = ds[0]
    assert x.shape == (32, 32, 3) and int(x[0, 0, 1]) == 0 and y == 0     # class 0 is painted 0 in green / blue


def test_cifar_batches_crop_and_flip(cifar_tree):
    tr = Cifar10U8(cifar_tree, train=True, seed=5)
    te = Cifar10U8(cifar_tree, train=False)
    assert len(tr) == 64 and len(te) == 16
    raw = tr.x[7]
    x, y = tr[7]
    assert x.shape == (32, 32, 3) and x.dtype == torch.uint8 and y == int(tr.y[7])
    # an augmented item is a 32x32 window of the zero-padded image, possibly mirrored
    pad = np.zeros((40, 40, 3), dtype=np.uint8)
    pad[4:36, 4:36] = raw
    windows = [pad[a:a + 32, b:b + 32] for a in range(9) for b in range(9)]
    assert any(np.array_equal(x.numpy(), w) or np.array_equal(x.numpy(), w[:, ::-1]) for w in windows)
    xt, _ = te[3]
    assert np.array_equal(xt.numpy(), te.x[3])                   # no augmentation on the test split
    loader = EpochLoader(tr, 16, 1, 2, True, workers=2, seed=5)
    batches = list(loader)
    assert len(batches) == 2 and batches[0][0].shape == (16, 32, 32, 3)


def test_torchvision_architectures_run_on_swapped_layers():
    from gcow_b200.models import build_model, torchvision_names
    from gcow_b200.ops import nn as gnn
    assert "mobilenet_v2" in torchvision_names() and "resnet18" in torchvision_names()
    net = build_model("squeezenet1_1", num_classes=7)
    assert any(isinstance(m, gnn.Conv2d) for m in net.modules())
    assert not any(type(m) is torch.nn.Conv2d for m in net.modules())
    y = net(torch.randn(2, 3, 64, 64))                            # on the CPU the layers fall back to PyTorch's math
    assert y.shape == (2, 7)
    ref = build_model("resnet18", num_classes=7)
    assert type(ref).__module__.startswith("gcow_b200.models")   # own zoo first
