"""Input pipelines of the two studies: an image-folder tree with the ImageNet augmentations and the
CIFAR-10 batches with crop-and-flip, both read by worker processes and sharded over ranks.

The reference builds ``ImageFolder(train, RandomResizedCrop(224) + RandomHorizontalFlip + ToTensor +
Normalize)`` and ``ImageFolder(val, Resize(256) + CenterCrop(224) + ...)`` behind DataLoaders with
``--workers`` processes, pinned memory and a DistributedSampler (hw/models/train_imagenet.py:283-324), and
CIFAR-10 with ``RandomCrop(32, padding=4) + RandomHorizontalFlip`` (hw/models/train_resnet_cifar10.py:17-32).
Here the workers stop at uint8: a batch leaves the loader as a pinned ``[B, H, W, 3]`` uint8 tensor (a
quarter of the float bytes over PCIe) and ``ToTensor + Normalize`` happen on the GPU inside the trainer's
image-normalise kernel. Decoding and the geometric augmentations are torchvision's, run on the CPU workers.
"""
from __future__ import annotations

import os
import pickle
from typing import Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset
from torch.utils.data.distributed import DistributedSampler


def _to_u8_hwc(img) -> torch.Tensor:
    """PIL image -> uint8 [H, W, 3] tensor."""
    return torch.from_numpy(np.array(img.convert("RGB"), dtype=np.uint8))      # np.array copies: a writable buffer


class ImageFolderU8(Dataset):
    """``root/<class>/<image>`` as torchvision's ImageFolder reads it; items are (uint8 HWC image, label)."""

    def __init__(self, root: str, train: bool, size: int = 224):
        import torchvision.datasets as datasets
        import torchvision.transforms as T
        if train:          # hw/models/train_imagenet.py:296-301
            tf = T.Compose([T.RandomResizedCrop(size), T.RandomHorizontalFlip(), T.Lambda(_to_u8_hwc)])
        else:              # hw/models/train_imagenet.py:306-310 (256 / 224 scaled with the crop size)
            tf = T.Compose([T.Resize(int(round(size * 256 / 224))), T.CenterCrop(size), T.Lambda(_to_u8_hwc)])
        self.inner = datasets.ImageFolder(root, tf)
        self.classes = self.inner.classes

    def __len__(self):
        return len(self.inner)

    def __getitem__(self, i):
        return self.inner[i]


class Cifar10U8(Dataset):
    """The python version of CIFAR-10 (``cifar-10-batches-py``: data_batch_1..5, test_batch; each a pickle with a
    ``data`` array [n, 3072] uint8 in CHW order and ``labels``). Training items get RandomCrop(32, padding=4) and a
    random horizontal flip, as the reference's study does; items are (uint8 HWC image, label)."""

    def __init__(self, root: str, train: bool, seed: int = 0):
        d = root if os.path.exists(os.path.join(root, "test_batch")) else os.path.join(root, "cifar-10-batches-py")
        names = [f"data_batch_{i}" for i in range(1, 6)] if train else ["test_batch"]
        xs, ys = [], []
        for n in names:
            path = os.path.join(d, n)
            if not os.path.exists(path):
                if train and xs:
                    continue                      # a partial copy (fewer training batches) still trains
                raise FileNotFoundError(f"{path}: expected the python version of CIFAR-10 under {root}")
            with open(path, "rb") as f:
                rec = pickle.load(f, encoding="latin1")
            xs.append(np.asarray(rec["data"], dtype=np.uint8).reshape(-1, 3, 32, 32))
            ys.append(np.asarray(rec.get("labels", rec.get("fine_labels")), dtype=np.int64))
        self.x = np.ascontiguousarray(np.concatenate(xs).transpose(0, 2, 3, 1))       # NHWC
        self.y = np.concatenate(ys)
        self.train = train
        self.classes = [str(i) for i in range(10)]
        self.seed = seed

    def __len__(self):
        return len(self.y)

    def __getitem__(self, i):
        img = self.x[i]
        if self.train:
            # per-item generator: reproducible and independent of which worker serves the item
            g = np.random.default_rng((self.seed, int(i), int(torch.initial_seed() & 0xffffffff)))
            pad = np.zeros((40, 40, 3), dtype=np.uint8)
            pad[4:36, 4:36] = img
            oy, ox = g.integers(0, 9, 2)
            img = pad[oy:oy + 32, ox:ox + 32]
            if g.random() < 0.5:
                img = img[:, ::-1]
        return torch.from_numpy(np.ascontiguousarray(img)), int(self.y[i])


def _collate_u8(items):
    return torch.stack([x for x, _ in items]), torch.tensor([y for _, y in items], dtype=torch.int64)


class EpochLoader:
    """DataLoader + DistributedSampler with the epoch re-seeding done at iteration start, so the training loop
    can simply ``for x, y in loader``. ``drop_last`` keeps every step's shape (and every rank's step count) equal."""

    def __init__(self, dataset: Dataset, batch: int, rank: int, world: int, train: bool, workers: int, seed: int = 0):
        self.sampler: Optional[DistributedSampler] = None
        if world > 1 or train:
            self.sampler = DistributedSampler(dataset, num_replicas=world, rank=rank, shuffle=train, seed=seed,
                                              drop_last=train)
        self.loader = DataLoader(dataset, batch_size=batch, shuffle=False, sampler=self.sampler, num_workers=workers,
                                 pin_memory=torch.cuda.is_available(), drop_last=train, collate_fn=_collate_u8,
                                 persistent_workers=workers > 0)
        self.epoch = 0
        self.classes = len(getattr(dataset, "classes", [])) or None

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        if self.sampler is not None:
            self.sampler.set_epoch(self.epoch)
        self.epoch += 1
        return iter(self.loader)


def make_loaders(root: str, cifar: bool, batch: int, rank: int, world: int, workers: int, seed: int = 0,
                 image: int = 224):
    """(train_loader, val_loader) for ``root``: ``train/`` and ``val/`` class folders, or the CIFAR-10 batches."""
    if cifar:
        tr, va = Cifar10U8(root, True, seed), Cifar10U8(root, False, seed)
    else:
        tr = ImageFolderU8(os.path.join(root, "train"), True, image)
        va = ImageFolderU8(os.path.join(root, "val"), False, image)
    return (EpochLoader(tr, batch, rank, world, True, workers, seed),
            EpochLoader(va, batch, rank, world, False, workers, seed))
