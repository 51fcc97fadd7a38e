"""Checkpoint / resume. Rank 0 writes ``<path>`` atomically (temp file + rename)
and optionally a ``_best`` copy; every rank can load with a device remap.
Same content as the reference's tar (epoch, arch, state_dict, best_acc1,
optimizer, scheduler: hw/models/train_imagenet.py:360-369,579-583) plus the
compression hook's state."""
from __future__ import annotations

import os
import shutil
from pathlib import Path

import torch
import torch.distributed as dist


def save_checkpoint(state: dict, path: str, is_best: bool = False, rank: int | None = None) -> None:
    if rank is None:
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if rank != 0:
        return
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    tmp = p.with_suffix(p.suffix + ".tmp")
    torch.save(state, tmp)
    os.replace(tmp, p)
    if is_best:
        shutil.copyfile(p, p.with_name(p.stem + "_best" + p.suffix))


def load_checkpoint(path: str, map_location=None) -> dict:
    return torch.load(path, map_location=map_location or "cpu", weights_only=False)
