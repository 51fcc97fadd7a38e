"""Structured metrics: JSONL logger, running meters, top-k accuracy, CSV export.

Counterpart of the reference's AverageMeter / ProgressMeter / accuracy helpers
and its per-epoch pandas CSV (hw/models/train_imagenet.py:372-393,585-678), with
records as JSON lines instead of prints.
"""
from __future__ import annotations

import csv
import json
import time
from pathlib import Path

import torch
import torch.distributed as dist


class MetricsLogger:
    """Appends one JSON object per call to ``path`` (rank 0 only unless all_ranks)."""

    def __init__(self, path: str = "", rank: int = 0, all_ranks: bool = False):
        self.enabled = bool(path) and (all_ranks or rank == 0)
        self.rank = rank
        self.f = None
        if self.enabled:
            p = Path(path if not all_ranks else f"{path}.rank{rank}")
            p.parent.mkdir(parents=True, exist_ok=True)
            self.f = open(p, "a", buffering=1)

    def log(self, **kv) -> None:
        if self.f is None:
            return
        kv = {k: v for k, v in kv.items() if v is not None}
        kv["t"] = time.time()
        kv["rank"] = self.rank
        self.f.write(json.dumps(kv) + "\n")

    def close(self) -> None:
        if self.f is not None:
            self.f.close()
            self.f = None


class AverageMeter:
    """Running sum / count / average, all-reducible across ranks
    (hw/models/train_imagenet.py:591-641)."""

    def __init__(self, name: str, fmt: str = ":f"):
        self.name, self.fmt = name, fmt
        self.reset()

    def reset(self) -> None:
        self.val = self.sum = self.count = 0.0

    @property
    def avg(self) -> float:
        return self.sum / self.count if self.count else 0.0

    def update(self, val: float, n: int = 1) -> None:
        self.val = float(val)
        self.sum += float(val) * n
        self.count += n

    def all_reduce(self, device=None) -> None:
        if not (dist.is_available() and dist.is_initialized()):
            return
        dev = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
        t = torch.tensor([self.sum, self.count], dtype=torch.float32, device=dev)
        dist.all_reduce(t)
        self.sum, self.count = (float(v) for v in t.tolist())

    def __str__(self) -> str:
        return ("{name} {val" + self.fmt + "} ({avg" + self.fmt + "})").format(name=self.name, val=self.val, avg=self.avg)


class ProgressMeter:
    def __init__(self, num_batches: int, meters, prefix: str = ""):
        width = len(str(num_batches))
        self.fmt = "[{:" + str(width) + "d}/" + str(num_batches) + "]"
        self.meters, self.prefix = meters, prefix

    def line(self, batch: int) -> str:
        return "\t".join([self.prefix + self.fmt.format(batch)] + [str(m) for m in self.meters])

    def display(self, batch: int) -> None:
        print(self.line(batch), flush=True)


@torch.no_grad()
def accuracy(output: torch.Tensor, target: torch.Tensor, topk=(1,)):
    """Top-k accuracy in percent (hw/models/train_imagenet.py:664-678)."""
    maxk = max(topk)
    _, pred = output.topk(maxk, 1, True, True)
    correct = pred.t().eq(target.view(1, -1).expand(maxk, -1))
    return [correct[:k].reshape(-1).float().sum() * (100.0 / target.size(0)) for k in topk]


def append_csv(path: str, row: dict) -> None:
    """Append one row; the header is written when the file is new."""
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    new = not p.exists()
    with open(p, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(row))
        if new:
            w.writeheader()
        w.writerow(row)
