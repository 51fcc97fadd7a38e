"""Training front end: the call a user makes to train with compressed gradients.

    trainer = Trainer("resnet50", batch_size=256)          # one process per GPU
    for images_u8, labels in loader:                        # pinned host tensors
        loss = trainer.step(images_u8, labels)              # host float (one step late)

``Trainer.step`` copies the batch host->device on a prefetch stream, runs forward
and backward in bf16 autocast with fp32 gradients, lets the DDP hook all-reduce
each 25 MB bucket with the fused compressed kernel on the communication stream,
checks the collective status, applies the fused optimizer and copies the loss
back to pinned memory. The same loop with ``variant="nccl"`` and
``ops="torch"`` is the uncompressed NCCL(+cuBLAS/cuDNN) baseline.

Mirrors the reference's loops (hw/models/train_imagenet.py:404-486,
hw/models/train_resnet_cifar10.py:74-125) with the host codec round trip replaced
by the on-the-wire kernel; SGD 0.1/0.9/1e-4 and StepLR(30, 0.1) as there
(hw/models/train_imagenet.py:251-256).
"""
from __future__ import annotations

import math
import os
import tempfile
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .config import GcowConfig
from .models import build_model
from .ops import backend as ops_backend
from .ops.optim import FusedAdamW, FusedSGD
from .parallel.ddp import wrap_ddp
from .utils.logging import MetricsLogger

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def ensure_process_group(device: torch.device) -> None:
    """Join the job's process group, or create a single-rank one for 1-GPU runs."""
    if dist.is_initialized():
        return
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo",
                                device_id=device if device.type == "cuda" else None)
        return
    f = tempfile.NamedTemporaryFile(prefix="gcow_pg_", delete=False)
    f.close()
    dist.init_process_group("nccl" if device.type == "cuda" else "gloo", init_method=f"file://{f.name}",
                            rank=0, world_size=1)


class SyntheticImages:
    """Fixed pool of random uint8 NHWC images + labels in pinned host memory."""

    def __init__(self, batch: int, size: int = 224, classes: int = 1000, pool: int = 4, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.x = [torch.randint(0, 256, (batch, size, size, 3), dtype=torch.uint8, generator=g) for _ in range(pool)]
        self.y = [torch.randint(0, classes, (batch,), dtype=torch.int64, generator=g) for _ in range(pool)]
        if torch.cuda.is_available():
            self.x = [t.pin_memory() for t in self.x]
            self.y = [t.pin_memory() for t in self.y]
        self.i = 0

    def next(self):
        i = self.i % len(self.x)
        self.i += 1
        return self.x[i], self.y[i]

    @property
    def bytes_per_batch(self) -> int:
        return self.x[0].numel() * self.x[0].element_size() + self.y[0].numel() * 8


class LearnableImages:
    """A classification task that can be learned: every class has a fixed random low-resolution pattern, an image is
    its class pattern plus pixel noise. Fresh batches every call (uint8 NHWC, pinned), the same patterns on every
    rank, different samples per rank. Used to compare loss curves across compression rates."""

    def __init__(self, batch: int, size: int = 64, classes: int = 10, seed: int = 0, noise: float = 48.0,
                 pattern_seed: int = 1234):
        g = torch.Generator().manual_seed(pattern_seed)
        coarse = torch.rand((classes, 8, 8, 3), generator=g) * 160.0 + 48.0
        rep = size // 8
        self.patterns = coarse.repeat_interleave(rep, 1).repeat_interleave(rep, 2)          # [classes, size, size, 3]
        self.batch, self.classes, self.noise = batch, classes, noise
        self.gen = torch.Generator().manual_seed(seed)

    def next(self):
        y = torch.randint(0, self.classes, (self.batch,), generator=self.gen)
        x = self.patterns[y] + torch.randn((self.batch,) + tuple(self.patterns.shape[1:]), generator=self.gen) * self.noise
        x = x.clamp_(0, 255).to(torch.uint8)
        if torch.cuda.is_available():
            x, y = x.pin_memory(), y.pin_memory()
        return x, y


class SyntheticTokens:
    """Random token ids uniform over the vocabulary, 15 % masked-LM labels, NSP labels."""

    def __init__(self, batch: int, seq: int = 512, vocab: int = 30522, pool: int = 4, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.ids, self.mlm, self.nsp = [], [], []
        for _ in range(pool):
            ids = torch.randint(0, vocab, (batch, seq), dtype=torch.int64, generator=g)
            mask = torch.rand((batch, seq), generator=g) < 0.15
            lab = torch.where(mask, ids, torch.full_like(ids, -100))
            nsp = torch.randint(0, 2, (batch,), dtype=torch.int64, generator=g)
            self.ids.append(ids); self.mlm.append(lab); self.nsp.append(nsp)
        if torch.cuda.is_available():
            self.ids = [t.pin_memory() for t in self.ids]
            self.mlm = [t.pin_memory() for t in self.mlm]
            self.nsp = [t.pin_memory() for t in self.nsp]
        self.i = 0

    def next(self):
        i = self.i % len(self.ids)
        self.i += 1
        return (self.ids[i], self.mlm[i], self.nsp[i]), None

    @property
    def bytes_per_batch(self) -> int:
        return (self.ids[0].numel() + self.mlm[0].numel() + self.nsp[0].numel()) * 8


@dataclass
class StepResult:
    loss: Optional[float]      # loss of the PREVIOUS step (None on the first call)
    step: int
    acc1: Optional[float] = None   # training top-1 / top-5 of the previous step in percent (with track_accuracy)
    acc5: Optional[float] = None


class Trainer:
    def __init__(self, model: str = "resnet50", batch_size: int = 256, cfg: GcowConfig | None = None,
                 ops: str = "own", lr: float | None = None, num_classes: int = 1000, seq_len: int = 512,
                 device: torch.device | None = None, log_path: str = "", seed: int = 0,
                 model_kwargs: dict | None = None, pretrained: bool = False, track_accuracy: bool = False):
        self.device = device or torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(self.device)
        ensure_process_group(self.device)
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.cfg = cfg or GcowConfig.from_env()
        ops_backend.set_backend(ops)
        model = model.replace("-", "_")
        self.kind = "bert" if model.startswith("bert") else "resnet"
        self.model_name, self.batch_size, self.seq_len = model, batch_size, seq_len
        torch.manual_seed(seed)                       # same initial weights on every rank
        kw = dict(model_kwargs or {})
        if self.kind == "resnet":
            kw.setdefault("num_classes", num_classes)
        net = build_model(model, pretrained=pretrained, **kw).to(self.device)
        if self.kind == "resnet":
            net = net.to(memory_format=torch.channels_last)
        self.ddp, self.hook_state = wrap_ddp(net, self.cfg, self.device)
        params = [p for p in net.parameters() if p.requires_grad]
        self._grad_view_hints = ops == "own" and self.device.type == "cuda"
        self._hint_params = params
        if self.kind == "resnet":
            opt_cls = FusedSGD if ops == "own" else torch.optim.SGD
            self.opt = opt_cls(params, lr=lr or 0.1, momentum=0.9, weight_decay=1e-4)
            self.sched = torch.optim.lr_scheduler.StepLR(self.opt, step_size=30, gamma=0.1)
        else:
            if ops == "own":
                self.opt = FusedAdamW(params, lr=lr or 1e-4, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01)
            else:
                self.opt = torch.optim.AdamW(params, lr=lr or 1e-4, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01)
            self.sched = None
        self.mean = torch.tensor(IMAGENET_MEAN, device=self.device).view(1, 3, 1, 1) * 255.0
        self.std = torch.tensor(IMAGENET_STD, device=self.device).view(1, 3, 1, 1) * 255.0
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.track_accuracy = track_accuracy and self.kind == "resnet"
        self.loss_host = torch.zeros((2, 4), dtype=torch.float32)      # per slot: loss, top-1, top-5, unused
        if torch.cuda.is_available():
            self.loss_host = self.loss_host.pin_memory()
        self._stats = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.h2d_events: list = []          # (start, end) CUDA events of the batch copies, read by h2d_seconds()
        self.err_host = torch.zeros(2, dtype=torch.int32).pin_memory()    # compute kernels' error word, per slot
        self.loss_event: list[Optional[torch.cuda.Event]] = [None, None]
        self.steps = 0
        self.epoch = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.logger = MetricsLogger(log_path or self.cfg.log_path, self.rank)
        self._staged = None

    # ------------------------------------------------------------- data path
    def stage(self, inputs, targets):
        """Start the host->device copy of a batch on the prefetch stream."""
        with torch.cuda.stream(self.copy_stream):
            t0 = torch.cuda.Event(enable_timing=True)
            t0.record(self.copy_stream)
            if self.kind == "resnet":
                x = inputs.to(self.device, non_blocking=True)
                y = targets.to(self.device, non_blocking=True)
                self.h2d_bytes += inputs.numel() * inputs.element_size() + targets.numel() * targets.element_size()
                dev = (x, y)
            else:
                dev = tuple(t.to(self.device, non_blocking=True) for t in inputs)
                self.h2d_bytes += sum(t.numel() * t.element_size() for t in inputs)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(self.copy_stream)
            if len(self.h2d_events) < 100000:
                self.h2d_events.append((t0, ev))
        self._staged = (dev, ev)

    def _take_staged(self):
        dev, ev = self._staged
        self._staged = None
        torch.cuda.current_stream().wait_event(ev)
        for t in dev:
            t.record_stream(torch.cuda.current_stream())
        return dev

    def preprocess(self, x_u8: torch.Tensor) -> torch.Tensor:
        """uint8 NHWC -> normalised bf16, logical NCHW in channels-last memory."""
        if ops_backend.get_backend() == "own":
            from .ops import kernels
            return kernels.u8_to_bf16_norm(x_u8, [m * 255.0 for m in IMAGENET_MEAN], [s * 255.0 for s in IMAGENET_STD])
        x = x_u8.permute(0, 3, 1, 2)
        return ((x.to(torch.float32) - self.mean) / self.std).to(torch.bfloat16).contiguous(
            memory_format=torch.channels_last)

    # ------------------------------------------------------------------ step
    def compute_loss(self, dev) -> torch.Tensor:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            if self.kind == "resnet":
                x, y = dev
                if x.dtype == torch.uint8:
                    x = self.preprocess(x)
                out = self.ddp(x)
                logits = out.float()
                if self.track_accuracy:      # top-1 / top-5 as the reference's loop reports them (train_imagenet.py:437-440)
                    with torch.no_grad():
                        k = min(5, logits.shape[1])
                        hit = logits.topk(k, 1).indices.eq(y.view(-1, 1))
                        self._stats[1] = hit[:, :1].any(1).float().mean() * 100.0
                        self._stats[2] = hit.any(1).float().mean() * 100.0
                return F.cross_entropy(logits, y)
            ids, mlm, nsp = dev
            return self.ddp(ids, None, mlm, nsp)

    def step_device(self, dev) -> torch.Tensor:
        """One optimisation step on device-resident inputs. Returns the loss tensor."""
        if self.hook_state is not None:
            self.hook_state.begin_step()
        # Last step's gradients are DDP's bucket views, which is where this step's gradients will end up again: the
        # weight-gradient kernels may write there directly (kernels.take_grad_view, taken during the forward pass, at
        # most once per weight and step) and DDP then has nothing to copy.
        if self._grad_view_hints:
            for p in self._hint_params:
                p._gcow_grad_view = p.grad
        loss = self.compute_loss(dev)
        # gradients are dropped rather than zeroed: autograd then assigns instead of accumulating, and DDP points
        # .grad back at its bucket views during backward
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        if self.hook_state is not None:
            self.hook_state.finish_step()
        self.opt.step()
        self.steps += 1
        return loss.detach()

    def step(self, inputs, targets=None, prefetch=None) -> StepResult:
        """One end-to-end step from pinned host tensors. The returned loss is the
        previous step's (its device->host copy has completed by now), so the host
        never stalls the device. ``prefetch=(inputs, targets)`` of the NEXT step starts
        that batch's host->device copy on the prefetch stream while this step computes."""
        if self._staged is None:
            self.stage(inputs, targets)
        dev = self._take_staged()
        if prefetch is not None:
            self.stage(*prefetch)
        loss = self.step_device(dev)
        slot = self.steps & 1
        self._stats[0] = loss
        self.loss_host[slot].copy_(self._stats, non_blocking=True)
        if ops_backend.get_backend() == "own":
            from .ops import kernels
            self.err_host[slot:slot + 1].copy_(kernels.error_word(self.device), non_blocking=True)
            self.d2h_bytes += 4
        ev = torch.cuda.Event()
        ev.record()
        self.loss_event[slot] = ev
        self.d2h_bytes += 16
        prev = a1 = a5 = None
        pslot = slot ^ 1
        if self.loss_event[pslot] is not None:
            self.loss_event[pslot].synchronize()
            prev = float(self.loss_host[pslot, 0])
            if self.track_accuracy:
                a1, a5 = float(self.loss_host[pslot, 1]), float(self.loss_host[pslot, 2])
            self._raise_on_kernel_error(int(self.err_host[pslot]))
            if math.isnan(prev):
                raise FloatingPointError("loss is NaN: training diverged")   # train_imagenet.py:445-446
        if self.logger.enabled:
            self.logger.log(step=self.steps, loss=prev, **(self.hook_state.step_record() if self.hook_state else {}))
        return StepResult(prev, self.steps, a1, a5)

    def _raise_on_kernel_error(self, code: int) -> None:
        if code:
            from .ops import kernels
            kernels.error_word(self.device).zero_()
            self.err_host.zero_()
            raise kernels.KernelWaitAbandoned(
                f"a tensor-core kernel on {self.device} abandoned a wait (role code {code}) in step {self.steps - 1}: "
                f"that step's activations or gradients are incomplete")

    def last_loss(self) -> float:
        """Loss of the latest ``step`` call (synchronises); raises if a compute kernel gave up during it."""
        torch.cuda.current_stream().synchronize()
        if self.hook_state is not None:          # the per-step check of the collective lags by one step: settle it here
            self.hook_state.ar.check()
        self._raise_on_kernel_error(int(self.err_host[self.steps & 1]))
        return float(self.loss_host[self.steps & 1, 0])

    def h2d_seconds(self) -> float:
        """Device time of the host->device batch copies since the last call (synchronises with the copy stream)."""
        self.copy_stream.synchronize()
        t = sum(a.elapsed_time(b) for a, b in self.h2d_events) / 1e3
        self.h2d_events.clear()
        return t

    # ------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        return {"model": self.ddp.module.state_dict(), "optimizer": self.opt.state_dict(),
                "scheduler": self.sched.state_dict() if self.sched else None, "steps": self.steps,
                "epoch": self.epoch, "arch": self.model_name, "cfg": self.cfg.asdict(),
                "hook": self.hook_state.state_dict() if self.hook_state else None}

    def load_state_dict(self, sd: dict) -> None:
        self.ddp.module.load_state_dict(sd["model"])
        self.opt.load_state_dict(sd["optimizer"])
        if self.sched and sd.get("scheduler"):
            self.sched.load_state_dict(sd["scheduler"])
        self.steps, self.epoch = sd["steps"], sd.get("epoch", 0)
        if self.hook_state and sd.get("hook"):
            self.hook_state.load_state_dict(sd["hook"])

    def gpu_launches(self) -> int:
        """Launches of this library's own kernels so far (collective + optimizer + ops)."""
        from .ops import kernels
        n = self.hook_state.launches if self.hook_state else 0
        n += getattr(self.opt, "launches", 0)
        n += kernels.launch_count()
        return n


def make_loader(kind: str, batch: int, seq_len: int = 512, image: int = 224, classes: int = 1000,
                vocab: int = 30522, seed: int = 0):
    return SyntheticImages(batch, image, classes, seed=seed) if kind == "resnet" else \
        SyntheticTokens(batch, seq_len, vocab, seed=seed)


def smoke_step() -> None:
    """One tiny forward+backward+update of the flagship path on cuda:0."""
    cfg = GcowConfig(rate=8, comm_ctas=16, bucket_mb=1)
    tr = Trainer("resnet18", batch_size=4, cfg=cfg, num_classes=10, device=torch.device("cuda", 0))
    loader = SyntheticImages(4, 64, 10, pool=2)
    for _ in range(2):
        x, y = loader.next()
        tr.step(x, y)
    loss = tr.last_loss()
    assert math.isfinite(loss), loss
    assert tr.hook_state.launches > 0
