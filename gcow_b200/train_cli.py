"""gcow-train: data-parallel training with compressed gradients.

Counterpart of the reference's two study scripts (hw/models/train_imagenet.py and
hw/models/train_resnet_cifar10.py): same optimiser settings, learning-rate
schedules, meters, per-epoch CSV, checkpoint/resume, NaN stop and plateau early
stop, and the same sweep over codec modes x one variable - but the codec runs on
the GPU and, in rate mode, inside the gradient all-reduce itself.

    torchrun --nproc-per-node 8 -m gcow_b200.train_cli --arch resnet50 --dummy --epochs 1 \
        --zfp-mode rate --rates 8 --batch-size 256
    python -m gcow_b200.train_cli --arch resnet50 --cifar --dummy --zfp-mode accuracy --tolerances 1e-3

Codec modes (hw/models/train_imagenet.py:449-475):
  rate       fused compressed all-reduce at `rate` bits/value (compression on the wire)
  accuracy   with --accuracy-cap-rate R (4, 8, 16 or 32): inside the fused all-reduce too - bit planes below the
             tolerance are dropped, a block wholly below it sends nothing, no block exceeds 4R bits (ZFP expert
             mode). Without the cap: every bucket is round-tripped through the uncapped fixed-accuracy codec on the
             GPU and then all-reduced by NCCL in fp32
  precision  fixed-precision codec round trip on the GPU, then NCCL fp32
  lossless   plain NCCL fp32 all-reduce (the control arm)
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

from .config import GcowConfig
from .parallel.ddp import codec_roundtrip_nccl_hook
from .train import Trainer, make_loader
from .utils.checkpoint import load_checkpoint, save_checkpoint
from .utils.logging import AverageMeter, ProgressMeter, accuracy, append_csv


def parse(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(prog="gcow-train", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("data", nargs="?", default="",
                    help="dataset directory: train/ and val/ class folders (as torchvision's ImageFolder reads them), the "
                         "python version of CIFAR-10 with --cifar, or pre-decoded train_x.npy/train_y.npy/val_x.npy/val_y.npy "
                         "(uint8 NHWC)")
    ap.add_argument("-a", "--arch", default="resnet18")
    ap.add_argument("--zfp-mode", default="", choices=["", "precision", "accuracy", "rate", "lossless"])
    ap.add_argument("--rates", type=float, nargs="+", default=[16])
    ap.add_argument("--tolerances", type=float, nargs="+", default=[1e-6])
    ap.add_argument("--accuracy-cap-rate", type=float, default=0,
                    help="accuracy mode on the wire: cap of 4, 8, 16 or 32 bits/value per block (0: codec round trip + NCCL)")
    ap.add_argument("--precisions", type=int, nargs="+", default=[16])
    ap.add_argument("--reversed", action="store_true", help="walk the sweep variables in reverse order")
    ap.add_argument("--epochs", type=int, default=90)
    ap.add_argument("--start-epoch", type=int, default=0)
    ap.add_argument("-b", "--batch-size", type=int, default=128, help="per-GPU batch")
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--momentum", type=float, default=0.9)
    ap.add_argument("--wd", "--weight-decay", type=float, default=1e-4, dest="wd")
    ap.add_argument("-p", "--print-freq", type=int, default=10)
    ap.add_argument("--resume", default="")
    ap.add_argument("-e", "--evaluate", action="store_true")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--dummy", action="store_true", help="synthetic data")
    ap.add_argument("--num-classes", type=int, default=0,
                    help="0: 10 with --cifar, else the number of class folders under DATA/train, else 1000")
    ap.add_argument("--cifar", action="store_true", help="32x32 inputs, 10 classes, ReduceLROnPlateau (the CIFAR-10 study)")
    ap.add_argument("--steps-per-epoch", type=int, default=100, help="with --dummy")
    ap.add_argument("--patience", type=int, default=5, help="epochs without top-1 improvement before stopping")
    ap.add_argument("--out-dir", default="results")
    ap.add_argument("--ops", default="own", choices=["own", "torch"])
    # launch flags of the reference script (hw/models/train_imagenet.py:60-94); torchrun's environment wins when present
    ap.add_argument("-j", "--workers", type=int, default=4, help="data loading worker processes per rank")
    ap.add_argument("--pretrained", action="store_true",
                    help="start from torchvision's weights (they must already be in the local torch hub cache)")
    ap.add_argument("--world-size", type=int, default=-1, help="number of nodes (with --multiprocessing-distributed) or of processes")
    ap.add_argument("--rank", type=int, default=-1, help="node rank (with --multiprocessing-distributed) or process rank")
    ap.add_argument("--dist-url", default="tcp://127.0.0.1:23456", help="rendezvous tcp://host:port when not started by torchrun")
    ap.add_argument("--dist-backend", default="nccl", help="accepted for compatibility: GPUs always use NCCL for the control plane")
    ap.add_argument("--gpu", type=int, default=None, help="GPU of this process when not started by torchrun")
    ap.add_argument("--multiprocessing-distributed", action="store_true",
                    help="start one process per visible GPU from this one (what torchrun does otherwise)")
    GcowConfig.add_cli(ap)
    return ap.parse_args(argv)


class FileLoader:
    """uint8 NHWC images + int64 labels from .npy files, sharded by rank, pinned batches."""

    def __init__(self, xpath, ypath, batch, rank, world, shuffle, seed):
        import numpy as np
        self.x = torch.from_numpy(np.load(xpath, mmap_mode="r")[rank::world].copy())
        self.y = torch.from_numpy(np.load(ypath)[rank::world].astype("int64"))
        self.batch, self.shuffle, self.gen = batch, shuffle, torch.Generator().manual_seed(seed + rank)
        self.classes = int(self.y.max()) + 1

    def __len__(self):
        return len(self.y) // self.batch

    def __iter__(self):
        idx = torch.randperm(len(self.y), generator=self.gen) if self.shuffle else torch.arange(len(self.y))
        for i in range(len(self)):
            sel = idx[i * self.batch:(i + 1) * self.batch]
            yield self.x[sel].pin_memory(), self.y[sel].pin_memory()


class DummyLoader:
    def __init__(self, kind, batch, steps, image, classes, seed):
        self.src, self.steps = make_loader(kind, batch, image=image, classes=classes, seed=seed), steps

    def __len__(self):
        return self.steps

    def __iter__(self):
        for _ in range(self.steps):
            yield self.src.next()


def validate(tr: Trainer, loader, print_freq: int):
    top1, top5, losses = AverageMeter("Acc@1", ":6.2f"), AverageMeter("Acc@5", ":6.2f"), AverageMeter("Loss", ":.4e")
    tr.ddp.eval()
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for i, (x, y) in enumerate(loader):
            x, y = x.to(tr.device, non_blocking=True), y.to(tr.device, non_blocking=True)
            out = tr.ddp.module(tr.preprocess(x)).float()
            loss = torch.nn.functional.cross_entropy(out, y)
            a1, a5 = accuracy(out, y, topk=(1, min(5, out.shape[1])))
            losses.update(loss.item(), y.numel()); top1.update(a1.item(), y.numel()); top5.update(a5.item(), y.numel())
    for m in (top1, top5, losses):
        m.all_reduce(tr.device)
    tr.ddp.train()
    if tr.device.type == "cuda":
        from .ops import kernels
        kernels.check_errors(tr.device)              # a tensor-core kernel that gave up would have skewed the metrics
    return top1.avg, top5.avg, losses.avg


def run_one(args, mode: str, variable) -> dict:
    rank = int(os.environ.get("RANK", 0))
    cfg_over = dict(rate=float(variable) if mode == "rate" else None)
    cfg = GcowConfig.from_cli(args)
    wire_accuracy = mode == "accuracy" and args.accuracy_cap_rate > 0
    if mode == "rate":
        cfg.mode, cfg.rate = "rate", float(variable)
    elif wire_accuracy:      # fixed accuracy inside the all-reduce: planes below the tolerance dropped, blocks capped
        cfg.mode, cfg.tolerance, cfg.rate = "accuracy", float(variable), float(args.accuracy_cap_rate)
    else:
        cfg.variant = "nccl"                     # DDP's own NCCL path; a hook is added below for the lossy modes
    classes = args.num_classes or (10 if args.cifar else 1000)
    if not args.num_classes and not args.cifar and args.data and os.path.isdir(os.path.join(args.data, "train")):
        classes = sum(e.is_dir() for e in os.scandir(os.path.join(args.data, "train"))) or classes
    image = 32 if args.cifar else 224
    tr = Trainer(args.arch, batch_size=args.batch_size, cfg=cfg, ops=args.ops, lr=args.lr, num_classes=classes,
                 seed=args.seed, model_kwargs={"small_input": True} if args.cifar else None, pretrained=args.pretrained,
                 track_accuracy=True)
    if tr.hook_state is not None:
        tr.hook_state.timing = True
    for g in tr.opt.param_groups:
        g["momentum"], g["weight_decay"] = args.momentum, args.wd
    hook_state = None
    if mode in ("accuracy", "precision") and not wire_accuracy:
        from .codec import ZfpParams
        p = ZfpParams.from_accuracy(float(variable)) if mode == "accuracy" else ZfpParams.from_precision(int(variable))
        hook_state = {"params": p, "bytes_in": 0, "bytes_out": 0}
        tr.ddp.register_comm_hook(hook_state, codec_roundtrip_nccl_hook)
    if args.cifar:
        sched = torch.optim.lr_scheduler.ReduceLROnPlateau(tr.opt, factor=0.1, patience=5)   # train_resnet_cifar10.py:159
    else:
        sched = tr.sched                                                                      # StepLR(30, 0.1)
    if args.dummy or not args.data:
        train_loader = DummyLoader(tr.kind, args.batch_size, args.steps_per_epoch, image, classes, args.seed + tr.rank)
        val_loader = DummyLoader(tr.kind, args.batch_size, max(1, args.steps_per_epoch // 10), image, classes, 10_000 + tr.rank)
    elif os.path.exists(os.path.join(args.data, "train_x.npy")):
        train_loader = FileLoader(os.path.join(args.data, "train_x.npy"), os.path.join(args.data, "train_y.npy"),
                                  args.batch_size, tr.rank, tr.world, True, args.seed)
        val_loader = FileLoader(os.path.join(args.data, "val_x.npy"), os.path.join(args.data, "val_y.npy"),
                                args.batch_size, tr.rank, tr.world, False, args.seed)
    else:               # image folders / CIFAR-10 batches, decoded and augmented by worker processes
        from .data import make_loaders
        train_loader, val_loader = make_loaders(args.data, args.cifar, args.batch_size, tr.rank, tr.world, args.workers,
                                                args.seed, image)
    tag = f"{args.arch}_{mode}_{variable}"
    ckpt = os.path.join(args.out_dir, "models", tag + "_ckp.tar")
    best_acc1, start_epoch, stale = 0.0, args.start_epoch, 0
    if args.resume and os.path.isfile(args.resume):
        sd = load_checkpoint(args.resume, map_location=f"cuda:{tr.device.index}")
        tr.load_state_dict(sd["trainer"])
        start_epoch, best_acc1 = sd["epoch"], sd.get("best_acc1", 0.0)
        if rank == 0:
            print(f"=> resumed '{args.resume}' (epoch {start_epoch})")
    if args.evaluate:
        a1, a5, vl = validate(tr, val_loader, args.print_freq)
        return {"mode": mode, "variable": variable, "acc1": a1, "acc5": a5, "val_loss": vl}
    result = {"mode": mode, "variable": variable, "diverged": False}
    for epoch in range(start_epoch, args.epochs):
        batch_time, data_time = AverageMeter("Time", ":6.3f"), AverageMeter("Data", ":6.3f")
        losses, top1, top5 = AverageMeter("Loss", ":.4e"), AverageMeter("Acc@1", ":6.2f"), AverageMeter("Acc@5", ":6.2f")
        prog = ProgressMeter(len(train_loader), [batch_time, data_time, losses, top1, top5], prefix=f"Epoch: [{epoch}]")
        t_epoch = end = time.time()
        try:
            for i, (x, y) in enumerate(train_loader):
                data_time.update(time.time() - end)
                r = tr.step(x, y)
                if r.loss is not None:
                    losses.update(r.loss, args.batch_size)
                if r.acc1 is not None:
                    top1.update(r.acc1, args.batch_size)
                    top5.update(r.acc5, args.batch_size)
                batch_time.update(time.time() - end)
                end = time.time()
                if rank == 0 and i % args.print_freq == 0:
                    prog.display(i + 1)
        except FloatingPointError:                   # NaN loss: stop this sweep point (train_imagenet.py:445-446)
            result["diverged"] = True
            break
        a1, a5, vl = validate(tr, val_loader, args.print_freq)
        if args.cifar:
            sched.step(vl)
        elif sched is not None:
            sched.step()
        tr.epoch = epoch + 1
        is_best = a1 > best_acc1
        best_acc1 = max(a1, best_acc1)
        stale = 0 if is_best else stale + 1
        save_checkpoint({"epoch": epoch + 1, "arch": args.arch, "best_acc1": best_acc1, "trainer": tr.state_dict()},
                        ckpt, is_best)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()      # rank 0 writes alone; the others must not start waiting on it inside a collective
        secs = time.time() - t_epoch
        # device seconds of this epoch: batch copies (the reference's "transfer" time, hw/models/train_imagenet.py:452-473),
        # the compressed collectives (codec and wire are one kernel in rate mode) and the stand-alone codec (other modes)
        h2d_sec = tr.h2d_seconds()
        comm_sec = tr.hook_state.comm_seconds() if tr.hook_state else 0.0
        codec_sec = 0.0
        if hook_state and hook_state.get("codec_events"):
            torch.cuda.synchronize()
            codec_sec = sum(a.elapsed_time(b) for a, b in hook_state["codec_events"]) / 1e3
            hook_state["codec_events"].clear()
        row = {"mode": mode, "variable": variable, "epoch": epoch, "train_loss": losses.avg, "train_acc1": top1.avg,
               "train_acc5": top5.avg, "val_loss": vl, "acc1": a1, "acc5": a5, "epoch_sec": secs,
               "h2d_sec": h2d_sec, "allreduce_sec": comm_sec, "codec_sec": codec_sec,
               "samples_per_sec": len(train_loader) * args.batch_size * tr.world / secs,
               "wire_ratio": tr.hook_state.ar.wire_ratio() if tr.hook_state else 0.0,
               "codec_ratio": (hook_state["bytes_in"] / max(1, hook_state["bytes_out"])) if hook_state else 0.0}
        if rank == 0:
            append_csv(os.path.join(args.out_dir, f"{args.arch}.csv"), row)
            print(row, flush=True)
        result.update(row)
        if stale > args.patience:                    # plateau early stop (train_imagenet.py:354-358)
            break
    return result


def launch_env(args, ngpus: int, local: int = 0) -> dict:
    """RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* for a process that torchrun did not start, from the reference's
    launch flags: with --multiprocessing-distributed, --world-size counts nodes and every node runs one process per
    GPU (hw/models/train_imagenet.py:139-147); otherwise it counts processes and --rank is this process's rank."""
    host, _, port = args.dist_url.replace("tcp://", "").partition(":")
    nodes_or_procs = max(1, args.world_size)
    node_or_rank = max(0, args.rank)
    if args.multiprocessing_distributed:
        world, rank = nodes_or_procs * ngpus, node_or_rank * ngpus + local
    else:
        world, rank = nodes_or_procs, node_or_rank
        local = args.gpu if args.gpu is not None else 0
    return {"RANK": str(rank), "LOCAL_RANK": str(local), "WORLD_SIZE": str(world),
            "MASTER_ADDR": host or "127.0.0.1", "MASTER_PORT": port or "23456"}


def _spawned(local: int, ngpus: int, argv) -> None:
    args = parse(argv)
    os.environ.update(launch_env(args, ngpus, local))
    _run(args)


def main(argv=None) -> int:
    args = parse(argv)
    if "RANK" not in os.environ:                  # not under torchrun: honour the reference's launch flags
        ngpus = max(1, torch.cuda.device_count())
        if args.multiprocessing_distributed and ngpus > 1:
            import torch.multiprocessing as mp
            mp.spawn(_spawned, nprocs=ngpus, args=(ngpus, list(argv) if argv is not None else sys.argv[1:]))
            return 0
        if args.world_size > 1 or args.gpu is not None:
            os.environ.update(launch_env(args, ngpus))
    return _run(args)


def _run(args) -> int:
    modes = ["precision", "accuracy", "rate", "lossless"] if not args.zfp_mode else [args.zfp_mode]
    for mode in modes:
        variables = {"rate": args.rates, "accuracy": args.tolerances, "precision": args.precisions, "lossless": [0]}[mode]
        if args.reversed:
            variables = list(reversed(variables))
        for v in variables:
            if int(os.environ.get("RANK", 0)) == 0:
                print(f"\nRunning zfp_mode={mode}, variable={v}", flush=True)
            res = run_one(args, mode, v)
            if int(os.environ.get("RANK", 0)) == 0:
                print(res, flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
