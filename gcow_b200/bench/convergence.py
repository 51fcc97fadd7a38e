"""Does training survive the compression? Loss curves of the same model, data and seed at several rates.

    torchrun --nproc-per-node 2 -m gcow_b200.bench.convergence [--steps 300] [--rates 4 8 16] [--json out.json]

The question the reference's two study scripts exist to answer (sweeps over rates and tolerances,
hw/models/train_resnet_cifar10.py:38-42,190-217; hw/models/train_imagenet.py:154-155,372-393), asked here of the
on-the-wire path: ResNet-18 on a learnable synthetic 100-class task (class patterns plus heavy pixel noise), the same
initial weights and sample stream in every arm; the lossless arm is the NCCL fp32 all-reduce, the others the fused
compressed all-reduce at the given bits per value. Prints one JSON line per arm with the mean loss of every
window of 25 steps and the training accuracy of the last window.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from gcow_b200.config import GcowConfig
from gcow_b200.train import LearnableImages, Trainer


def run_arm(name: str, cfg: GcowConfig, args, device) -> dict:
    tr = Trainer(args.arch, batch_size=args.batch, cfg=cfg, lr=args.lr, num_classes=args.classes, device=device, seed=0,
                 track_accuracy=True)
    data = LearnableImages(args.batch, args.image, args.classes, seed=100 + tr.rank, noise=args.noise)
    losses, accs = [], []
    nxt = data.next()
    diverged = 0
    for _ in range(args.steps + 1):
        cur, nxt = nxt, data.next()
        try:
            r = tr.step(cur[0], cur[1], prefetch=nxt)
        except FloatingPointError:          # NaN loss: this arm has diverged; the sweep goes on (train_imagenet.py:445-446)
            diverged = 1
            break
        if r.loss is not None:
            losses.append(r.loss)
            accs.append(r.acc1)
    flag = torch.tensor([diverged], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if int(flag):
        del tr
        torch.cuda.empty_cache()
        return {"arm": name, "diverged": True, "steps": len(losses)}
    t = torch.tensor(losses, device=device, dtype=torch.float64)
    a = torch.tensor(accs, device=device, dtype=torch.float64)
    dist.all_reduce(t)
    dist.all_reduce(a)
    t, a = (t / tr.world).cpu(), (a / tr.world).cpu()
    w = args.window
    wins = [float(t[i:i + w].mean()) for i in range(0, len(t) - w + 1, w)]
    out = {"arm": name, "world": tr.world, "steps": len(t), "window": w, "loss_windows": [round(v, 4) for v in wins],
           "final_loss": wins[-1], "final_acc1": float(a[-w:].mean()),
           "wire_ratio": tr.hook_state.ar.wire_ratio() if tr.hook_state else 1.0}
    del tr
    torch.cuda.empty_cache()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="resnet18")
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--image", type=int, default=64)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--classes", type=int, default=100)
    ap.add_argument("--noise", type=float, default=96.0, help="standard deviation of the pixel noise (patterns span 48..208)")
    ap.add_argument("--window", type=int, default=25)
    ap.add_argument("--rates", type=float, nargs="+", default=[16, 8, 4])
    ap.add_argument("--error-feedback-rates", type=float, nargs="*", default=[8])
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    rows = [run_arm("lossless (NCCL fp32)", GcowConfig(variant="nccl"), args, device)]
    for r in args.rates:
        rows.append(run_arm(f"rate {r:g}", GcowConfig(rate=r, comm_ctas=32, bucket_mb=4), args, device))
    for r in args.error_feedback_rates:
        rows.append(run_arm(f"rate {r:g} + error feedback", GcowConfig(rate=r, comm_ctas=32, bucket_mb=4, error_feedback=True),
                            args, device))
    if dist.get_rank() == 0:
        for row in rows:
            print(json.dumps(row), flush=True)
        if args.json:
            Path(args.json).parent.mkdir(parents=True, exist_ok=True)
            Path(args.json).write_text(json.dumps(rows, indent=1))
    dist.barrier()
    dist.destroy_process_group()
    return rows


if __name__ == "__main__":
    main()
