"""Headline benchmark: ResNet-50 data-parallel training with compressed gradients.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                      (the reference arm)

Config (weak scaling): ResNet-50, batch 256 per GPU, 224x224x3 synthetic images,
1000 classes, random init, bf16 autocast with fp32 gradients, 25 MB DDP buckets,
every bucket all-reduced by the fused compressed kernel at 8 bits/value, fused
SGD. ``value`` is total images/s over all GPUs for K steps with device-resident
inputs (CUDA events, max over ranks); ``e2e`` is the same K steps through
``Trainer.step`` with each step's uint8 batch copied from pinned host memory and
the loss read back. Inputs plus activations exceed the 126 MB L2 by far, so no
L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

METRIC = "train samples/s (ResNet-50 DDP, compressed gradient all-reduce at 8 bit/value)"


def reference_arm(args) -> int:
    """The reference ships no installable package (pip: "neither setup.py nor
    pyproject.toml") and its training scripts import zfpy, which this image does
    not have, so its own training loop cannot run here."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference has no setup.py/pyproject.toml to install and hw/models/train_imagenet.py "
                      "imports zfpy, which is not in this image; only its sw/ CPU codec builds "
                      "(baseline/build_ref.sh) and that is measured by gcow_b200.bench.codec_bench"}))
    return 0


def timed_steps(fn, steps: int):
    """K calls of fn bracketed by barrier + synchronize; device time via CUDA events, max over ranks."""
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    dist.barrier()
    ms = torch.tensor([a.elapsed_time(b), wall * 1e3], device="cuda", dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms[0]), float(ms[1])


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="gcow", choices=["gcow", "reference", "nccl"])
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    ap.add_argument("--rate", type=float, default=8.0)
    ap.add_argument("--ops", default="own", choices=["own", "torch"])
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--comm-ctas", type=int, default=0,
                    help="CTAs of the fused all-reduce (0: 148 for ResNet, 296 for BERT, whose 1.3 GB of gradients per step "
                         "make the collective itself worth more SM time)")
    ap.add_argument("--seq-len", type=int, default=512)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    if args.gpus > 1 and "RANK" not in os.environ:
        # convenience: re-launch under torchrun
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", __file__] + sys.argv[1:]
        return subprocess.call(cmd)

    from gcow_b200.config import GcowConfig
    from gcow_b200.train import Trainer, make_loader
    from gcow_b200.utils.tracing import ClockSampler

    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    variant = "nccl" if args.impl == "nccl" else args.variant
    comm_ctas = args.comm_ctas or (296 if args.model.startswith("bert") else 148)
    cfg = GcowConfig.from_env(rate=args.rate, variant=variant, comm_ctas=comm_ctas, timeout_ms=20000)
    tr = Trainer(args.model, batch_size=args.batch, cfg=cfg, ops=args.ops if args.impl != "nccl" else "torch",
                 seq_len=args.seq_len, device=device)
    rank, world = tr.rank, tr.world
    loader = make_loader(tr.kind, args.batch, args.seq_len, seed=rank)

    # device-resident copies of the pool for the kernel-only loop
    pool = []
    for _ in range(4):
        inp, tgt = loader.next()
        if tr.kind == "resnet":
            pool.append((inp.to(device), tgt.to(device)))
        else:
            pool.append(tuple(t.to(device) for t in inp))
    it = {"i": 0}

    def dev_step():
        tr.step_device(pool[it["i"] % len(pool)])
        it["i"] += 1

    nxt = {"b": loader.next()}

    def e2e_step():
        # this step's batch was staged by the previous call; the next one is copied while this step computes
        cur, nxt["b"] = nxt["b"], loader.next()
        tr.step(cur[0], cur[1], prefetch=nxt["b"])

    for _ in range(args.warmup):
        dev_step()
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()

    sampler = ClockSampler(local).start() if rank == 0 else None
    l0 = tr.gpu_launches()
    dev_ms, _ = timed_steps(dev_step, args.steps)
    launches = tr.gpu_launches() - l0
    h0, d0 = tr.h2d_bytes, tr.d2h_bytes
    e2e_ms, e2e_wall = timed_steps(e2e_step, args.steps)
    h2d = (tr.h2d_bytes - h0) // args.steps
    d2h = (tr.d2h_bytes - d0) // args.steps
    clocks = sampler.stop() if sampler else None
    final_loss = tr.last_loss()

    if rank == 0:
        total = args.batch * world
        unit = "images/s" if tr.kind == "resnet" else "sequences/s"
        out = {
            "metric": METRIC if args.model == "resnet50" else f"train samples/s ({args.model})",
            "value": total * args.steps / (dev_ms / 1e3), "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random uint8 images / labels, random-init weights)",
            "impl": args.impl,
            "config": {"model": args.model, "global_batch": total, "per_gpu_batch": args.batch,
                       "seq_len": args.seq_len if tr.kind == "bert" else None, "image": 224,
                       "parallelism": f"dp{world}", "bucket_mb": cfg.bucket_mb, "rate_bits_per_value": args.rate,
                       "variant": cfg.variant, "ops": args.ops, "comm_ctas": tr.hook_state.ar.ctas if tr.hook_state else 0,
                       "l2": "inputs+activations larger than L2, no flush"},
            "e2e": {"value": total * args.steps / (e2e_ms / 1e3), "unit": unit, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "final_loss": final_loss,
        }
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
