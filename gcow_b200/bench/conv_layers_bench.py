"""Every convolution of a ResNet, own kernels against cuDNN, layer shape by layer shape.

    python -m gcow_b200.bench.conv_layers_bench [--arch resnet50] [--batch 256] [--json out.json]

The distinct convolution configurations of the model (input channels, output channels, filter, stride,
input extent) are collected with forward hooks on one forward pass; each is then timed as the model runs
it: ``gcow_b200.ops.nn.Conv2d`` forward plus backward through autograd (forward, data gradient and weight
gradient together, including the layout and weight-format kernels the module runs around them; device time, with
the calls enqueued behind a spin kernel so that host latency does not count), once
on the default own routing and once with every convolution sent to cuDNN (``GCOW_CONV=lib``). The
table's last row sums ``count x time`` over the model: the convolution cost of one training step on
either arm. The reference's models call nn.Conv2d at hw/models/resenet.py:11-17,79,113.
"""
from __future__ import annotations

import argparse
import json
import os
from collections import OrderedDict
from pathlib import Path

import torch

from gcow_b200.models import MODELS
from gcow_b200.ops import backend
from gcow_b200.ops import nn as gnn


def time_queued(fn, iters: int, warmup: int = 2) -> float:
    """Device milliseconds per call with the host out of the picture: a spin kernel keeps the GPU busy while all
    ``iters`` calls are enqueued behind it, so the timed region (CUDA events) runs back to back on the device."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(int(6e7))          # about 30 ms at 1.9 GHz: far longer than enqueueing the calls takes
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def collect(arch: str, batch: int, image: int):
    """OrderedDict {(cin, cout, k, stride, pad, h): count} of the model's convolutions."""
    backend.set_backend("torch")
    net = MODELS[arch]().cuda().to(memory_format=torch.channels_last).bfloat16()
    seen: OrderedDict = OrderedDict()
    first = []

    def hook(m, inp, out):
        x = inp[0]
        key = (m.in_channels, m.out_channels, m.kernel_size[0], m.stride[0], m.padding[0], x.shape[2])
        seen[key] = seen.get(key, 0) + 1
        if not first:
            first.append(key)
    hs = [m.register_forward_hook(hook) for m in net.modules() if isinstance(m, gnn.Conv2d)]
    with torch.no_grad():
        net(torch.zeros(min(batch, 2), 3, image, image, device="cuda", dtype=torch.bfloat16)
            .contiguous(memory_format=torch.channels_last))
    for h in hs:
        h.remove()
    return seen, first[0]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="resnet50")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    ap.add_argument("--alt-1x1", action="store_true",
                    help="also time every stride-1 1x1 layer on the path the routing did NOT choose (GEMM or one-tap implicit GEMM)")
    ap.add_argument("--layer", type=int, nargs=5, default=None, metavar=("CI", "CO", "K", "STRIDE", "H"),
                    help="time this one layer shape only (padding K // 2), e.g. for a profiler capture")
    args = ap.parse_args(argv)
    if args.layer:
        ci, co, k, st, h = args.layer
        layers = OrderedDict({(ci, co, k, st, k // 2, h): 1})
        stem = next(iter(layers)) if ci < 8 else None        # an image layer: its input needs no gradient
    else:
        layers, stem = collect(args.arch, args.batch, args.image)
    backend.set_backend("own")
    rows, tot = [], {"own": 0.0, "cudnn": 0.0}
    for (cin, cout, k, s, p, h), count in layers.items():
        conv = gnn.Conv2d(cin, cout, k, stride=s, padding=p, bias=False).cuda().to(memory_format=torch.channels_last)
        x = torch.randn(args.batch, cin, h, h, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
        x.requires_grad_((cin, cout, k, s, p, h) != stem)          # the stem's input needs no gradient
        row = {"cin": cin, "cout": cout, "k": k, "stride": s, "h": h, "count": count}
        gy = None
        arms = [("own", None), ("cudnn", "lib")]
        if args.alt_1x1 and k == 1 and s == 1:
            arms.append(("alt1x1", "auto"))        # forces the other 1x1 path, whatever the pixel count
        for arm, env in arms:
            if env is None:
                os.environ.pop("GCOW_CONV", None)
            else:
                os.environ["GCOW_CONV"] = env
            if arm == "alt1x1":
                os.environ["GCOW_CONV1X1"] = "gemm" if row["own_path"] == "igemm" else "igemm"
            else:
                os.environ.pop("GCOW_CONV1X1", None)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = conv(x)
            if gy is None:
                gy = torch.randn_like(y)
            row[f"{arm}_path"] = gnn.last_conv_path()

            def step():
                conv.weight.grad = None
                x.grad = None
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    out = conv(x)
                out.backward(gy)
            ms = time_queued(step, args.iters)
            row[f"{arm}_ms"] = round(ms, 4)
            if arm in tot:
                tot[arm] += ms * count
        row["own_over_cudnn"] = round(row["own_ms"] / row["cudnn_ms"], 3)
        os.environ.pop("GCOW_CONV", None)
        rows.append(row)
        print(json.dumps(row), flush=True)
    summary = {"arch": args.arch, "batch": args.batch, "convolutions": sum(layers.values()),
               "own_ms_per_step": round(tot["own"], 3), "cudnn_ms_per_step": round(tot["cudnn"], 3)}
    print(json.dumps(summary), flush=True)
    if args.json:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps({"layers": rows, "summary": summary}, indent=1))


if __name__ == "__main__":
    main()
