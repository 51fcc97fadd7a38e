"""Fused BatchNorm(+add)+ReLU kernels against the PyTorch operators on ResNet-50 shapes.

    python -m gcow_b200.bench.bn_bench [--json out.json] [--shape N C HW]

Forward+backward of relu(bn(x) + residual) on channels-last bf16 tensors, CUDA-event
timed. The roofline is the algorithmic traffic (forward: read x twice, read residual,
write y; backward: read dy, y, x, write dres, then read dres, x, write dx) over the
measured copy bandwidth in MEASURED_PEAKS.json."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from gcow_b200.ops import nn as gnn, set_backend
from gcow_b200.bench.codec_bench import time_cuda, peaks

SHAPES = [(256, 64, 112), (256, 256, 56), (256, 512, 28), (256, 1024, 14), (256, 2048, 7)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shape", type=int, nargs=3, default=None, metavar=("N", "C", "HW"))
    args = ap.parse_args(argv)
    hbm, how = peaks()
    rows = []
    for N, C, hw in ([tuple(args.shape)] if args.shape else SHAPES):
        x = torch.randn(N, C, hw, hw, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
        r = torch.randn(N, C, hw, hw, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
        g = torch.randn(N, C, hw, hw, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
        res = {}
        for be in ("own", "torch"):
            set_backend(be)
            bn = gnn.BatchNorm2d(C).cuda()

            def step():
                x.grad = r.grad = None
                bn(x, residual=r, relu=True).backward(g)
            res[be], _ = time_cuda(step, args.iters)
        set_backend("own")
        elems = N * C * hw * hw
        traffic = elems * 2 * (4 + 4 + 3)          # bf16: fwd 3R+1W, bwd sweep 1 3R+1W, sweep 2 2R+1W
        row = {"N": N, "C": C, "HW": hw, "own_ms": res["own"], "torch_ms": res["torch"], "speedup": res["torch"] / res["own"],
               "own_gbs": traffic / res["own"] / 1e6, "frac_hbm": traffic / res["own"] / 1e6 / hbm,
               "roofline": f"of {how} {hbm:.0f} GB/s copy"}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.json:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
