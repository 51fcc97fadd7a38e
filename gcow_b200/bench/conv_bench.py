"""Implicit-GEMM convolution (tcgen05) against cuDNN on the stride-1 3x3 layers of ResNet-50.

    python -m gcow_b200.bench.conv_bench [--batch 256] [--json out.json]

Times forward, data gradient and weight gradient separately with CUDA events; TFLOP/s =
2 * N*H*W * 9*Ci*Co / time. The cuDNN arm is torch's convolution on the same bf16
channels-last tensors (aten.convolution_backward with one output selected at a time)."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch
import torch.nn.functional as F

from gcow_b200 import _native
from gcow_b200.bench.codec_bench import time_cuda

LAYERS = [(64, 56), (128, 28), (256, 14), (512, 7)]     # (channels, spatial extent)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    ap.add_argument("--channels", type=int, default=0, help="time only the layer with this channel count")
    args = ap.parse_args(argv)
    lib = _native.cuda()
    st = torch.cuda.current_stream().cuda_stream
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = []
    for C, HW in LAYERS:
        if args.channels and C != args.channels:
            continue
        N = args.batch
        x = torch.randn(N, C, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
        w = (torch.randn(C, C, 3, 3, device="cuda") * 0.05).bfloat16().contiguous(memory_format=torch.channels_last)
        gy = torch.randn(N, C, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
        wr = w.permute(0, 2, 3, 1).contiguous()
        wt = torch.empty_like(wr)
        lib.gcow_conv_flip_weights(wr.data_ptr(), wt.data_ptr(), C, 3, 3, C, st)
        y = torch.empty_like(x)
        split = lib.gcow_conv_wgrad_split(N, HW, HW, C, C, 3, 3, 1, 1)
        part = torch.empty(split, C, 9 * C, device="cuda")
        dw = torch.empty(C, 9 * C, device="cuda")

        def own_fwd():
            lib.gcow_conv_fwd(x.data_ptr(), wr.data_ptr(), y.data_ptr(), None, N, HW, HW, C, C, 3, 3, 1, 1, err.data_ptr(), st)

        def own_dgrad():
            lib.gcow_conv_fwd(gy.data_ptr(), wt.data_ptr(), y.data_ptr(), None, N, HW, HW, C, C, 3, 3, 1, 1, err.data_ptr(), st)

        def own_wgrad():
            lib.gcow_conv_wgrad(gy.data_ptr(), x.data_ptr(), part.data_ptr(), N, HW, HW, C, C, 3, 3, 1, 1, err.data_ptr(), st)
            lib.gcow_reduce_partials(part.data_ptr(), dw.data_ptr(), split, dw.numel(), st)

        def lib_bwd(mask):
            return lambda: torch.ops.aten.convolution_backward(gy, x, w, None, (1, 1), (1, 1), (1, 1), False, (0, 0), 1, mask)

        fl = 2.0 * N * HW * HW * 9 * C * C
        row = {"N": N, "C": C, "HW": HW, "wgrad_split": split}
        for name, own, ref in (("fwd", own_fwd, lambda: F.conv2d(x, w, padding=1)),
                               ("dgrad", own_dgrad, lib_bwd((True, False, False))),
                               ("wgrad", own_wgrad, lib_bwd((False, True, False)))):
            ms_own, _ = time_cuda(own, args.iters)
            ms_lib, _ = time_cuda(ref, args.iters)
            row[f"{name}_own_ms"], row[f"{name}_cudnn_ms"] = round(ms_own, 4), round(ms_lib, 4)
            row[f"{name}_own_tflops"], row[f"{name}_cudnn_tflops"] = round(fl / ms_own / 1e9, 1), round(fl / ms_lib / 1e9, 1)
        assert int(err.item()) == 0, "a device-side wait gave up"
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.json:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
