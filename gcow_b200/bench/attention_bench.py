"""Fused tcgen05 self-attention against PyTorch's scaled_dot_product_attention on the BERT-large shape.

    python -m gcow_b200.bench.attention_bench [--batch 32] [--seq 512] [--heads 16] [--iters 10]

Forward and forward+backward times (CUDA events, median) on packed qkv [B, S, 3, H, 64] in bf16, and the
achieved TFLOP/s counting 4 B H S^2 d flops forward and 10 B H S^2 d backward (the library kernel's count; the
own backward recomputes S and dP in its second kernel, which is not counted).
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.nn.functional as F

from gcow_b200.bench.codec_bench import time_cuda
from gcow_b200.ops import kernels as K


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    B, S, H, D = args.batch, args.seq, args.heads, 64
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    go = torch.randn(B, S, H * D, device="cuda").bfloat16()
    fl_f, fl_b = 4.0 * B * H * S * S * D, 10.0 * B * H * S * S * D

    def own_fwd():
        with torch.no_grad():
            K.fused_attention(qkv)

    def own_fb():
        qkv.grad = None
        K.fused_attention(qkv).backward(go)

    q, k, v = (qkv.detach()[:, :, i].transpose(1, 2).contiguous().requires_grad_(True) for i in range(3))
    go4 = go.view(B, S, H, D).transpose(1, 2)

    def lib_fwd():
        with torch.no_grad():
            F.scaled_dot_product_attention(q, k, v)

    def lib_fb():
        q.grad = k.grad = v.grad = None
        F.scaled_dot_product_attention(q, k, v).backward(go4)

    row = {"B": B, "S": S, "H": H}
    for name, fn, fl in (("own_fwd", own_fwd, fl_f), ("lib_fwd", lib_fwd, fl_f), ("own_fwd_bwd", own_fb, fl_f + fl_b),
                         ("lib_fwd_bwd", lib_fb, fl_f + fl_b)):
        ms, _ = time_cuda(fn, args.iters)
        row[name + "_ms"] = round(ms, 4)
        row[name + "_tflops"] = round(fl / ms / 1e9, 1)
    K.check_errors()
    print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
