"""The memory-bound kernels of the training paths on tensors larger than L2: LayerNorm, GELU, fused softmax
cross-entropy, the three-table embedding gather, pooling, the image normalise kernel and the fused optimisers.

    python -m gcow_b200.bench.memops_bench [--iters 10] [--only layernorm]

Each row: device milliseconds (CUDA events, median), the bytes the operation has to move and that figure as a
fraction of the measured copy bandwidth (MEASURED_PEAKS.json). Also the workload for ncu captures of these kernels.
"""
from __future__ import annotations

import argparse
import json

import torch

from gcow_b200.bench.codec_bench import peaks, time_cuda
from gcow_b200.ops import kernels as K
from gcow_b200.ops.optim import FusedAdamW, FusedSGD


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="")
    args = ap.parse_args(argv)
    hbm, how = peaks()
    dev = torch.device("cuda")
    cases = []

    rows, H = 65536, 1024                                            # 4 x BERT-large's token count: 134 MB per tensor
    x = torch.randn(rows, H, device=dev).bfloat16().requires_grad_(True)
    w, b = torch.ones(H, device=dev, requires_grad=True), torch.zeros(H, device=dev, requires_grad=True)
    g = torch.randn(rows, H, device=dev).bfloat16()
    cases.append(("layernorm forward", lambda: K.layernorm(x.detach(), w.detach(), b.detach(), 1e-12), 2 * rows * H * 2))

    def ln_fb():
        x.grad = None
        K.layernorm(x, w, b, 1e-12).backward(g)
    cases.append(("layernorm forward + backward", ln_fb, 6 * rows * H * 2))
    cases.append(("gelu forward", lambda: K.gelu(x.detach()), 2 * rows * H * 2))

    V, R = 30528, 8192                                               # vocabulary logits of 8192 tokens: 500 MB
    logits = torch.randn(R, V, device=dev).bfloat16()
    tgt = torch.randint(0, V, (R,), device=dev)

    def xent():
        lg = logits.clone().requires_grad_(True) * 1.0               # the kernel consumes a non-leaf buffer
        K.softmax_xent(lg, tgt, -100)
    cases.append(("softmax cross-entropy (+ the clone and scale feeding it)", xent, 2 * R * V * 2 + 3 * R * V * 2))

    Bq, S = 128, 512
    tok = torch.randn(30522, H, device=dev, requires_grad=True)
    pos = torch.randn(512, H, device=dev, requires_grad=True)
    typ = torch.randn(2, H, device=dev, requires_grad=True)
    ids = torch.randint(0, 30522, (Bq, S), device=dev)
    tys = torch.zeros_like(ids)
    cases.append(("embedding gather (token + position + type)", lambda: K.embed3(ids, tys, tok.detach(), pos.detach(), typ.detach()),
                  Bq * S * H * (4 + 2)))

    N, C, HW = 256, 64, 112
    a = torch.randn(N, C, HW, HW, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
    cases.append(("maxpool 3x3/2 forward", lambda: K.maxpool3x3s2(a), int(N * C * HW * HW * 2 * 1.25 + N * C * HW * HW // 4)))
    a2 = torch.randn(N, 2048, 7, 7, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
    cases.append(("global average pool forward", lambda: K.global_avgpool(a2), N * 2048 * 49 * 2))
    img = torch.randint(0, 256, (N, 224, 224, 3), dtype=torch.uint8, device=dev)
    cases.append(("uint8 image -> normalised bf16", lambda: K.u8_to_bf16_norm(img, [120.0] * 3, [60.0] * 3), N * 224 * 224 * 3 * 3))

    params = [torch.randn(1 << 24, device=dev, requires_grad=True) for _ in range(4)]      # 64 M parameters
    for p in params:
        p.grad = torch.randn_like(p)
    sgd = FusedSGD(params, lr=0.1, momentum=0.9, weight_decay=1e-4)
    adam = FusedAdamW(params, lr=1e-4)
    n = sum(p.numel() for p in params)
    cases.append(("fused SGD step (momentum)", sgd.step, n * 4 * 5))            # read p, g, m; write p, m
    cases.append(("fused AdamW step", adam.step, n * 4 * 7))                   # read p, g, m, v; write p, m, v

    for name, fn, nbytes in cases:
        if args.only and args.only not in name:
            continue
        ms, _ = time_cuda(fn, args.iters)
        print(json.dumps({"op": name, "ms": round(ms, 4), "gb_moved": round(nbytes / 1e9, 3),
                          "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm": round(nbytes / ms / 1e6 / hbm, 3),
                          "roofline": f"of {how} {hbm:.0f} GB/s copy"}), flush=True)
    K.check_errors()


if __name__ == "__main__":
    main()
