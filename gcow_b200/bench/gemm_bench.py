"""tcgen05 GEMM throughput against torch.matmul (cuBLAS) on the same shapes.

    python -m gcow_b200.bench.gemm_bench [--json out.json]

TFLOP/s = 2*M*N*K / CUDA-event time; the roofline denominator is the measured
cuBLAS bf16 burst figure in MEASURED_PEAKS.json (1.59 PFLOP/s fallback)."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from gcow_b200.ops import kernels as K
from gcow_b200.bench.codec_bench import time_cuda

SHAPES = [  # (M, N, K)  BERT-large tokens x projections, ResNet-50 1x1 convs as GEMMs
    (16384, 3072, 1024), (16384, 1024, 1024), (16384, 4096, 1024), (16384, 1024, 4096), (16384, 30522 // 8 * 8, 1024),
    (8192, 8192, 8192), (200704, 256, 64), (50176, 512, 256), (12544, 2048, 512), (256, 1000, 2048),
]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--layouts", action="store_true", help="also time the MN-major operand layouts of the backward products")
    ap.add_argument("--shape", type=int, nargs=3, default=None, metavar=("M", "N", "K"), help="time one shape only")
    args = ap.parse_args(argv)
    pk = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak, how = (json.loads(pk.read_text()).get("bf16_tflops", 1590.0), "measured") if pk.exists() else (1590.0, "fallback")
    rows = []
    for M, N, Kd in ([tuple(args.shape)] if args.shape else SHAPES):
        a = torch.randn(M, Kd, device="cuda").bfloat16()
        b = torch.randn(N, Kd, device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms_own, _ = time_cuda(lambda: K.gemm_bf16(a, b, out=out), args.iters)
        ms_128, _ = time_cuda(lambda: K.gemm_bf16(a, b, out=out, tile_rows=128), args.iters)
        ms_256, _ = time_cuda(lambda: K.gemm_bf16(a, b, out=out, tile_rows=256), args.iters)
        K.check_errors()
        ms_lib, _ = time_cuda(lambda: torch.matmul(a, b.t(), out=out), args.iters)
        fl = 2.0 * M * N * Kd
        row = {"M": M, "N": N, "K": Kd, "own_ms": ms_own, "tile128_ms": ms_128, "tile256_ms": ms_256, "cublas_ms": ms_lib, "own_tflops": fl / ms_own / 1e9,
               "cublas_tflops": fl / ms_lib / 1e9, "own_frac_of_peak": fl / ms_own / 1e9 / peak,
               "peak": f"{how} {peak:.0f} TFLOP/s"}
        if args.layouts:
            at, bt = a.t().contiguous(), b.t().contiguous()          # [K, M], [K, N]
            for name, (x, y, kw) in {"b_mn": (a, bt, dict(b_t=True)), "a_mn_b_mn": (at, bt, dict(a_t=True, b_t=True))}.items():
                ms, _ = time_cuda(lambda: K.gemm_bf16(x, y, out=out, **kw), args.iters)
                row[f"{name}_ms"], row[f"{name}_tflops"] = ms, fl / ms / 1e9
            K.check_errors()
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.json:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
