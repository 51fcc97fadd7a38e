"""Codec throughput: the sm_100a encode/decode kernels against the HBM copy
roofline, and the reference CPU codec / this library's CPU oracle on the same box.

    python -m gcow_b200.bench.codec_bench [--mb 256] [--rates 4 8 16] [--json out.json]

GB/s is uncompressed fp32 bytes over device time (CUDA events, after warm-up);
the 256 MB input and its output exceed the 126 MB L2, so every iteration streams
from HBM. The reference's own stage probes use a 268.6 MB field
(hw/tests/test_emax.cpp:70)."""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import numpy as np
import torch

import gcow_b200 as g
from gcow_b200.codec import ZfpParams


def time_cuda(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in ev)
    return ts[len(ts) // 2], ts[0]


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()).get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--rates", type=float, nargs="+", default=[4, 8, 16])
    ap.add_argument("--cpu-mb", type=int, default=16)
    ap.add_argument("--json", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU reference / oracle timings")
    args = ap.parse_args(argv)
    res = {"mb": args.mb, "gpu": [], "cpu": []}
    hbm, how = peaks()
    if torch.cuda.is_available():
        n = args.mb * (1 << 20) // 4
        x = torch.randn(n, device="cuda") * 1e-3
        for rate in args.rates:
            p = ZfpParams.from_rate(rate, 1)
            c = g.compress(x, params=p)
            out = torch.empty_like(x)
            med_e, best_e = time_cuda(lambda: g.compress(x, params=p), args.iters)
            med_d, best_d = time_cuda(lambda: g.decompress(c, out=out), args.iters)
            traffic = n * 4 + c.nbytes
            row = {"rate": rate, "enc_ms": med_e, "dec_ms": med_d,
                   "enc_gbs": n * 4 / med_e / 1e6, "dec_gbs": n * 4 / med_d / 1e6,
                   "enc_frac_hbm": traffic / med_e / 1e6 / hbm, "dec_frac_hbm": traffic / med_d / 1e6 / hbm,
                   "roofline": f"of {how} {hbm:.0f} GB/s copy"}
            res["gpu"].append(row)
            print(json.dumps(row), flush=True)
    if torch.cuda.is_available():
        # 2-D (the reference codec's own case): 8192 x 8192 smooth field, fixed rate 8 and tolerance 1e-3
        n2 = 8192
        i = torch.arange(n2, device="cuda", dtype=torch.float32) * (2.0 / n2)
        field = torch.exp(-(i[None, :] ** 2 + i[:, None] ** 2)).contiguous()
        res["gpu_2d"] = []
        for name, kw in (("rate8", dict(rate=8)), ("tol1e-3", dict(tolerance=1e-3))):
            c = g.compress(field, dim=2, return_index=True, **kw)
            out2 = torch.empty_like(field)
            med_e, _ = time_cuda(lambda: g.compress(field, dim=2, **kw), args.iters)
            med_d, _ = time_cuda(lambda: g.decompress(c, out=out2), args.iters)
            row = {"case": "2d " + name, "n": n2, "enc_ms": med_e, "dec_ms": med_d, "enc_gbs": field.numel() * 4 / med_e / 1e6,
                   "dec_gbs": field.numel() * 4 / med_d / 1e6, "bits_per_value": 8.0 * c.nbytes / field.numel()}
            res["gpu_2d"].append(row)
            print(json.dumps(row), flush=True)
    if args.no_cpu:
        return res
    # CPU side: reference sw codec (1 thread) and this library's oracle
    sys.path.insert(0, str(Path(__file__).resolve().parents[2] / "tests"))
    try:
        import refcodec
        have_ref = refcodec.load() is not None
    except Exception:
        have_ref = False
    n = args.cpu_mb * (1 << 20) // 4
    xs = (np.random.default_rng(0).standard_normal(n) * 1e-3).astype(np.float32)
    for rate in args.rates:
        p = ZfpParams.from_rate(rate, 1)
        tup = (p.minbits, p.maxbits, p.maxprec, p.minexp)
        row = {"rate": rate}
        if have_ref:
            t0 = time.perf_counter(); s = refcodec.compress(xs, tup, 1); t1 = time.perf_counter()
            refcodec.decompress(s, xs.shape, tup); t2 = time.perf_counter()
            row["ref_enc_gbs"] = n * 4 / (t1 - t0) / 1e9
            row["ref_dec_gbs"] = n * 4 / (t2 - t1) / 1e9
        xt = torch.from_numpy(xs)
        t0 = time.perf_counter(); c = g.compress(xt, params=p); t1 = time.perf_counter()
        g.decompress(c); t2 = time.perf_counter()
        row["oracle_mt_enc_gbs"] = n * 4 / (t1 - t0) / 1e9
        row["oracle_mt_dec_gbs"] = n * 4 / (t2 - t1) / 1e9
        res["cpu"].append(row)
        print(json.dumps(row), flush=True)
    if have_ref:
        # the reference's own entry point: 2-D zfp_compress, tolerance 1e-3 and fixed rate 8
        n2 = 2048
        ii = np.arange(n2, dtype=np.float64) * 2.0 / n2
        f2 = np.exp(-(ii[None, :] ** 2 + ii[:, None] ** 2)).astype(np.float32)
        for name, p in (("tol1e-3", ZfpParams.from_accuracy(1e-3)), ("rate8", ZfpParams.from_rate(8, 2))):
            tup = (p.minbits, p.maxbits, p.maxprec, p.minexp)
            t0 = time.perf_counter(); s2 = refcodec.compress(f2, tup, 2); t1 = time.perf_counter()
            row = {"case": "2d " + name + " reference zfp_compress", "n": n2, "ref_enc_gbs": f2.size * 4 / (t1 - t0) / 1e9,
                   "bytes": len(s2)}
            res["cpu"].append(row)
            print(json.dumps(row), flush=True)
    if args.json:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
