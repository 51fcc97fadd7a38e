"""gcow-codec: generate or load a float32 field, compress it, time it, dump the stream,
and compare with a golden file - the GPU counterpart of the reference's host program
``gcow_host <xclbin> <n>`` (hw/src/host.cpp:13-198: n x n field exp(-(x^2+y^2)),
run the kernel, print milliseconds and values per second, write ``.gcow``, diff
against the ``.zfp`` golden).

    python -m gcow_b200.cli 510 --tolerance 1e-3 --golden path/compressed_2d_510.zfp
    python -m gcow_b200.cli 4096 --rate 8 --dim 2 --out field.gcow --device cuda
    python -m gcow_b200.cli --input grad.npy --dim 1 --rate 8 --roundtrip
    python -m gcow_b200.cli --input AEROD_v_1_1800_3600.dat --shape 1800 3600 --print 4     # a raw float32 field

The last form is the counterpart of the reference's data probe (hw/tests/parse_dat.cpp:1-38), which reads a raw
1800 x 3600 float field and prints a few values.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time

import numpy as np
import torch

import gcow_b200 as g


def reference_field(n: int) -> np.ndarray:
    """exp(-(x^2+y^2)) sampled at x = 2i/n, y = 2j/n (hw/src/host.cpp:201-212)."""
    i = np.arange(n, dtype=np.float64) * 2.0 / n
    return np.exp(-(i[None, :] ** 2 + i[:, None] ** 2)).astype(np.float32)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gcow-codec", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("n", nargs="?", type=int, default=0, help="side of the generated n x n field")
    ap.add_argument("--input", default="", help=".npy file, or with --shape a raw float32 file, to compress instead of the generated field")
    ap.add_argument("--shape", type=int, nargs="+", default=None, metavar="N",
                    help="rows [columns] of a raw little-endian float32 --input file (no header)")
    ap.add_argument("--dim", type=int, default=2, choices=[1, 2])
    m = ap.add_mutually_exclusive_group()
    m.add_argument("--rate", type=float)
    m.add_argument("--tolerance", type=float)
    m.add_argument("--precision", type=int)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="", help="write the compressed stream here (.gcow)")
    ap.add_argument("--golden", default="", help="compare the stream byte for byte with this file")
    ap.add_argument("--roundtrip", action="store_true", help="decompress and report the error")
    ap.add_argument("--pad64", action="store_true", help="pad the stream to 64-byte words like the FPGA build (hw/include/types.hpp:80)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--print", type=int, default=0, metavar="K", dest="show",
                    help="print the top-left K x K corner of the field and the first K stream words "
                         "(the reference's print_2d debugging aid, sw/include/common.hpp:1-21)")
    args = ap.parse_args(argv)
    if not (args.rate or args.tolerance or args.precision):
        args.tolerance = 1e-3                      # the reference kernel's hard-wired setting (hw/src/gcow.cpp:44-45)
    if args.input and args.shape:
        arr = np.fromfile(args.input, dtype="<f4")
        want = int(np.prod(args.shape))
        if arr.size < want:
            ap.error(f"{args.input} holds {arr.size} float32 values, --shape asks for {want}")
        arr = arr[:want].reshape(args.shape)
    elif args.input:
        arr = np.load(args.input).astype(np.float32)
    elif args.n > 0:
        arr = reference_field(args.n)
    else:
        ap.error("give a field size n or --input")
    if args.dim == 1:
        arr = arr.reshape(-1)
    x = torch.from_numpy(np.ascontiguousarray(arr)).to(args.device)
    kw = dict(rate=args.rate, tolerance=args.tolerance, precision=args.precision, dim=args.dim)

    def sync():
        if x.is_cuda:
            torch.cuda.synchronize()

    c = g.compress(x, **kw)                        # warm-up (table upload, allocations)
    sync()
    t0 = time.perf_counter()
    for _ in range(args.iters):
        c = g.compress(x, **kw)
    sync()
    dt = (time.perf_counter() - t0) / args.iters
    stream = c.stream.cpu().numpy().tobytes()
    if args.pad64 and len(stream) % 64:
        stream += bytes(64 - len(stream) % 64)
    rep = {"values": int(x.numel()), "device": args.device, "ms": dt * 1e3, "values_per_second": x.numel() / dt,
           "input_gbs": x.numel() * 4 / dt / 1e9, "compressed_bytes": len(stream),
           "bits_per_value": 8.0 * len(stream) / max(1, x.numel())}
    if args.roundtrip:
        y = g.decompress(c).cpu().numpy()
        err = np.abs(y.astype(np.float64) - arr.astype(np.float64))
        rep["max_abs_error"] = float(err.max())
        rep["rmse"] = float(math.sqrt((err ** 2).mean()))
    if args.out:
        with open(args.out, "wb") as f:
            f.write(stream)
    if args.show > 0:
        k = args.show
        corner = arr[:k, :k] if arr.ndim == 2 else arr[:k * k].reshape(-1, k)
        for row in corner:
            print(" ".join(f"{v: .6e}" for v in row))
        words = np.frombuffer(stream[:8 * k], dtype="<u8")
        print(" ".join(f"{int(w):016x}" for w in words))
    rc = 0
    if args.golden:
        gold = open(args.golden, "rb").read()
        rep["golden_match"] = gold == stream
        rc = 0 if rep["golden_match"] else 1
    print(json.dumps(rep))
    return rc


if __name__ == "__main__":
    sys.exit(main())
