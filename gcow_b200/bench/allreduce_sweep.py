"""All-reduce sweep: fused compressed variants against NCCL fp32 and the roofline.

    torchrun --nproc-per-node N -m gcow_b200.bench.allreduce_sweep \
        [--sizes-kb 1 ... 1048576] [--rates 4 8 16] [--json out.json]

For each message size x rate x variant the kernel is timed on the device (CUDA
events around `iters` back-to-back calls on the launching stream, after warm-up)
and the MAX over ranks is reported. Effective GB/s = fp32 message bytes / time.
Roofline per call = the slower of (a) codec HBM traffic at the measured copy
bandwidth and (b) compressed bytes leaving one GPU at the measured 770 GB/s
per-direction NVLink peer bandwidth; `frac` = roofline time / measured time.
Messages rotate through a pool larger than L2 (126 MB) when they are small.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from gcow_b200.comm import CompressedAllReduce
from gcow_b200.config import GcowConfig

NVLINK_GBS = 770.0   # peer copy per direction per GPU as measured on this pool; --peer-copy re-measures it (row "peer_copy")


def peer_copy_gbs(dev, rank, P, nbytes=1 << 30, iters=5):
    """One-directional peer copy bandwidth: every rank copies `nbytes` from its right neighbour's symmetric buffer
    into local memory (plain device-to-device copy over NVLink), device-timed, minimum over ranks."""
    import torch.distributed._symmetric_memory as symm
    t = symm.empty(nbytes, dtype=torch.uint8, device=dev)
    hdl = symm.rendezvous(t, dist.group.WORLD)
    src = hdl.get_buffer((rank + 1) % P, (nbytes,), torch.uint8)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    ms = time_calls(lambda: dst.copy_(src), iters)       # time_calls takes the MAX time over ranks
    return nbytes / ms / 1e6


def hbm_gbs():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()).get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


def time_calls(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def roofline_ms(nbytes, rate, P, variant, hbm):
    comp = nbytes * rate / 32.0
    if variant == "oneshot":
        link = comp * (P - 1)
        mem = nbytes + comp * P + comp * P + nbytes          # read in, write P copies, read P copies, write out
    else:
        link = 2.0 * comp * (P - 1) / P
        mem = nbytes + comp + comp + comp / P * P + comp + nbytes   # enc(read fp32, write comp), reduce(read P/P.., write), decode
    return max(link / (NVLINK_GBS * 1e6), mem / (hbm * 1e6)) if P > 1 else mem / (hbm * 1e6)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-kb", type=int, nargs="+",
                    default=[1, 16, 256, 1024, 4096, 25600, 65536, 262144, 1048576])
    ap.add_argument("--rates", type=float, nargs="+", default=[2, 4, 8, 16],
                    help="bits per value; 2 is floored to the 9-bit block header, decodes to zeros and moves no data")
    ap.add_argument("--variants", nargs="+", default=["twoshot", "oneshot", "nvls"])
    ap.add_argument("--ctas", type=int, default=0, help="0 = as many as are co-resident")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    ap.add_argument("--accuracy", nargs="*", default=["1e-3:8", "1e-2:8", "1e-3:8:0.5"],
                    help="fixed-accuracy rows as tolerance:cap[:fraction] (cap in bits/value; `fraction` of the buffer, "
                         "its tail, is scaled to 1e-8, far below the tolerance); the wire bytes per call are measured")
    ap.add_argument("--peer-copy", action="store_true", help="also measure the NVLink peer-copy bandwidth (1 GiB, one direction)")
    args = ap.parse_args(argv)

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if "RANK" in os.environ:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if dist.is_initialized() else 0
    P = dist.get_world_size() if dist.is_initialized() else 1
    hbm, how = hbm_gbs()
    max_numel = max(args.sizes_kb) * 256
    rows = []
    pool_bytes = 192 << 20
    if args.peer_copy and P > 1:
        try:
            gbs = peer_copy_gbs(dev, rank, P)
            rows.append({"impl": "peer_copy", "kb": 1 << 20, "gbs": gbs, "P": P})
        except Exception as e:  # noqa: BLE001 - symmetric memory may be unavailable; the sweep goes on
            rows.append({"impl": "peer_copy", "error": repr(e)[:200], "P": P})
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)

    # NCCL fp32 baseline
    for kb in args.sizes_kb:
        n = kb * 256
        copies = max(1, min(8, pool_bytes // (n * 4)))
        bufs = [torch.randn(n, device=dev) * 1e-3 for _ in range(copies)]
        k = {"i": 0}

        def nccl():
            if P > 1:
                dist.all_reduce(bufs[k["i"] % copies])
            k["i"] += 1
        iters = args.iters if kb >= 1024 else args.iters * 10
        ms = time_calls(nccl, iters) if P > 1 else float("nan")
        rows.append({"impl": "nccl_fp32", "kb": kb, "ms": ms, "eff_gbs": n * 4 / ms / 1e6 if P > 1 else None, "P": P})
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)
        del bufs

    for rate in args.rates:
        ctas = args.ctas or 4096
        cfg = GcowConfig(rate=rate, comm_ctas=ctas, timeout_ms=10000, oneshot_max_bytes=4 << 20, average=True)
        ar = CompressedAllReduce(max_numel, cfg, device=dev)
        for kb in args.sizes_kb:
            n = kb * 256
            copies = max(1, min(8, pool_bytes // (n * 4)))
            bufs = [torch.randn(n, device=dev) * 1e-3 for _ in range(copies)]
            for variant in (["twoshot"] if ar.header_only else args.variants):   # header-only blocks: zeros, no traffic
                if variant == "nvls" and not ar.arena.mc_ptr:
                    continue
                if variant == "oneshot" and (n > ar.oneshot_numel or P == 1):
                    continue
                k = {"i": 0}

                def call():
                    ar(bufs[k["i"] % copies], variant=variant)
                    k["i"] += 1
                iters = args.iters if kb >= 1024 else args.iters * 10
                ms = time_calls(call, iters)
                ar.check()
                roof = roofline_ms(n * 4, rate, P, variant, hbm)
                rows.append({"impl": "header_only" if ar.header_only else variant, "rate": rate, "kb": kb, "ms": ms,
                             "eff_gbs": n * 4 / ms / 1e6,
                             "roofline_ms": roof, "frac": roof / ms, "roofline": f"{how} HBM {hbm:.0f} GB/s, NVLink {NVLINK_GBS:.0f} GB/s",
                             "P": P, "ctas": ar.ctas})
                if rank == 0:
                    print(json.dumps(rows[-1]), flush=True)
            del bufs
        del ar
    # fixed accuracy with a bit cap (sparse variant): the bytes on the wire follow the data
    for spec in args.accuracy:
        tol, cap, *rest = spec.split(":")
        tiny = float(rest[0]) if rest else 0.0

        def fresh_values(n):
            t = torch.randn(n, device=dev) * 1e-3
            if tiny:
                t[int(n * (1 - tiny)):] *= 1e-5
            return t
        cfg = GcowConfig(mode="accuracy", tolerance=float(tol), rate=float(cap), comm_ctas=args.ctas or 4096,
                         timeout_ms=10000, average=True)
        ar = CompressedAllReduce(max_numel, cfg, device=dev)
        for kb in args.sizes_kb:
            n = kb * 256
            copies = max(1, min(8, pool_bytes // (n * 4)))
            bufs = [fresh_values(n) for _ in range(copies)]
            k = {"i": 0}

            def call():
                ar(bufs[k["i"] % copies])
                k["i"] += 1
            iters = args.iters if kb >= 1024 else args.iters * 10
            ms = time_calls(call, iters)
            ar.check()
            w0 = ar.wire_bytes()
            fresh = fresh_values(n)
            ar(fresh)
            ar.check()
            wire = ar.wire_bytes() - w0
            rows.append({"impl": "sparse", "tolerance": float(tol), "cap_rate": float(cap), "tiny_fraction": tiny,
                         "kb": kb, "ms": ms,
                         "eff_gbs": n * 4 / ms / 1e6, "wire_bytes_per_call": wire,
                         "fp32_ring_bytes": int(2 * (P - 1) / P * n * 4), "P": P, "ctas": ar.ctas})
            if rank == 0:
                print(json.dumps(rows[-1]), flush=True)
            del bufs, fresh
        del ar
    if rank == 0 and args.json:
        Path(args.json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
