"""Worker of the multi-GPU all-reduce tests (one process per GPU, torchrun).
Every rank regenerates all ranks' inputs from their seeds, computes the host
oracle and compares its own device result bit for bit. Results go to the JSON
file named by GCOW_TEST_OUT (rank 0) and to the exit code."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gcow_b200.codec import ZfpParams  # noqa: E402
from gcow_b200.comm import CompressedAllReduce, allreduce_oracle  # noqa: E402
from gcow_b200.config import GcowConfig  # noqa: E402


def gen(seed, n):
    return (np.random.default_rng(seed).standard_normal(n) * 1e-3).astype(np.float32)


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    backend = os.environ.get("GCOW_COMM_BACKEND", "auto")
    shift = {1: 0, 2: 1, 4: 2, 8: 3}.get(world, 0)
    fails, ran = [], 0
    info = {}
    sizes = [5, 4099, (1 << 16) | 3, 1 << 21]
    for rate in (8, 4, 16, 32):
        cfg = GcowConfig(rate=rate, comm_ctas=int(os.environ.get("GCOW_TEST_CTAS", "24")), timeout_ms=5000,
                         oneshot_max_bytes=1 << 20)
        ar = CompressedAllReduce(1 << 21, cfg, device=dev, backend=backend)
        info = {"backend": ar.arena.backend, "multicast": bool(ar.arena.mc_ptr), "ctas": ar.ctas,
                "max_ctas": ar.max_ctas}
        p = ZfpParams.from_rate(rate, 1)
        variants = ["twoshot", "oneshot"] + (["nvls"] if ar.arena.mc_ptr else [])
        for variant in variants:
            for n in sizes:
                if variant == "oneshot" and n > ar.oneshot_numel:
                    continue
                xs = np.stack([gen(1000 * n + 17 * rate + r, n) for r in range(world)])
                ref = allreduce_oracle(xs, p, "oneshot" if variant == "oneshot" else "twoshot", shift)
                x = torch.from_numpy(xs[rank]).to(dev)
                # two back-to-back calls on fresh copies exercise both parities
                y1 = ar(x.clone(), variant=variant)
                y2 = ar(x.clone(), variant=variant)
                ar.check()
                ran += 1
                for y in (y1, y2):
                    if not np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32)):
                        bad = int((y.cpu().numpy().view(np.uint32) != ref.view(np.uint32)).sum())
                        fails.append(f"rate {rate} {variant} n {n}: {bad} words differ")
                        break
        # unaligned in-place view through the automatic variant choice
        base = torch.zeros((1 << 16) + 8, device=dev)
        n = (1 << 16) + 1
        xs = np.stack([gen(99 + r, n) for r in range(world)])
        base[1:1 + n] = torch.from_numpy(xs[rank]).to(dev)
        v = ar.pick_variant(n)
        ar(base[1:1 + n])
        ar.check()
        ref = allreduce_oracle(xs, p, "oneshot" if v == "oneshot" else "twoshot", shift)
        if not np.array_equal(base[1:1 + n].cpu().numpy().view(np.uint32), ref.view(np.uint32)):
            fails.append(f"rate {rate} unaligned view ({v}) differs")
        if float(base[0]) != 0.0 or float(base[1 + n:].abs().sum()) != 0.0:
            fails.append(f"rate {rate} unaligned view wrote outside its range")
        ran += 1
        del ar
    # fixed accuracy with a bit cap (the sparse variant): half of every input lies far below the tolerance, so the
    # blocks there send nothing; results against the host model at the same parameters, wire bytes against the count
    for cap, tol in ((8, 1e-3), (4, 1e-2), (16, 1e-6), (32, 1e-4)):
        cfg = GcowConfig(mode="accuracy", tolerance=tol, rate=cap, comm_ctas=int(os.environ.get("GCOW_TEST_CTAS", "24")),
                         timeout_ms=5000)
        ar = CompressedAllReduce(1 << 21, cfg, device=dev, backend=backend)
        for n in sizes:
            xs = np.stack([gen(7000 * n + 31 * cap + r, n) for r in range(world)])
            xs[:, n // 2:] *= np.float32(1e-5)
            ref = allreduce_oracle(xs, ar.params, "twoshot", shift)
            x = torch.from_numpy(xs[rank]).to(dev)
            y1 = ar(x.clone())
            y2 = ar(x.clone())
            ar.check()
            ran += 1
            for y in (y1, y2):
                if not np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32)):
                    bad = int((y.cpu().numpy().view(np.uint32) != ref.view(np.uint32)).sum())
                    fails.append(f"accuracy tol {tol} cap {cap} n {n}: {bad} words differ")
                    break
        if world > 1:
            dense = ar.bytes_in * cap / 32.0 * 2.0 * (world - 1) / world
            if not (0 < ar.wire_bytes() < 0.8 * dense):
                fails.append(f"accuracy tol {tol} cap {cap}: {ar.wire_bytes()} wire bytes, dense would be {dense:.0f}")
        del ar
    if os.environ.get("GCOW_TEST_BIG") == "1":
        # One 256 MB fp32 buffer per rank (values ~N(0, 1e-3), seed = rank) at 4, 8 and 16 bit/value against the host
        # model: rank 0 computes decode-sum-encode on the CPU and broadcasts it, every rank compares on the device.
        n = 64 << 20
        xs = None
        if rank == 0:
            xs = np.stack([gen(r, n) for r in range(world)])
        mine = torch.from_numpy(gen(rank, n)).to(dev)
        for rate in (8, 4, 16):
            cfg = GcowConfig(rate=rate, comm_ctas=4096, timeout_ms=20000)
            ar = CompressedAllReduce(n, cfg, device=dev, backend=backend)
            p = ZfpParams.from_rate(rate, 1)
            ref = torch.empty(n, device=dev)
            if rank == 0:
                ref.copy_(torch.from_numpy(allreduce_oracle(xs, p, "twoshot", shift)))
            dist.broadcast(ref, 0)
            for variant in ["twoshot"] + (["nvls"] if ar.arena.mc_ptr else []):
                y = ar(mine.clone(), variant=variant)
                ar.check()
                bad = int((y.view(torch.int32) != ref.view(torch.int32)).sum())
                if bad:
                    fails.append(f"256 MB rate {rate} {variant}: {bad} words differ")
                ran += 1
            del ar
    allf = [None] * world
    dist.all_gather_object(allf, fails)
    if rank == 0:
        out = os.environ.get("GCOW_TEST_OUT")
        res = {"world": world, "cases": ran, "fails": allf, **info}
        print(json.dumps(res))
        if out:
            with open(out, "w") as f:
                json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if any(allf) else 0)


if __name__ == "__main__":
    main()
