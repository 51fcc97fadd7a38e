"""Worker of test_late_peer_times_out_on_both_ranks_then_recovers (2 GPUs, torchrun).

The failure is made on the host and between steps: rank 1 sleeps before it launches its kernel, so rank 0's
bounded waits run out (and rank 1's in turn, because rank 0 has left). No kernel or collective is in flight
when a rank is late, every device wait is 50 ms, peer memory is mapped through CUDA IPC (no multicast object).
"""
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gcow_b200.codec import ZfpParams  # noqa: E402
from gcow_b200.comm import CollectiveTimeout, CompressedAllReduce, allreduce_oracle  # noqa: E402
from gcow_b200.config import GcowConfig  # noqa: E402


def gen(seed, n):
    return (np.random.default_rng(seed).standard_normal(n) * 1e-3).astype(np.float32)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n = 1 << 18
    p = ZfpParams.from_rate(8, 1)
    xs = np.stack([gen(5 + r, n) for r in range(world)])
    ref = allreduce_oracle(xs, p, "twoshot", 1)
    cfg = GcowConfig(rate=8, comm_ctas=16, timeout_ms=50, variant="twoshot")
    ar = CompressedAllReduce(n, cfg, device=dev)          # GCOW_COMM_BACKEND=ipc from the test's environment
    x = torch.from_numpy(xs[rank]).to(dev)

    # healthy call first
    y = ar(x.clone()); ar.check()
    ok0 = np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))

    # the late peer
    dist.barrier(); torch.cuda.synchronize()
    if rank == 1:
        time.sleep(0.3)
    timed_out = False
    keep = x.clone()
    try:
        ar(keep); ar.check()
    except CollectiveTimeout:
        timed_out = True
    torch.cuda.synchronize()
    dist.barrier()                      # both ranks are out of the failed call before the next one starts

    # next call, fresh epoch: bit-exact again
    y = ar(x.clone()); ar.check()
    ok1 = ok0 and np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    del ar

    # the training hook in safe mode: the step with the late rank completes through NCCL, replicas stay equal
    from gcow_b200.train import SyntheticImages, Trainer
    tcfg = GcowConfig(rate=8, comm_ctas=16, bucket_mb=1, timeout_ms=50, fallback_nccl=True)
    tr = Trainer("resnet18", batch_size=4, cfg=tcfg, num_classes=10, device=dev)
    bx, by = SyntheticImages(4, 64, 10, pool=1, seed=rank).next()
    tr.step(bx, by)
    torch.cuda.synchronize(); dist.barrier()
    if rank == 1:
        time.sleep(0.3)
    tr.step(bx, by)                     # rank 0 times out, the ranks agree, NCCL redoes the buckets
    torch.cuda.synchronize(); dist.barrier()
    tr.step(bx, by)
    tr.last_loss()
    w = tr.ddp.module.fc.weight.detach().float().contiguous()
    ws = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(ws, w)
    equal = all(torch.equal(ws[0], t) for t in ws)

    rec = {"timed_out": timed_out, "ok": ok1, "fallbacks": tr.hook_state.fallbacks}
    allr = [None] * world
    dist.all_gather_object(allr, rec)
    if rank == 0:
        res = {"timed_out": [r["timed_out"] for r in allr], "recovered_bit_exact": [r["ok"] for r in allr],
               "safe_mode_fallbacks": [r["fallbacks"] for r in allr], "replicas_equal": bool(equal)}
        print(json.dumps(res))
        out = os.environ.get("GCOW_TEST_OUT")
        if out:
            with open(out, "w") as f:
                json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
