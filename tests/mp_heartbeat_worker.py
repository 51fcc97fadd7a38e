"""Worker of the CPU liveness test: gloo ranks with a shared store; one rank leaves
(between steps, nothing in flight) and the others must notice through the heartbeat."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gcow_b200.parallel.elastic import Heartbeat, PeerFailure, RestartRequired, elastic_loop  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    mode = os.environ["GCOW_HB_MODE"]
    out = os.environ["GCOW_TEST_OUT"] + f".{rank}"
    dist.init_process_group("gloo")
    store = dist.distributed_c10d._get_default_store()
    # a generous time-out: on a loaded test machine a healthy rank's beat can be late by a second
    hb = Heartbeat(store, rank, world, interval_s=0.1, timeout_s=3.0).start()
    dist.barrier()                                        # every rank is up and beating before the steps begin
    res = {"rank": rank, "steps": 0}

    def step(i):
        if mode == "leave" and rank == world - 1 and i == 3:
            hb.stop()
            json.dump({"rank": rank, "left": True}, open(out, "w"))
            os._exit(0)                                   # dies between steps
        if mode == "raise" and rank == 1 and i == 3:
            raise PeerFailure([1], "(simulated local failure)")
        time.sleep(0.1)
        res["steps"] = i + 1

    t0 = time.time()
    try:
        elastic_loop(step, 200, hb)
        res["outcome"] = "finished"
    except RestartRequired as e:
        res["outcome"] = "restart"
        res["why"] = str(e)
    res["seconds"] = time.time() - t0
    hb.stop()
    json.dump(res, open(out, "w"))
    os._exit(0)     # skip the collective teardown: a peer may be gone


if __name__ == "__main__":
    main()
