"""Worker of test_elastic_cpu.py::test_safe_mode_redo_is_agreed_across_ranks: gloo ranks on CPU run
GcowDDPState.finish_step with a stand-in collective whose status check fails on chosen ranks only."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gcow_b200.comm.allreduce import CollectiveTimeout  # noqa: E402
from gcow_b200.config import GcowConfig  # noqa: E402
from gcow_b200.parallel.ddp import GcowDDPState  # noqa: E402


class FakeCollective:
    """Only what finish_step touches: a stream handle, check() and reset_status()."""
    stream = None

    def __init__(self, rank, failing):
        self.rank, self.failing, self.resets = rank, failing, 0

    def check(self, stream=None):
        if self.rank in self.failing:
            raise CollectiveTimeout(self.rank, {"code": 1})

    def reset_status(self, stream=None):
        self.resets += 1


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    failing = {int(v) for v in os.environ.get("FAILING", "").split(",") if v}
    dist.init_process_group("gloo", rank=rank, world_size=world)
    st = GcowDDPState(FakeCollective(rank, failing), GcowConfig(fallback_nccl=True, average=True))
    local = [torch.full((8,), float(rank + 1 + 10 * b)) for b in range(3)]        # what backward left in the buckets
    fused = [torch.full((8,), -1.0 - b) for b in range(3)]                        # what the fused kernel produced
    st.pending = [(l.clone(), f) for l, f in zip(local, fused)]
    st.finish_step()
    mean = [sum(float(r + 1 + 10 * b) for r in range(world)) / world for b in range(3)]
    for b, (buf, _) in enumerate(st.pending):
        want = mean[b] if failing else -1.0 - b
        assert torch.allclose(buf, torch.full((8,), want)), (rank, b, buf, want)
    assert st.fallbacks == (3 if failing else 0) and st.timeouts == (1 if rank in failing else 0)
    dist.barrier()
    dist.destroy_process_group()
    print("ok", rank)


if __name__ == "__main__":
    main()
