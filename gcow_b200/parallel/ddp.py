"""DistributedDataParallel integration: the gradient buckets of stock PyTorch DDP
are all-reduced by the fused compressed kernel instead of NCCL.

``wrap_ddp`` builds DDP with 25 MB buckets that alias the parameters' .grad
(``gradient_as_bucket_view``), registers ``compressed_allreduce_hook`` and
returns the hook state. For each bucket the hook makes the communication stream
wait for the producer stream, launches ONE fused kernel there and completes a
CUDA-aware future, so backward keeps running while earlier buckets travel.

The reference runs stock DDP (NCCL fp32) and only afterwards round-trips the
whole gradient through a host codec (hw/models/train_imagenet.py:219,449-475);
at one GPU it still applies the codec round trip to the local gradient, which is
what this hook does when the world size is 1.

(No postponed evaluation of annotations in this module: DDP inspects the hook's
``bucket`` annotation and requires the class object itself.)
"""
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from ..comm.allreduce import CompressedAllReduce, CollectiveTimeout
from ..config import GcowConfig


@dataclass
class GcowDDPState:
    ar: CompressedAllReduce
    cfg: GcowConfig
    group: object = None
    buckets_seen: int = 0
    launches: int = 0
    residual: dict = field(default_factory=dict)   # error-feedback memory per bucket index
    last_buckets: list = field(default_factory=list)
    side: dict = field(default_factory=dict)       # out-of-place result buffers per bucket index (safe mode)
    pending: list = field(default_factory=list)    # (bucket buffer, side buffer) of this step (safe mode)
    timeouts: int = 0
    fallbacks: int = 0
    timing: bool = False                           # record CUDA events around every bucket's collective
    comm_events: list = field(default_factory=list)

    def begin_step(self) -> None:
        self.last_buckets.clear()
        self.pending.clear()

    def agree_on_failure(self, failed_here: bool) -> bool:
        """True on every rank if the collective gave up on ANY rank in this step. A time-out can hit some
        ranks only (a rank that arrives after its peers' deadline finds every flag set and succeeds), so the
        decision to redo the step's buckets must not be taken by each rank alone: ranks that redo would call
        NCCL while the others do not. One MAX all-reduce of a flag over the control group settles it."""
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if world == 1:
            return failed_here
        dev = self.pending[0][0].device if self.pending else torch.device("cpu")
        flag = torch.tensor([1 if failed_here else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        return bool(int(flag.item()))

    def finish_step(self) -> None:
        """Call after backward, before the optimizer step: reads the collective's status record. Default mode: a
        time-out raises CollectiveTimeout, one step late (see below). Safe mode
        (``cfg.fallback_nccl``): every bucket was reduced into a side buffer and its own buffer still holds
        the local gradient; the ranks agree whether any of them saw a failure, then either all copy the
        side buffers in, or all redo every bucket of the step with NCCL in fp32."""
        if not self.cfg.fallback_nccl:
            # The status record is read one step late, so that the host never waits for the device here (a wait at
            # this point drains the launch queue every step and the short kernels of the next forward pass then run
            # at the pace of the host). A failed bucket leaves the local gradient in place (the kernel writes its
            # output only after its last wait), the optimiser applies it, and the next step raises.
            try:
                self.ar.check_lagged(self.ar.stream)
            except CollectiveTimeout:
                self.timeouts += 1
                raise
            return
        failed = False
        try:
            self.ar.check(self.ar.stream)
        except CollectiveTimeout:
            failed = True
            self.timeouts += 1
        if self.agree_on_failure(failed):
            world = dist.get_world_size(self.group) if dist.is_initialized() else 1
            for buf, _side in self.pending:
                if world > 1:
                    dist.all_reduce(buf, group=self.group)
                    if self.cfg.average:
                        buf.div_(world)
                self.fallbacks += 1
            self.ar.reset_status()
        else:
            for buf, side in self.pending:
                buf.copy_(side)

    def comm_seconds(self) -> float:
        """Device time the communication stream spent in the buckets' collectives (codec and transfer are one
        kernel here) since the last call; needs ``timing = True``. Synchronises with the communication stream."""
        self.ar.stream.synchronize()
        t = sum(a.elapsed_time(b) for a, b in self.comm_events) / 1e3
        self.comm_events.clear()
        return t

    def step_record(self) -> dict:
        """Metrics of the step that just finished, for the JSONL log."""
        ar = self.ar
        return {"buckets": len(self.last_buckets), "bucket_numel": list(self.last_buckets),
                "variants": [ar.pick_variant(n) for n in self.last_buckets],
                "fp32_bytes": sum(self.last_buckets) * 4,
                "wire_bytes_per_rank": sum(((n + 3) // 4) * ar.bits // 8 for n in self.last_buckets),
                "rate": self.cfg.rate, "world": ar.world, "timeouts": self.timeouts, "fallbacks": self.fallbacks}

    def state_dict(self) -> dict:
        return {"cfg": self.cfg.asdict(), "residual": {k: v.cpu() for k, v in self.residual.items()}}

    def load_state_dict(self, sd: dict) -> None:
        dev = self.ar.device
        self.residual = {int(k): v.to(dev) for k, v in sd.get("residual", {}).items()}


def compressed_allreduce_hook(state: GcowDDPState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    buf = bucket.buffer()
    ar = state.ar
    cur = torch.cuda.current_stream(buf.device)
    ar.stream.wait_stream(cur)
    if state.cfg.trace:
        torch.cuda.nvtx.range_push(f"gcow_allreduce bucket {bucket.index()} {buf.numel() * 4 >> 20} MB "
                                   f"{ar.pick_variant(buf.numel())}")
    with torch.cuda.stream(ar.stream):
        if state.timing:
            t0 = torch.cuda.Event(enable_timing=True)
            t0.record(ar.stream)
        res = None
        if state.cfg.error_feedback:
            # the kernel's encode phase adds the residual to this rank's contribution and leaves behind what the
            # code of that sum dropped - no copy of the bucket and no separate codec pass
            idx = bucket.index()
            res = state.residual.get(idx)
            if res is None or res.numel() != buf.numel():
                res = torch.zeros_like(buf)
                state.residual[idx] = res
        if state.cfg.fallback_nccl:
            # safe mode: reduce into a side buffer; finish_step copies it in once all ranks
            # agree that the step's collectives succeeded, so until then the bucket keeps its local gradient
            idx = bucket.index()
            side = state.side.get(idx)
            if side is None or side.numel() != buf.numel():
                side = torch.empty_like(buf)
                state.side[idx] = side
            ar(buf, out=side, stream=ar.stream, residual=res)
            state.pending.append((buf, side))
        else:
            ar(buf, stream=ar.stream, residual=res)
        if state.timing and len(state.comm_events) < 100000:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record(ar.stream)
            state.comm_events.append((t0, t1))
        buf.record_stream(ar.stream)
        fut = torch.futures.Future(devices=[buf.device])
        fut.set_result(buf)
    if state.cfg.trace:
        torch.cuda.nvtx.range_pop()
    state.buckets_seen += 1
    state.launches += 1
    state.last_buckets.append(buf.numel())
    return fut


def nccl_fp32_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Uncompressed baseline with the same averaging semantics."""
    group = state.group if state is not None else None
    buf = bucket.buffer()
    world = dist.get_world_size(group)
    fut = dist.all_reduce(buf, group=group, async_op=True).get_future()
    return fut.then(lambda f: f.value()[0].div_(world))


def codec_roundtrip_nccl_hook(state: dict, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Variable-rate modes (fixed accuracy / fixed precision): round-trip the local bucket
    through the codec on the GPU, then all-reduce it with NCCL in fp32. ``state`` holds
    ``params`` (ZfpParams) and the byte counters ``bytes_in`` / ``bytes_out``."""
    from ..codec import compress, decompress
    buf = bucket.buffer()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    c = compress(buf, params=state["params"], dim=1, return_index=True)
    decompress(c, out=buf)
    t1.record()
    state.setdefault("codec_events", []).append((t0, t1))
    state["bytes_in"] += buf.numel() * 4
    state["bytes_out"] += c.nbytes
    world = dist.get_world_size()
    fut = dist.all_reduce(buf, async_op=True).get_future()
    return fut.then(lambda f: f.value()[0].div_(world))


def wrap_ddp(model: torch.nn.Module, cfg: Optional[GcowConfig] = None, device: Optional[torch.device] = None,
             group=None, max_bucket_numel: Optional[int] = None):
    """Returns (ddp_model, state). ``cfg.variant == 'nccl'`` gives the uncompressed baseline."""
    cfg = cfg or GcowConfig.from_env()
    device = device or torch.device("cuda", torch.cuda.current_device())
    ddp = DDP(model, device_ids=[device.index], bucket_cap_mb=cfg.bucket_mb, gradient_as_bucket_view=True,
              process_group=group, broadcast_buffers=False)
    if cfg.variant == "nccl":
        return ddp, None
    cap = max_bucket_numel or max(int(cfg.bucket_mb * (1 << 20) // 4 * 2), 1 << 20)
    biggest = max((p.numel() for p in model.parameters()), default=1)
    cap = max(cap, biggest)
    ar = CompressedAllReduce(cap, cfg, group=group, device=device)
    state = GcowDDPState(ar, cfg, group)
    ddp.register_comm_hook(state, compressed_allreduce_hook)
    return ddp, state
