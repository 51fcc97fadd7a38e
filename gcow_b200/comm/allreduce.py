"""Fused compressed all-reduce: Python front end of csrc/comm/allreduce_kernels.cu.

One process per GPU. Every rank owns an *arena* (flags + two data regions) that
is mapped into all peers, either through ``torch.distributed._symmetric_memory``
(which also yields the NVSwitch multicast mapping used by the NVLS variant) or
through plain CUDA IPC handles exchanged over the host process group. A call
launches ONE kernel on the communication stream; there is no NCCL collective on
the data path. NCCL is used for the control plane only (rendezvous, the optional
fp32 fall-back after a time-out, and the uncompressed baseline).

The reference reduces gradients with stock DDP/NCCL and compresses afterwards on
the host (hw/models/train_imagenet.py:219,449-475); this class is the
"compression on the wire" that its name asks for.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..codec import ZfpParams
from ..config import GcowConfig

VARIANTS = {"twoshot": 0, "oneshot": 1, "nvls": 2, "sparse": 3}
_FUSED_BITS = (16, 32, 64, 128)


class CollectiveTimeout(RuntimeError):
    """A device-side wait of the fused all-reduce gave up (peer missing or late)."""

    def __init__(self, rank: int, record: dict):
        self.rank, self.record = rank, record
        super().__init__(f"rank {rank}: compressed all-reduce gave up waiting: {record}")


@dataclass
class _Arena:
    local_ptr: int
    peer_ptrs: list
    mc_ptr: int
    nbytes: int
    backend: str
    keep: object  # owning objects (tensor / handle / raw allocation)


def _make_arena(nbytes: int, group, device: torch.device, backend: str) -> _Arena:
    world = dist.get_world_size(group) if (dist.is_initialized() and group is not False) else 1
    lib = _native.cuda()
    if world == 1:
        t = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        return _Arena(t.data_ptr(), [t.data_ptr()], 0, nbytes, "local", t)
    if backend in ("auto", "symm"):
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(nbytes, dtype=torch.uint8, device=device)
            t.zero_()
            hdl = symm.rendezvous(t, group if group is not None else dist.group.WORLD)
            torch.cuda.synchronize(device)
            hdl.barrier()
            mc = int(hdl.multicast_ptr) if getattr(hdl, "multicast_ptr", 0) else 0
            if os.environ.get("GCOW_DISABLE_MULTICAST", "0") == "1":
                mc = 0
            return _Arena(t.data_ptr(), [int(p) for p in hdl.buffer_ptrs], mc, nbytes, "symm", (t, hdl))
        except Exception as e:  # pragma: no cover - depends on the platform
            if backend == "symm":
                raise
            if dist.get_rank(group) == 0:
                print(f"[gcow] symmetric memory unavailable ({type(e).__name__}: {e}); using CUDA IPC")
    # CUDA IPC fallback
    p = C.c_void_p()
    err = lib.gcow_ipc_alloc(nbytes, C.byref(p))
    if err:
        raise RuntimeError(f"cudaMalloc of the arena failed: {err}")
    handle = (C.c_ubyte * 64)()
    err = lib.gcow_ipc_export(p, handle)
    if err:
        raise RuntimeError(f"cudaIpcGetMemHandle failed: {err}")
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle), group=group)
    rank = dist.get_rank(group)
    ptrs = []
    for r, h in enumerate(handles):
        if r == rank:
            ptrs.append(p.value)
            continue
        q = C.c_void_p()
        buf = (C.c_ubyte * 64).from_buffer_copy(h)
        err = lib.gcow_ipc_open(buf, C.byref(q))
        if err:
            raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed: {err}")
        ptrs.append(q.value)
    dist.barrier(group=group)
    return _Arena(p.value, ptrs, 0, nbytes, "ipc", None)


class CompressedAllReduce:
    """All-reduce (sum or mean) of float32 tensors with on-the-wire ZFP compression.

    ``max_numel`` fixes the arena size; larger tensors are processed in pieces.
    Calls must be issued in the same order on every rank (as DDP does).

    ``cfg.mode == "rate"``: fixed rate, every block is ``4 * rate`` bits on the wire.
    ``cfg.mode == "accuracy"``: fixed accuracy with a bit cap (ZFP's expert mode: ``minexp`` from ``cfg.tolerance``,
    ``maxbits = 4 * cfg.rate``, ``minbits = 1``) on the sparse variant of the kernel: bit planes below the tolerance
    are dropped, and a block whose values all lie below it sends one bitmap bit and no code, so the bytes on the wire
    follow the data (``wire_bytes()``). The reference's accuracy mode is the host round trip of
    hw/models/train_imagenet.py:449-475 with ``tolerance=``.
    """

    def __init__(self, max_numel: int, cfg: GcowConfig | None = None, group=None,
                 device: torch.device | None = None, backend: str = "auto"):
        self.cfg = cfg or GcowConfig.from_env()
        if backend == "auto":      # GCOW_COMM_BACKEND=ipc|symm picks how peer memory is mapped when the caller does not
            backend = os.environ.get("GCOW_COMM_BACKEND", "auto")
        if self.cfg.dim != 1 or self.cfg.mode not in ("rate", "accuracy"):
            raise ValueError("the fused all-reduce uses the 1-D codec at fixed rate or fixed accuracy")
        self.params = ZfpParams.from_rate(self.cfg.rate, 1)
        self.sparse = self.cfg.mode == "accuracy"
        if self.sparse:
            acc = ZfpParams.from_accuracy(self.cfg.tolerance)
            if self.params.maxbits not in _FUSED_BITS:
                raise ValueError("accuracy mode needs a cap of 4, 8, 16 or 32 bits/value in cfg.rate")
            self.params = ZfpParams(1, self.params.maxbits, acc.maxprec, acc.minexp)
        # A 1-D block can never be shorter than its 9-bit header, so rates below 2.25 are floored
        # to 9 bits/block: the header alone, no bit plane. Every such block decodes to zeros, hence
        # the "all-reduce" at that rate is the zero vector on every rank and needs no traffic at all.
        self.header_only = self.params.maxbits == 9 and not self.sparse
        if self.params.maxbits not in _FUSED_BITS and not self.header_only:
            raise ValueError(f"fused all-reduce supports 4, 8, 16 or 32 bits/value (or the 9-bit floor), "
                             f"not rate {self.cfg.rate}")
        self.bits = 32 if self.header_only else self.params.maxbits
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        if self.world > 8:
            raise ValueError("one NVSwitch domain of at most 8 ranks")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.lib = _native.cuda()
        with torch.cuda.device(self.device):
            self.max_ctas = int(self.lib.gcow_ar_max_ctas_v(self.bits, 3 if self.sparse else 0))
        self.ctas = max(1, min(self.cfg.comm_ctas, self.max_ctas))
        self.max_numel = int(max_numel)
        two = self.lib.gcow_ar_region_bytes(self.max_numel, self.world, self.ctas, self.bits, 3 if self.sparse else 0)
        # A single rank always takes the one-shot path: y = D(E(x)), ONE lossy round trip, which is what the
        # reference does to the local gradient on one GPU (hw/models/train_imagenet.py:449-475).
        one_n = self.max_numel if self.world == 1 else min(self.max_numel, max(1, self.cfg.oneshot_max_bytes // 4))
        if self.sparse:
            one_n = 0               # the sparse variant is two-shot at every size and world
        one = self.lib.gcow_ar_region_bytes(one_n, self.world, self.ctas, self.bits, 1)
        self.region_cap = int(max(two, one))
        self.oneshot_numel = one_n
        nbytes = int(self.lib.gcow_ar_arena_bytes(self.region_cap))
        self.arena = _make_arena(nbytes, group if self.distributed else False, self.device, backend)
        self._peer_array = (C.c_void_p * 8)(*([C.c_void_p(p) for p in self.arena.peer_ptrs] +
                                               [C.c_void_p(0)] * (8 - len(self.arena.peer_ptrs))))
        self.status = torch.zeros(16, dtype=torch.int32, device=self.device)   # [0:8] record, [8] abort
        self.status_host = torch.zeros(16, dtype=torch.int32).pin_memory()
        self._lag_host = None          # check_lagged's two pinned slots, made on first use
        self.stamps = None
        self.epoch = 0
        self.stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._pending_event: Optional[torch.cuda.Event] = None
        self.calls = 0
        self.bytes_in = 0
        self.bytes_wire = 0
        self.wire_codes = torch.zeros(1, dtype=torch.int64, device=self.device)   # sparse variant: codes sent to peers
        self._bitmap_bytes = 0
        pow2 = self.world & (self.world - 1) == 0
        self._avg_shift = int(math.log2(self.world)) if (self.cfg.average and pow2) else 0
        self._avg_scale = 1.0 if (not self.cfg.average or pow2) else 1.0 / self.world

    # ------------------------------------------------------------------ policy
    def pick_variant(self, numel: int) -> str:
        """Deterministic in (numel, config, world) so that all ranks agree."""
        v = self.cfg.variant
        if self.sparse:
            return "sparse"
        if v == "auto":
            if self.world == 1:
                return "oneshot"
            if numel <= self.oneshot_numel:
                return "oneshot"
            return "nvls" if (self.arena.mc_ptr and self.world > 1) else "twoshot"
        if v == "nvls" and not self.arena.mc_ptr:
            return "twoshot"
        if v == "oneshot" and numel > self.oneshot_numel:
            return "twoshot"
        return v

    def ctas_for(self, numel: int) -> int:
        """Grid size for a message: one CTA per 64 blocks of a shard (each of its
        warps then handles one destination), capped by the configured grid.
        Depends only on (numel, world, configuration): identical on every rank."""
        shard_blocks = -(-((numel + 3) // 4) // self.world)
        return max(1, min(self.ctas, -(-shard_blocks // (256 if self.sparse else 64))))

    def enable_tracing(self, on: bool = True) -> None:
        """Per-CTA globaltimer stamps at the four phase boundaries of the last call."""
        self.stamps = torch.zeros(self.ctas * 4, dtype=torch.int64, device=self.device) if on else None

    # -------------------------------------------------------------------- call
    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, stream: torch.cuda.Stream | None = None,
                 variant: str | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Launch the all-reduce of ``x`` (in place unless ``out`` is given) on
        ``stream`` (default: the current stream). Does not synchronise.
        ``residual`` (float32, same size): error feedback inside the kernel - this rank contributes
        ``x + residual`` and ``residual`` becomes what its compressed code of that sum dropped."""
        if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
            raise TypeError("need a contiguous float32 CUDA tensor")
        out = x if out is None else out
        n = x.numel()
        s = stream or torch.cuda.current_stream(self.device)
        if residual is not None and (residual.dtype != torch.float32 or residual.numel() != n or not residual.is_contiguous()
                                     or residual.device != x.device):
            raise TypeError("residual must be a contiguous float32 tensor of the input's size on the same device")
        for lo in range(0, n, self.max_numel):
            hi = min(n, lo + self.max_numel)
            self._launch(x.view(-1)[lo:hi], out.view(-1)[lo:hi], s, variant,
                         residual.view(-1)[lo:hi] if residual is not None else None)
        return out

    def _launch(self, x: torch.Tensor, out: torch.Tensor, s: torch.cuda.Stream, variant: str | None,
                residual: torch.Tensor | None = None) -> None:
        n = x.numel()
        if n == 0:
            return
        if self.header_only:
            with torch.cuda.stream(s):
                if residual is not None:          # everything is dropped: the residual keeps the whole input
                    residual.add_(x)
                out.zero_()
            self.calls += 1
            self.bytes_in += n * 4
            return
        vname = variant or self.pick_variant(n)
        v = VARIANTS[vname]
        if (v == 3) != self.sparse:
            raise ValueError("the sparse variant goes with cfg.mode == 'accuracy', the others with 'rate'")
        if v == 2 and not self.arena.mc_ptr:
            raise RuntimeError("NVLS variant needs a multicast mapping")
        self.epoch += 1
        shift = self._avg_shift
        post = self._avg_scale
        if v == 3:
            err = self.lib.gcow_ar_launch_sparse(
                x.data_ptr(), out.data_ptr(), n, self.rank, self.world, self.bits, self.ctas_for(n), shift,
                C.c_float(post), self._peer_array, self.region_cap, self.epoch, int(self.cfg.timeout_ms) * 1_000_000,
                self.status.data_ptr(), self.status[8:].data_ptr(),
                self.stamps.data_ptr() if self.stamps is not None else None,
                residual.data_ptr() if residual is not None else None, self.params.minexp,
                self.wire_codes.data_ptr(), s.cuda_stream)
            if err:
                raise RuntimeError(f"gcow_ar_launch_sparse failed: {err}")
            self.calls += 1
            self.bytes_in += n * 4
            P = self.world
            shard_blocks = -(-(-(-((n + 3) // 4) // P)) // 64) * 64
            self._bitmap_bytes += 2 * (P - 1) * shard_blocks // 8       # one bit per block, both phases
            return
        if v == 1 and shift:          # one-shot has no final decode to fold the shift into
            post, shift = post * 2.0 ** (-shift), 0
        err = self.lib.gcow_ar_launch_ef(
            x.data_ptr(), out.data_ptr(), n, self.rank, self.world, v, self.bits, self.ctas_for(n), shift,
            C.c_float(post), self._peer_array, C.c_void_p(self.arena.mc_ptr), self.region_cap, self.epoch,
            int(self.cfg.timeout_ms) * 1_000_000, self.status.data_ptr(), self.status[8:].data_ptr(),
            self.stamps.data_ptr() if self.stamps is not None else None,
            residual.data_ptr() if residual is not None else None, s.cuda_stream)
        if err:
            raise RuntimeError(f"gcow_ar_launch failed: {err}")
        self.calls += 1
        self.bytes_in += n * 4
        cb = ((n + 3) // 4) * self.bits // 8
        P = self.world
        self.bytes_wire += int(cb * (P - 1) * (1 if v == 1 else 2.0 / P)) if P > 1 else 0

    def commit(self, src: torch.Tensor, dst: torch.Tensor, verdict: torch.Tensor, stream: torch.cuda.Stream) -> None:
        """Enqueue ``dst <- src`` on ``stream`` unless a call has failed since the last
        ``check``; ``verdict`` (one int32 on the device) receives 1 = copied, 2 = skipped."""
        err = self.lib.gcow_ar_commit(self.status.data_ptr(), src.data_ptr(), dst.data_ptr(), src.numel(),
                                      verdict.data_ptr(), self.ctas, stream.cuda_stream)
        if err:
            raise RuntimeError(f"gcow_ar_commit failed: {err}")

    def reset_status(self, stream: torch.cuda.Stream | None = None) -> None:
        s = stream or torch.cuda.current_stream(self.device)
        with torch.cuda.stream(s):
            self.status.zero_()

    # ------------------------------------------------------------------ status
    def check(self, stream: torch.cuda.Stream | None = None) -> None:
        """Synchronise with ``stream`` and raise CollectiveTimeout if any call
        since the last check gave up. The status record is cleared."""
        s = stream or torch.cuda.current_stream(self.device)
        with torch.cuda.stream(s):
            self.status_host.copy_(self.status, non_blocking=True)
        s.synchronize()
        if int(self.status_host[0]) != 0:
            rec = dict(zip(("code", "phase", "peer", "cta", "expected", "seen", "epoch"),
                           (int(v) for v in self.status_host[:7])))
            with torch.cuda.stream(s):
                self.status.zero_()
            s.synchronize()
            raise CollectiveTimeout(self.rank, rec)

    def check_lagged(self, stream: torch.cuda.Stream | None = None) -> None:
        """As ``check`` without stalling the host: enqueue a copy of the status record on ``stream`` and raise for the
        record copied by the PREVIOUS call (whose copy finished a step ago). A time-out is therefore reported one
        call late; callers that must act on it before using the result (safe mode) use ``check``."""
        s = stream or torch.cuda.current_stream(self.device)
        if self._lag_host is None:
            self._lag_host = torch.zeros(2, 16, dtype=torch.int32).pin_memory()
            self._lag_events = [None, None]
            self._lag_calls = 0
        slot = self._lag_calls & 1
        self._lag_calls += 1
        with torch.cuda.stream(s):
            self._lag_host[slot].copy_(self.status, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(s)
        self._lag_events[slot] = ev
        prev = slot ^ 1
        if self._lag_events[prev] is not None:
            self._lag_events[prev].synchronize()
            self._lag_events[prev] = None
            if int(self._lag_host[prev, 0]) != 0:
                rec = dict(zip(("code", "phase", "peer", "cta", "expected", "seen", "epoch"),
                               (int(v) for v in self._lag_host[prev, :7])))
                with torch.cuda.stream(s):
                    self.status.zero_()
                self._lag_events = [None, None]
                raise CollectiveTimeout(self.rank, rec)

    def phase_stamps(self) -> torch.Tensor | None:
        """[ctas, 4] device nanosecond stamps (start, pushed, reduced, done) of the last call."""
        return None if self.stamps is None else self.stamps.view(self.ctas, 4).cpu()

    def wire_bytes(self) -> int:
        """Bytes this rank has stored into other ranks' memory so far. Fixed rate: known from the sizes. Accuracy mode:
        the kernel's count of codes sent plus the bitmaps (reads the device counter, so it synchronises)."""
        if self.sparse:
            return int(self.wire_codes.item()) * self.bits // 8 + self._bitmap_bytes
        return self.bytes_wire

    def wire_ratio(self) -> float:
        """fp32 bytes a ring all-reduce would move per rank over compressed bytes moved."""
        P = self.world
        wire = self.wire_bytes()
        if P == 1 or not wire:
            return 0.0
        return (2.0 * (P - 1) / P * self.bytes_in) / wire


def nccl_allreduce_mean(x: torch.Tensor, group=None) -> torch.Tensor:
    """Uncompressed baseline: NCCL fp32 all-reduce followed by the division."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, group=group)
        x.div_(dist.get_world_size(group))
    return x
