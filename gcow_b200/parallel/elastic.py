"""Liveness and restart helpers for the host side of a training job.

Failures are detected where they can be detected without touching a GPU:

* ``Heartbeat`` - every rank bumps a key in the job's c10d store from a host
  thread; a peer whose stamp is older than ``timeout_s`` is reported dead, and any
  rank can post an abort reason that all others see before their next launch.
* the fused all-reduce bounds every device wait and reports through
  ``CollectiveTimeout`` (see comm/allreduce.py);
* ``elastic_loop`` wraps a step function: on a collective time-out, a dead peer or
  a posted abort it stops launching, tears the process group down and raises
  ``RestartRequired`` so that the launcher (torchrun --max-restarts) can
  re-rendezvous; ``resume_if_present`` then reloads the last checkpoint.

The reference has no failure handling beyond exiting on an OpenCL error
(hw/include/host.hpp:18-24) and stopping on a NaN loss (hw/models/train_imagenet.py:445-446).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, dead, reason=""):
        self.dead, self.reason = list(dead), reason
        super().__init__(f"peers {self.dead} stopped responding {reason}".strip())


class RestartRequired(RuntimeError):
    """The job must re-rendezvous and resume from its last checkpoint."""


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, timeout_s: float = 3.0,
                 prefix: str = "gcow/hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._th: Optional[threading.Thread] = None
        self._started = time.time()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self.store.set(self._key(self.rank), repr(time.time()))

    def start(self) -> "Heartbeat":
        self.beat()

        def run():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._th = threading.Thread(target=run, daemon=True)
        self._th.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=5)

    def last_seen(self, r: int) -> Optional[float]:
        key = self._key(r)
        try:
            if not self.store.check([key]):
                return None
            return float(self.store.get(key).decode())
        except Exception:
            return None

    def dead_peers(self) -> list:
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            t = self.last_seen(r)
            if t is None:
                if now - self._started > self.timeout:       # never showed up
                    dead.append(r)
            elif now - t > self.timeout:
                dead.append(r)
        return dead

    def post_abort(self, reason: str) -> None:
        self.store.set(f"{self.prefix}/abort", f"{self.rank}:{reason}")

    def abort_reason(self) -> Optional[str]:
        key = f"{self.prefix}/abort"
        try:
            return self.store.get(key).decode() if self.store.check([key]) else None
        except Exception:
            return None

    def check(self) -> None:
        """Raise before the next launch if a peer is gone or somebody asked to stop."""
        reason = self.abort_reason()
        if reason is not None:
            raise PeerFailure([int(reason.split(":", 1)[0])], f"(abort posted: {reason})")
        dead = self.dead_peers()
        if dead:
            raise PeerFailure(dead)


def elastic_loop(step: Callable[[int], None], steps: int, heartbeat: Optional[Heartbeat] = None,
                 on_failure: Optional[Callable[[Exception], None]] = None) -> int:
    """Run ``step(i)`` for i in range(steps). Between steps - never with a kernel or
    collective of this rank in flight - consult the heartbeat. Any failure is posted
    for the peers, passed to ``on_failure`` (e.g. save what can be saved) and turned
    into RestartRequired. Returns the number of completed steps."""
    from ..comm.allreduce import CollectiveTimeout
    done = 0
    try:
        for i in range(steps):
            if heartbeat is not None:
                heartbeat.check()
            step(i)
            done += 1
    except (CollectiveTimeout, PeerFailure, dist.DistBackendError) as e:   # type: ignore[attr-defined]
        if heartbeat is not None:
            try:
                heartbeat.post_abort(type(e).__name__)
            except Exception:
                pass
        if on_failure is not None:
            on_failure(e)
        raise RestartRequired(f"after {done} steps: {e}") from e
    return done


def resume_if_present(trainer, path: str) -> bool:
    """Load ``path`` into the trainer when it exists (the restart half of elastic recovery)."""
    from ..utils.checkpoint import load_checkpoint
    if not path or not os.path.isfile(path):
        return False
    sd = load_checkpoint(path, map_location=f"cuda:{trainer.device.index}" if trainer.device.type == "cuda" else "cpu")
    trainer.load_state_dict(sd["trainer"] if "trainer" in sd else sd)
    return True
