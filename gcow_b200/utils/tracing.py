"""Tracing helpers: NVTX ranges, CUDA-event phase timers and an nvidia-smi clock
sampler (read-only queries; no GPU setting is ever changed).

The reference profiles with XRT runtime tracing (hw/xrt.ini:1-10) and wall-clock
accumulators around codec and transfers (hw/models/train_imagenet.py:97-99,
452-473); here device work is timed with CUDA events on the launching stream and
the fused all-reduce can stamp its own phases with the device global timer
(CompressedAllReduce.enable_tracing)."""
from __future__ import annotations

import contextlib
import statistics
import subprocess
import threading

import torch

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimer:
    """Named CUDA-event intervals on the current stream; ``summary()`` syncs once."""

    def __init__(self):
        self.spans = []

    @contextlib.contextmanager
    def span(self, name: str):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self.spans.append((name, a, b))

    def summary(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for name, a, b in self.spans:
            out.setdefault(name, []).append(a.elapsed_time(b))
        self.spans.clear()
        return {k: {"n": len(v), "ms_mean": sum(v) / len(v), "ms_max": max(v)} for k, v in out.items()}


def sample_clocks(gpu: int | None = None) -> list[dict]:
    """One nvidia-smi sample per GPU (empty list if nvidia-smi is unavailable)."""
    cmd = ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits"]
    if gpu is not None:
        cmd += ["-i", str(gpu)]
    try:
        txt = subprocess.run(cmd, capture_output=True, text=True, timeout=10).stdout
    except Exception:
        return []
    rows = []
    for line in txt.strip().splitlines():
        f = [s.strip() for s in line.split(",")]
        if len(f) < 9:
            continue
        try:
            rows.append({"index": int(f[0]), "sm_mhz": float(f[1]), "sm_max_mhz": float(f[2]),
                         "power_w": float(f[3]) if f[3] not in ("[N/A]", "N/A") else None,
                         "reasons_active": f[4], "hw_slowdown": f[5], "hw_thermal_slowdown": f[6],
                         "sw_thermal_slowdown": f[7], "sw_power_cap": f[8]})
        except ValueError:
            continue
    return rows


class ClockSampler:
    """Samples SM clocks and throttle reasons in a background thread while a timed
    region runs; ``stop()`` returns {"sm_mhz": median, "sm_max_mhz": ..., "reasons": [...]}."""

    def __init__(self, gpu: int = 0, period_s: float = 0.1):
        self.gpu, self.period = gpu, period_s
        self.samples: list[dict] = []
        self._stop = threading.Event()
        self._th: threading.Thread | None = None

    def start(self) -> "ClockSampler":
        def run():
            while not self._stop.is_set():
                self.samples += sample_clocks(self.gpu)
                self._stop.wait(self.period)
        self._th = threading.Thread(target=run, daemon=True)
        self._th.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=15)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = set()
        for s in self.samples:
            for k in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"):
                if str(s[k]).lower().startswith("active"):
                    reasons.add(k)
        return {"sm_mhz": statistics.median(s["sm_mhz"] for s in self.samples),
                "sm_max_mhz": max(s["sm_max_mhz"] for s in self.samples),
                "reasons": sorted(reasons), "samples": len(self.samples)}
