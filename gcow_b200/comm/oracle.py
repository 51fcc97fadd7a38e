"""Host models of the compressed all-reduce.

``allreduce_oracle`` is the arithmetic definition the fused kernels must match
bit for bit: two-shot  y = D(E( sum_r D(E(x_r)) )) / 2^shift, one-shot
y = ( sum_r D(E(x_r)) ) / 2^shift, sums in ascending rank order in fp32.
``protocol_model`` runs the same three phases with host threads as ranks and
lets a test drop a flag, skip or delay a rank, or pre-seed stale epochs.
"""
from __future__ import annotations

import os

import numpy as np

from .. import _native
from ..codec import ZfpParams

_T = max(1, min(16, os.cpu_count() or 1))


def allreduce_oracle(xs: np.ndarray, params: ZfpParams, variant: str = "twoshot", shift: int = 0) -> np.ndarray:
    """xs: float32 array [P, n]. Returns the float32 result every rank must hold."""
    xs = np.ascontiguousarray(xs, dtype=np.float32)
    P, n = xs.shape
    out = np.zeros(n, dtype=np.float32)
    v = 1 if variant == "oneshot" else 0
    _native.cpu().gcow_oracle_allreduce(xs.ctypes.data, P, n, params.as_c(), v, shift, out.ctypes.data, _T)
    return out


def protocol_model(xs: np.ndarray, bits: int, variant: str = "twoshot", ctas: int = 4, shift: int = 0,
                   timeout_ms: int = 2000, fault_call: int = -1, skip_rank: int = -1, delay_rank: int = -1,
                   delay_ms: int = 0, drop: tuple = (-1, -1, -1), stale_epoch: int = -1, minexp: int = -1074):
    """xs: float32 [calls, P, n]. Returns (outs [calls, P, n], status [P, 8], failed_ranks).
    ``variant="sparse"`` is the fixed-accuracy variant: planes below ``2**minexp`` are dropped, ``bits`` caps a block."""
    xs = np.ascontiguousarray(xs, dtype=np.float32)
    calls, P, n = xs.shape
    outs = np.zeros_like(xs)
    status = np.zeros((P, 8), dtype=np.uint32)
    v = {"twoshot": 0, "oneshot": 1, "nvls": 0, "sparse": 3}[variant]
    failed = _native.cpu().gcow_protocol_model2(
        xs.ctypes.data, outs.ctypes.data, P, n, ctas, bits, v, shift, calls, timeout_ms, fault_call,
        skip_rank, delay_rank, delay_ms, drop[0], drop[1], drop[2], stale_epoch, status.ctypes.data, int(minexp))
    return outs, status, int(failed)
