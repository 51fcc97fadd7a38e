"""autograd.Function wrappers around the sm_100a compute kernels.

``*_usable`` predicates say whether a kernel covers a given call (dtype, layout,
alignment); callers fall back to PyTorch otherwise.
"""
from __future__ import annotations

import torch

from .. import _native


_launches = 0


def launch_count() -> int:
    """How many compute kernels of this library were launched through this module."""
    return _launches


def _have(name: str) -> bool:
    if not _native.cuda_available():
        return False
    try:
        return hasattr(_native.cuda(), name)
    except Exception:
        return False


def gemm_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    return False


def conv1x1_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    return False


def layernorm_usable(x: torch.Tensor, mod) -> bool:
    return False


def linear(x, w, b):  # pragma: no cover - replaced when the GEMM kernel lands
    raise NotImplementedError


def conv1x1(x, w, b):  # pragma: no cover
    raise NotImplementedError


def layernorm(x, w, b, eps):  # pragma: no cover
    raise NotImplementedError
