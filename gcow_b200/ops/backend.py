"""Which implementation the nn wrappers use.

``own``   – the sm_100a kernels of this library wherever one exists (default on a GPU);
``torch`` – PyTorch's library-backed operators (cuBLAS / cuDNN): the baseline arm.
"""
import os

_backend = os.environ.get("GCOW_OPS", "own")


def set_backend(name: str) -> None:
    global _backend
    if name not in ("own", "torch"):
        raise ValueError("backend must be 'own' or 'torch'")
    _backend = name


def get_backend() -> str:
    return _backend
