"""Drop-in stand-in for the two zfpy calls the reference's training studies make.

``hw/models/train_imagenet.py:459-465`` and ``hw/models/train_resnet_cifar10.py:84-95`` flatten the gradients into
one float32 numpy array, call ``zfpy.compress_numpy(arr, rate=... | precision=... | tolerance=...)`` and
``zfpy.decompress_numpy(buf)``, and copy the result back. With

    import gcow_b200.zfpy_compat as zfpy

those scripts run on this library's codec: the CPU oracle by default, the CUDA kernels with ``device="cuda"``.
Arrays of one dimension use 1-D blocks of 4 (what zfpy does for a flat array), two-dimensional arrays 4 x 4 blocks,
anything else is flattened. The returned buffer is this library's header-less ZFP stream behind a 40-byte
self-describing header (magic, rank, shape, the four codec parameters); it is not zfp's own header format, so the
buffers are not interchangeable with zfpy's.
"""
from __future__ import annotations

import struct

import numpy as np
import torch

from .codec import Compressed, ZfpParams, compress, decompress

_MAGIC = b"GCOWZFP1"
_HDR = struct.Struct("<8sIIqqiiii")     # magic, rank of the original, codec dim, n0, n1, minbits, maxbits, maxprec, minexp


def compress_numpy(arr: np.ndarray, tolerance: float = -1, rate: float = -1, precision: int = -1,
                   write_header: bool = True, device: str = "cpu") -> bytes:
    """zfpy.compress_numpy for float32 arrays. Exactly one of ``tolerance``, ``rate``, ``precision`` may be positive;
    none selects a near-lossless precision of 32 bit planes (zfpy's reversible mode is not reproduced)."""
    a = np.ascontiguousarray(arr)
    if a.dtype != np.float32:
        raise TypeError("only float32 arrays are supported (the reference compresses float32 gradients)")
    chosen = [(k, v) for k, v in (("tolerance", tolerance), ("rate", rate), ("precision", precision)) if v is not None and v > 0]
    if len(chosen) > 1:
        raise ValueError("give at most one of tolerance, rate, precision")
    dim = 2 if a.ndim == 2 else 1
    work = a if a.ndim == 2 else a.reshape(-1)
    kw = {chosen[0][0]: chosen[0][1]} if chosen else {"precision": 32}
    c = compress(torch.from_numpy(work).to(device), dim=dim, **kw)
    stream = c.stream.cpu().numpy().tobytes()
    if not write_header:
        return stream
    n0, n1 = (work.shape[0], work.shape[1]) if dim == 2 else (work.shape[0], 0)
    p = c.params
    # the original shape of a flattened array is not kept: zfpy callers reshape themselves (the reference does)
    return _HDR.pack(_MAGIC, a.ndim, dim, n0, n1, p.minbits, p.maxbits, p.maxprec, p.minexp) + stream


def decompress_numpy(buf: bytes, device: str = "cpu") -> np.ndarray:
    """zfpy.decompress_numpy for buffers written by :func:`compress_numpy` with ``write_header=True``."""
    if len(buf) < _HDR.size or buf[:8] != _MAGIC:
        raise ValueError("not a buffer written by gcow_b200.zfpy_compat.compress_numpy (header-less streams need "
                         "gcow_b200.decompress with explicit parameters)")
    _, _rank, dim, n0, n1, minbits, maxbits, maxprec, minexp = _HDR.unpack_from(buf)
    params = ZfpParams(minbits, maxbits, maxprec, minexp)
    shape = (n0, n1) if dim == 2 else (n0,)
    stream = torch.frombuffer(bytearray(buf[_HDR.size:]), dtype=torch.uint8).to(device)
    out = decompress(Compressed(stream, params, shape, None))
    return out.cpu().numpy()
