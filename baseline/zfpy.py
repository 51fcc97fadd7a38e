"""Stand-in for the third-party ``zfpy`` module that the reference's training
scripts import (hw/models/train_imagenet.py:10,459-465,
hw/models/train_resnet_cifar10.py:97-122) and that is not installed here.

Only the two calls those scripts make exist: ``compress_numpy(array,
rate=|tolerance=|precision=)`` and ``decompress_numpy(buffer)``. Both run the
REFERENCE's own CPU codec: ``ref_compress_1d`` / ``ref_decompress`` of
``_ref/libgcowref.so``, which is the unmodified sw/src/*.c plus the shim in
ref_driver.cpp that pushes blocks of four through the reference's stage
functions. Nothing of gcow_b200 is imported, so a training step that uses this
module is a reference-only code path.

The byte string carries a 32-byte header of this module's own (zfp's header
format is not reproduced): magic, element count, the four codec parameters.
"""
import ctypes as C
import struct
from pathlib import Path

import numpy as np

_SO = Path(__file__).resolve().parent / "_ref" / "libgcowref.so"
_MAGIC = b"RZF1"
_HDR = struct.Struct("<4sQiiii4x")
_lib = None


def _load():
    global _lib
    if _lib is None:
        if not _SO.exists():
            raise ImportError(f"{_SO} is missing: run baseline/build_ref.sh with a reference checkout")
        lib = C.CDLL(str(_SO))
        u64, ptr = C.c_uint64, C.c_void_p
        lib.ref_compress_1d.restype = u64
        lib.ref_compress_1d.argtypes = [ptr, u64, ptr, ptr, u64]
        lib.ref_decompress.restype = None
        lib.ref_decompress.argtypes = [ptr, u64, ptr, u64, u64, ptr]
        lib.ref_set_accuracy.restype = None
        lib.ref_set_accuracy.argtypes = [C.c_double, ptr]
        _lib = lib
    return _lib


def _params(tolerance, rate, precision):
    """(minbits, maxbits, maxprec, minexp) for one-dimensional float32 data, by zfp's rules."""
    lib = _load()
    chosen = [v for v in (tolerance, rate, precision) if v is not None and v >= 0]
    if len(chosen) > 1:
        raise ValueError("only one of tolerance, rate and precision may be given")
    if tolerance is not None and tolerance >= 0:
        p = (C.c_int32 * 4)()
        lib.ref_set_accuracy(float(tolerance), p)       # sw/src/common.c:6-21
        return tuple(int(v) for v in p)
    if rate is not None and rate >= 0:
        bits = max(int(np.floor(4 * float(rate) + 0.5)), 9)   # block of 4 values; header is 9 bits
        return (bits, bits, 64, -1074)
    if precision is not None and precision >= 0:
        return (1, 16658, int(precision), -1074)
    return (1, 16658, 64, -1074)                        # all defaults: near-lossless


def compress_numpy(arr, tolerance=-1, rate=-1, precision=-1, write_header=True):
    a = np.ascontiguousarray(arr, dtype=np.float32).reshape(-1)
    n = a.size
    prm = _params(tolerance, rate, precision)
    blocks = (n + 3) // 4
    per_block = min(max(9 + 3 + 4 * 32, prm[0]), max(prm[1], 9))
    cap = ((blocks * per_block + 63) // 64 + 2) * 8
    out = np.empty(cap, dtype=np.uint8)
    p = (C.c_int32 * 4)(*prm)
    used = _load().ref_compress_1d(a.ctypes.data, n, p, out.ctypes.data, cap)
    return _HDR.pack(_MAGIC, n, *prm) + out[:used].tobytes()


def decompress_numpy(buf):
    magic, n, *prm = _HDR.unpack_from(buf, 0)
    if magic != _MAGIC:
        raise ValueError("not a stream written by this module")
    payload = np.frombuffer(buf, dtype=np.uint8, offset=_HDR.size)
    padded = np.zeros(payload.size + 16, dtype=np.uint8)   # the reader may look one word ahead
    padded[:payload.size] = payload
    out = np.empty(n, dtype=np.float32)
    p = (C.c_int32 * 4)(*prm)
    _load().ref_decompress(padded.ctypes.data, padded.size, out.ctypes.data, n, 0, p)
    return out
