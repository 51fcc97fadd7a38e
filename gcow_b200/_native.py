"""ctypes access to the two native libraries (see build.py).

``cpu()`` is always available (built on demand with g++). ``cuda()`` returns the
sm_100a kernel library; on a machine with a GPU a missing library is an error,
never a silent fallback to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from . import build as _build

_lock = threading.Lock()
_cpu = None
_cuda = None

u64, u32, i32, f64 = C.c_uint64, C.c_uint32, C.c_int, C.c_double
ptr = C.c_void_p


def _proto(lib, name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


def cpu() -> C.CDLL:
    global _cpu
    with _lock:
        if _cpu is None:
            lib = C.CDLL(str(_build.build_cpu()))
            _proto(lib, "gcow_params_rate", None, f64, i32, ptr)
            _proto(lib, "gcow_params_accuracy", None, f64, ptr)
            _proto(lib, "gcow_params_precision", None, u32, ptr)
            _proto(lib, "gcow_max_output_bytes", u64, ptr, u64, u64)
            _proto(lib, "gcow_block_precision", u32, i32, u32, i32, i32)
            _proto(lib, "gcow_oracle_compress", u64, ptr, u64, u64, ptr, ptr, ptr, i32)
            _proto(lib, "gcow_oracle_decompress", u64, ptr, ptr, u64, u64, ptr, i32, i32)
            _proto(lib, "gcow_header_compress", u64, ptr, u64, u64, ptr, ptr)
            _proto(lib, "gcow_header_decompress", u64, ptr, ptr, u64, u64, ptr, i32)
            _proto(lib, "gcow_fast1d_compress", i32, ptr, u64, ptr, ptr)
            _proto(lib, "gcow_fast1d_decompress", i32, ptr, ptr, u64, ptr, i32)
            _proto(lib, "gcow_lean_accuracy_check", C.c_int64, ptr, u64, i32, i32, ptr)
            _proto(lib, "gcow_stage_emax", i32, ptr, i32, i32)
            _proto(lib, "gcow_stage_cast", None, ptr, ptr, i32, i32, i32)
            _proto(lib, "gcow_stage_inv_cast", None, ptr, ptr, i32, i32, i32, i32)
            _proto(lib, "gcow_stage_xform", None, ptr, i32, i32, i32)
            _proto(lib, "gcow_stage_reorder", None, ptr, ptr, i32, i32)
            _proto(lib, "gcow_stage_inv_reorder", None, ptr, ptr, i32, i32)
            _proto(lib, "gcow_stage_encode_planes", u64, ptr, i32, u32, u32, i32, i32, ptr, i32)
            _proto(lib, "gcow_stage_decode_planes", u32, ptr, u64, ptr, i32, u32, u32, i32)
            _proto(lib, "gcow_stage_stream_write", u64, ptr, ptr, i32, ptr, i32)
            _proto(lib, "gcow_stage_gather", None, ptr, u64, u64, u64, ptr)
            _proto(lib, "gcow_oracle_allreduce", None, ptr, i32, u64, ptr, i32, i32, ptr, i32)
            _proto(lib, "gcow_protocol_model", i32, ptr, ptr, i32, u64, i32, i32, i32, i32, i32, i32, i32,
                   i32, i32, i32, i32, i32, i32, i32, ptr)
            _proto(lib, "gcow_protocol_model2", i32, ptr, ptr, i32, u64, i32, i32, i32, i32, i32, i32, i32,
                   i32, i32, i32, i32, i32, i32, i32, ptr, i32)
            _cpu = lib
    return _cpu


def cuda_available() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def cuda() -> C.CDLL:
    """The sm_100a kernel library. Raises if it cannot be built or loaded."""
    global _cuda
    with _lock:
        if _cuda is None:
            so = _build.build_cuda()
            if so is None or not Path(so).exists():
                raise RuntimeError("libgcow_cuda.so is missing and nvcc is not available to build it")
            lib = C.CDLL(str(so))
            from . import _cuda_protos
            _cuda_protos.declare(lib, _proto)
            _cuda = lib
    return _cuda
