"""Loader for the reference CPU codec shim (baseline/_ref/libgcowref.so).

The library is the unmodified reference sw/src/*.c plus baseline/ref_driver.cpp;
it is built by baseline/build_ref.sh when a reference checkout is present and is
simply absent otherwise (tests that need it skip)."""
import ctypes as C
import os
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SO = ROOT / "baseline" / "_ref" / "libgcowref.so"
REF = Path(os.environ.get("GCOW_REFERENCE", str(ROOT.parent / "reference")))   # a checkout beside this repository

_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not SO.exists() and (REF / "sw" / "src" / "zfp.c").exists():
        subprocess.run([str(ROOT / "baseline" / "build_ref.sh"), str(REF)], check=True,
                       capture_output=True)
    if not SO.exists():
        return None
    lib = C.CDLL(str(SO))
    u64, i32, ptr = C.c_uint64, C.c_int, C.c_void_p
    lib.ref_compress_2d.restype = u64
    lib.ref_compress_2d.argtypes = [ptr, u64, u64, ptr, ptr, u64]
    lib.ref_compress_1d.restype = u64
    lib.ref_compress_1d.argtypes = [ptr, u64, ptr, ptr, u64]
    lib.ref_decompress.restype = None
    lib.ref_decompress.argtypes = [ptr, u64, ptr, u64, u64, ptr]
    lib.ref_set_accuracy.restype = None
    lib.ref_set_accuracy.argtypes = [C.c_double, ptr]
    lib.ref_stage_emax.restype = i32
    lib.ref_stage_emax.argtypes = [ptr, i32]
    lib.ref_stage_cast.restype = None
    lib.ref_stage_cast.argtypes = [ptr, ptr, i32, i32]
    lib.ref_stage_xform.restype = None
    lib.ref_stage_xform.argtypes = [ptr, i32]
    lib.ref_stage_reorder.restype = None
    lib.ref_stage_reorder.argtypes = [ptr, ptr, i32]
    lib.ref_get_precision.restype = C.c_uint32
    lib.ref_get_precision.argtypes = [i32, C.c_uint32, i32, i32]
    _lib = lib
    return lib


def compress(x, params, dim):
    """x: contiguous float32 numpy array; returns bytes."""
    import numpy as np
    lib = load()
    p = (C.c_int32 * 4)(*params)
    if dim == 2:
        ny, nx = x.shape
        blocks = ((nx + 3) // 4) * ((ny + 3) // 4)
    else:
        nx, ny = x.size, 0
        blocks = (nx + 3) // 4
    cap = (blocks * min(params[1], 9 + 15 + 16 * 32) + 148 + 63) // 64 * 8 + 64
    out = np.zeros(cap, dtype=np.uint8)
    if dim == 2:
        n = lib.ref_compress_2d(x.ctypes.data, nx, ny, p, out.ctypes.data, cap)
    else:
        n = lib.ref_compress_1d(x.ctypes.data, nx, p, out.ctypes.data, cap)
    return out[:n].tobytes()


def decompress(stream, shape, params):
    import numpy as np
    lib = load()
    p = (C.c_int32 * 4)(*params)
    buf = np.zeros(len(stream) + 16, dtype=np.uint8)
    buf[:len(stream)] = np.frombuffer(stream, dtype=np.uint8)
    out = np.zeros(shape, dtype=np.float32)
    if len(shape) == 2:
        lib.ref_decompress(buf.ctypes.data, buf.size, out.ctypes.data, shape[1], shape[0], p)
    else:
        lib.ref_decompress(buf.ctypes.data, buf.size, out.ctypes.data, shape[0], 0, p)
    return out
