"""The allocation-free encoder entry point (csrc/codec/gcow_static_api.h).

Some users of the library cannot allocate device memory at the point where they
need to compress: all of it may already belong to a memory pool, the implicit
synchronisation of an allocation may be unaffordable, or the embedding code may
only pass on buffers it was handed. For them the library keeps an 8 MiB scratch
array of its own. This test drives that entry point through its exported C
symbol, twice in a row with different inputs (the second call finds the first
call's leftovers in the shared scratch), and requires the very same bytes and
block offsets that the regular entry point produces with caller-owned scratch.
It also checks that an oversized request is refused with a message rather than
launched. The file sorts last so that a run stopping at the first failure has
already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gcow_b200 import _native
from gcow_b200.codec import ZfpParams, max_compressed_nbytes

pytestmark = pytest.mark.gpu

u64, i32, ptr = C.c_uint64, C.c_int, C.c_void_p


def _symbols():
    lib = _native.cuda()
    f = lib.gcow_encode_generic_static
    f.restype = i32
    f.argtypes = [ptr, u64, u64, ptr, ptr, u64, ptr, ptr]
    lib.gcow_encode_generic_static_capacity.restype = u64
    lib.gcow_encode_generic_static_capacity.argtypes = []
    lib.gcow_encode_generic_static_error.restype = C.c_char_p
    lib.gcow_encode_generic_static_error.argtypes = []
    return lib


def _regular(lib, x, nx, ny, p, blocks, cap):
    dim = 2 if ny else 1
    scratch = torch.empty(lib.gcow_encode_generic_scratch_bytes(p.as_c(), blocks, dim), dtype=torch.uint8, device="cuda")
    out = torch.full((cap,), 0x5a, dtype=torch.uint8, device="cuda")
    idx = torch.empty(blocks + 1, dtype=torch.int64, device="cuda")
    rc = lib.gcow_encode_generic(x.data_ptr(), nx, ny, p.as_c(), out.data_ptr(), cap, scratch.data_ptr(),
                                 idx.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out, idx


def _static(lib, x, nx, ny, p, blocks, cap):
    out = torch.full((cap,), 0xa5, dtype=torch.uint8, device="cuda")
    idx = torch.empty(blocks + 1, dtype=torch.int64, device="cuda")
    rc = lib.gcow_encode_generic_static(x.data_ptr(), nx, ny, p.as_c(), out.data_ptr(), cap, idx.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.gcow_encode_generic_static_error().decode()
    return out, idx


def test_static_scratch_entry_matches_regular_entry_twice():
    lib = _symbols()
    rng = np.random.default_rng(3)
    cases = [
        # (array, dim, params): variable-rate 2-D first, then a smaller 1-D odd-rate call
        ((rng.standard_normal((300, 517)) * 3).astype(np.float32), 2, ZfpParams.from_accuracy(1e-3)),
        ((rng.standard_normal(40001) * 1e-3).astype(np.float32), 1, ZfpParams.from_rate(3, 1)),
    ]
    for arr, dim, p in cases:
        x = torch.from_numpy(arr).cuda()
        if dim == 2:
            ny, nx = arr.shape
            blocks = ((nx + 3) // 4) * ((ny + 3) // 4)
        else:
            nx, ny = arr.size, 0
            blocks = (nx + 3) // 4
        cap = max_compressed_nbytes(tuple(arr.shape), p)
        want, want_idx = _regular(lib, x, nx, ny, p, blocks, cap)
        got, got_idx = _static(lib, x, nx, ny, p, blocks, cap)
        torch.cuda.synchronize()
        assert torch.equal(got_idx, want_idx)
        nbytes = ((int(want_idx[-1]) + 63) // 64) * 8
        assert nbytes > 0
        assert torch.equal(got[:nbytes], want[:nbytes])      # exact: the codec tests compare bytes, not tolerances
        assert int(got[nbytes:].max()) == 0 if nbytes < cap else True


def test_static_scratch_entry_refuses_oversized_requests():
    lib = _symbols()
    p = ZfpParams.from_accuracy(1e-6)
    nx = ny = 4096                      # 1M blocks x 9 words: far beyond 8 MiB
    blocks = (nx // 4) * (ny // 4)
    assert lib.gcow_encode_generic_scratch_bytes(p.as_c(), blocks, 2) > lib.gcow_encode_generic_static_capacity()
    x = torch.zeros(16, device="cuda")  # never read: the call must refuse before launching
    out = torch.zeros(64, dtype=torch.uint8, device="cuda")
    idx = torch.zeros(8, dtype=torch.int64, device="cuda")
    rc = lib.gcow_encode_generic_static(x.data_ptr(), nx, ny, p.as_c(), out.data_ptr(), 64, idx.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    msg = lib.gcow_encode_generic_static_error().decode()
    assert "scratch" in msg and "8388608" in msg
    torch.cuda.synchronize()
