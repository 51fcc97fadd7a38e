"""Host-side tiling rules of the implicit-GEMM convolution (no GPU needed: the launcher's pixel-box search is
exported from the CUDA library and runs on the CPU)."""
import ctypes as C

import pytest


def _lib():
    from gcow_b200 import _native
    try:
        lib = _native.cuda()
    except Exception as e:          # the CUDA runtime library is not loadable on this machine
        pytest.skip(f"CUDA library not loadable: {e}")
    if not hasattr(lib, "gcow_conv_pick_box"):
        pytest.skip("library built without the convolution kernels")
    return lib


def _box(lib, W, H, N, rows, exact):
    out = (C.c_int * 3)()
    lib.gcow_conv_pick_box(W, H, N, rows, exact, out)
    return tuple(out)


@pytest.mark.parametrize("W,H,N", [(56, 56, 256), (28, 28, 256), (14, 14, 256), (7, 7, 256), (5, 3, 2), (1, 1, 1), (9, 7, 3)])
def test_pixel_box_fits_the_tile(W, H, N):
    lib = _lib()
    for rows in (128, 256):
        bw, bh, bn = _box(lib, W, H, N, rows, 0)
        assert 1 <= bw <= 256 and 1 <= bh <= 256 and 1 <= bn <= 256
        assert bw * bh * bn <= rows
    bw, bh, bn = _box(lib, W, H, N, 64, 1)
    assert bw * bh * bn == 64          # a reduction step of the weight gradient is exactly 64 pixels


def test_pixel_box_wastes_nothing_on_resnet_extents():
    lib = _lib()
    for W in (56, 28, 14, 7):
        bw, bh, bn = _box(lib, W, W, 256, 128, 0)
        covered = -(-W // bw) * bw * -(-W // bh) * bh * -(-256 // bn) * bn
        assert covered == W * W * 256 and bw * bh * bn == 128, (W, bw, bh, bn)
