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


def test_forward_tile_choice_on_resnet_layers():
    """The launcher's cost model picks 256-pixel tiles where they were measured faster (64, 128 and 512 channels at
    batch 256 on 148 SMs) and 128-pixel tiles at 256 channels, where two 256-column accumulators would fill the
    tensor memory and a second wave would be mostly empty."""
    lib = _lib()
    if not hasattr(lib, "gcow_conv_fwd_plan"):
        pytest.skip("library built without the plan export")
    want = {64: (2, 64), 128: (2, 128), 256: (1, 256), 512: (2, 256)}
    for (ch, hw) in ((64, 56), (128, 28), (256, 14), (512, 7)):
        out = (C.c_int * 6)()
        lib.gcow_conv_fwd_plan(256, hw, hw, ch, ch, 3, 3, 1, 1, 148, out)
        halves, cols, bw, bh, bn, stages = list(out)
        assert (halves, cols) == want[ch], (ch, list(out))
        assert bw * bh * bn <= 128 * halves and 2 <= stages <= 8


def test_special_3x3_kernels_take_the_shapes_they_fit():
    """The weight-stationary, halo-tile weight-gradient and halo-tile forward kernels state on the host which extents
    they take: rows that fit their slot pitch, tiles that fit the shared memory."""
    lib = _lib()
    if not hasattr(lib, "gcow_conv_halo_usable"):
        pytest.skip("library built without the halo-tile kernels")
    # weight-stationary forward (64 -> 64): any image whose rows plus halo fit 128 slots, at least 6 pixels wide
    assert lib.gcow_conv_ws_usable(256, 56, 56) and lib.gcow_conv_ws_usable(1, 1, 6) and lib.gcow_conv_ws_usable(2, 9, 126)
    assert not lib.gcow_conv_ws_usable(2, 9, 127) and not lib.gcow_conv_ws_usable(2, 9, 5) and not lib.gcow_conv_ws_usable(0, 9, 9)
    # halo-tile weight gradient: slot pitch 64, one partial result per CTA, never more CTAs than SMs, none empty
    assert lib.gcow_conv_wgrad_ws_split(2, 9, 63) == 0 and lib.gcow_conv_wgrad_ws_split(0, 9, 9) == 0
    for (N, H, W) in ((256, 56, 56), (3, 30, 20), (1, 7, 9), (1, 1, 1), (1000, 5, 62)):
        split = lib.gcow_conv_wgrad_ws_split(N, H, W)
        tiles = N * -(-H // 4)
        per = -(-tiles // split)
        assert 1 <= split <= max(1, min(tiles, 148)) and (split - 1) * per < tiles <= split * per, (N, H, W, split)
    # halo-tile forward (Ci -> 128): two pixel stages of all 64-channel chunks plus three filter stages must fit
    assert lib.gcow_conv_halo_usable(256, 28, 28, 128) and lib.gcow_conv_halo_usable(256, 28, 28, 64)
    assert lib.gcow_conv_halo_usable(1, 5, 6, 192)
    assert not lib.gcow_conv_halo_usable(256, 28, 28, 512) and not lib.gcow_conv_halo_usable(256, 14, 14, 256)
    assert not lib.gcow_conv_halo_usable(256, 28, 28, 96) and not lib.gcow_conv_halo_usable(4, 8, 127, 64)
