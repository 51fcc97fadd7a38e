"""The zfpy-style entry points used by the reference's training studies (hw/models/train_imagenet.py:459-465)."""
import numpy as np
import pytest

import gcow_b200.zfpy_compat as zfpy


def test_rate_roundtrip_flat_gradient():
    rng = np.random.default_rng(0)
    g = (rng.standard_normal(10_001) * 1e-3).astype(np.float32)
    buf = zfpy.compress_numpy(g, rate=16)
    assert isinstance(buf, bytes) and len(buf) < g.nbytes * 0.55
    back = zfpy.decompress_numpy(buf)
    assert back.shape == g.shape and back.dtype == np.float32
    assert np.abs(back - g).max() < 2e-5                   # values of about 1e-3 at 16 bits each
    rough = zfpy.decompress_numpy(zfpy.compress_numpy(g, rate=4))
    assert np.abs(back - g).max() < np.abs(rough - g).max() < 1e-2          # lossier, but bounded


def test_tolerance_and_precision_modes():
    rng = np.random.default_rng(1)
    g = rng.standard_normal(4096).astype(np.float32)
    for tol in (1e-1, 1e-3, 1e-6):
        back = zfpy.decompress_numpy(zfpy.compress_numpy(g, tolerance=tol))
        assert np.abs(back - g).max() <= tol
    coarse = zfpy.decompress_numpy(zfpy.compress_numpy(g, precision=8))
    fine = zfpy.decompress_numpy(zfpy.compress_numpy(g, precision=24))
    assert np.abs(fine - g).max() < np.abs(coarse - g).max()
    default = zfpy.decompress_numpy(zfpy.compress_numpy(g))
    assert np.abs(default - g).max() < 1e-6


def test_two_dimensional_arrays_use_4x4_blocks_and_keep_their_shape():
    x = np.linspace(0, 1, 37 * 53, dtype=np.float32).reshape(37, 53)
    back = zfpy.decompress_numpy(zfpy.compress_numpy(x, tolerance=1e-4))
    assert back.shape == (37, 53) and np.abs(back - x).max() <= 1e-4
    cube = np.arange(2 * 3 * 5, dtype=np.float32).reshape(2, 3, 5)
    flat = zfpy.decompress_numpy(zfpy.compress_numpy(cube, rate=32))
    assert flat.shape == (30,) and np.allclose(flat, cube.reshape(-1), atol=1e-4)


def test_argument_checks():
    g = np.zeros(16, dtype=np.float32)
    with pytest.raises(ValueError):
        zfpy.compress_numpy(g, rate=8, tolerance=1e-3)
    with pytest.raises(TypeError):
        zfpy.compress_numpy(g.astype(np.float64), rate=8)
    with pytest.raises(ValueError):
        zfpy.decompress_numpy(zfpy.compress_numpy(g, rate=8, write_header=False))
