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


def test_streams_equal_the_reference_codec_behind_the_same_calls():
    """The stand-in `baseline/zfpy.py` serves the reference's training scripts from the REFERENCE's CPU codec. For the
    three call forms those scripts use, this library's stream (without its header) is byte for byte the same, and the
    reference's decoder reads it back to the same floats."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "baseline", "_ref", "libgcowref.so")):
        pytest.skip("reference library not built (baseline/build_ref.sh)")
    spec = importlib.util.spec_from_file_location("ref_zfpy", os.path.join(root, "baseline", "zfpy.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    rng = np.random.default_rng(1)
    g = (rng.standard_normal(4097) * 1e-3).astype(np.float32)
    for kw in ({"rate": 8}, {"rate": 16}, {"tolerance": 1e-6}, {"precision": 12}):
        mine = zfpy.compress_numpy(g, write_header=False, **kw)
        theirs = ref.compress_numpy(g, **kw)[ref._HDR.size:]
        n = min(len(mine), len(theirs))
        assert n > 0 and mine[:n] == theirs[:n] and not any(mine[n:]) and not any(theirs[n:]), kw
        a = zfpy.decompress_numpy(zfpy.compress_numpy(g, **kw))
        b = ref.decompress_numpy(ref.compress_numpy(g, **kw))
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), kw


def test_reference_arm_answers_without_a_gpu():
    """`bench.py --impl reference` on a machine without CUDA prints one JSON line with `unavailable` and exits 0."""
    import json
    import os
    import subprocess
    import sys
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the arm would run the reference's training loop")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=root)
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec
