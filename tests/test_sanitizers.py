"""Host-side sanitizer runs of the code shared between CPU and GPU (block codec,
arena layout, flag protocol): AddressSanitizer + UBSan, and ThreadSanitizer on the
thread model of the all-reduce."""
import os
import subprocess

import pytest

from gcow_b200 import build


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_sanitized_driver_is_clean(kind):
    try:
        exe = build.build_sanitizer_test(kind)
    except RuntimeError as e:
        pytest.skip(f"sanitizer runtime not available: {e}")
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=1")
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    out = proc.stdout + proc.stderr
    assert proc.returncode == 0, out[-3000:]
    assert "sanitize_main: ok" in out
    assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out and "runtime error" not in out
