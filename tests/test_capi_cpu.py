"""The host library used from plain C through csrc/include/gcow.h, like the reference's sw/ library is used
through zfp.h: compile csrc/tests/capi_main.c, compress the reference field, compare with the golden stream."""
import shutil
import subprocess
from pathlib import Path

import pytest

import refcodec

ROOT = Path(__file__).resolve().parents[1]


def test_c_program_reproduces_golden_stream(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    gold = refcodec.REF / "sw" / "tests" / "data" / "compressed_2d_100.zfp"
    if cc is None or not gold.exists():
        pytest.skip("needs a C compiler and the reference's golden data")
    from gcow_b200 import _native
    _native.cpu()                                            # makes sure libgcow_cpu.so is built
    lib = ROOT / "gcow_b200" / "_lib"
    exe = tmp_path / "capi_main"
    subprocess.run([cc, "-std=c99", "-O1", f"-I{ROOT / 'gcow_b200' / 'csrc' / 'include'}",
                    str(ROOT / "gcow_b200" / "csrc" / "tests" / "capi_main.c"), "-o", str(exe), f"-L{lib}", "-lgcow_cpu",
                    "-lm", f"-Wl,-rpath,{lib}"], check=True, capture_output=True)
    r = subprocess.run([str(exe), "100", str(gold)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "bytes 4536" in r.stdout
