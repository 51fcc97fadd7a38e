"""In-tree native build: plain g++/nvcc commands, no JIT cache.

Two shared libraries are produced next to this file, under ``_lib/``:

* ``libgcow_cpu.so``  – CPU oracle, host model of the flag protocol (g++ only).
* ``libgcow_cuda.so`` – every sm_100a kernel plus its C launchers (nvcc).

Both export a C ABI and are loaded with ctypes, so building needs neither the
PyTorch headers nor a GPU (nvcc cross-compiles). A content hash of the sources
is stored beside each library; an up-to-date library is never rebuilt, which is
what lets a prebuilt tree run on a machine without recompiling.

The reference drives its builds from make variables (hw/Makefile:30-36,
sw/Makefile:4-5); this is the equivalent single entry point.
"""
from __future__ import annotations

import contextlib
import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC",
    # exact float semantics matter for the codec: no fast-math, no flush-to-zero
    "-ftz=false", "-prec-div=true", "-prec-sqrt=true", "-fmad=true",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-pthread"]


def _sources(kind: str) -> list[Path]:
    if kind == "cpu":
        return sorted(p for p in CSRC.rglob("*.cpp") if "tests" not in p.parts)
    return sorted(CSRC.rglob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")))


def _digest(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for f in files:
        h.update(str(f.relative_to(ROOT)).encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _stamp_path(name: str) -> Path:
    return LIB / f"{name}.stamp.json"


def _up_to_date(name: str, digest: str) -> bool:
    so, st = LIB / f"{name}.so", _stamp_path(name)
    if not so.exists() or not st.exists():
        return False
    try:
        return json.loads(st.read_text()).get("digest") == digest
    except Exception:
        return False


def _run(cmd: list[str], log: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        raise RuntimeError(f"native build failed: {cmd[0]} exited {proc.returncode}")


@contextlib.contextmanager
def _build_lock():
    """Exclusive lock for builds: with one process per GPU every rank may find a stale tree at the same time, and
    they all write the same object files and libraries. The first rank in builds; the others wait here, then find
    the stamp up to date. Outputs are written under a temporary name and renamed, so a reader never maps a
    half-written library."""
    LIB.mkdir(exist_ok=True)
    with open(LIB / ".lock", "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def _replace_text(path: Path, text: str) -> None:
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    tmp.write_text(text)
    os.replace(tmp, path)


def build_cpu(force: bool = False, sanitize: str | None = None) -> Path:
    """Build libgcow_cpu.so; ``sanitize`` in {None, 'address', 'thread'} builds a
    separately named instrumented copy for the host-side race/memory checks."""
    LIB.mkdir(exist_ok=True)
    name = "libgcow_cpu" + (f"_{sanitize}" if sanitize else "")
    srcs = _sources("cpu")
    flags = list(CXX_FLAGS)
    if sanitize:
        flags += [f"-fsanitize={sanitize}", "-g", "-fno-omit-frame-pointer"]
    digest = _digest(srcs + _headers(), flags)
    if not force and _up_to_date(name, digest):
        return LIB / f"{name}.so"
    with _build_lock():
        if not force and _up_to_date(name, digest):      # another process built it while this one waited
            return LIB / f"{name}.so"
        inc = [f"-I{CSRC}", f"-I{CSRC / 'codec'}"]
        tmp = LIB / f"{name}.so.tmp{os.getpid()}"
        _run(["g++", *flags, *inc, "-shared", "-x", "c++", *map(str, srcs), "-o", str(tmp)])
        os.replace(tmp, LIB / f"{name}.so")
        _replace_text(_stamp_path(name), json.dumps({"digest": digest}))
    return LIB / f"{name}.so"


def build_cuda(force: bool = False, jobs: int | None = None) -> Path | None:
    """Compile every .cu for sm_100a and link libgcow_cuda.so. Returns None when
    nvcc is not installed and no prebuilt library exists."""
    LIB.mkdir(exist_ok=True)
    name = "libgcow_cuda"
    srcs = _sources("cuda")
    digest = _digest(srcs + _headers(), NVCC_FLAGS)
    if not force and _up_to_date(name, digest):
        return LIB / f"{name}.so"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        so = LIB / f"{name}.so"
        return so if so.exists() else None
    with _build_lock():
        if not force and _up_to_date(name, digest):
            return LIB / f"{name}.so"
        return _build_cuda_locked(force, jobs, name, srcs, digest, nvcc)


def _build_cuda_locked(force, jobs, name, srcs, digest, nvcc) -> Path:
    obj = LIB / "obj"
    obj.mkdir(exist_ok=True)
    inc = [f"-I{CSRC}", f"-I{CSRC / 'codec'}"]

    def one(src: Path) -> Path:
        o = obj / (src.stem + ".o")
        d = _digest([src] + _headers(), NVCC_FLAGS)
        st = obj / (src.stem + ".stamp")
        if not force and o.exists() and st.exists() and st.read_text() == d:
            return o
        tmp = obj / (src.stem + f".o.tmp{os.getpid()}")
        _run([nvcc, *NVCC_FLAGS, *inc, "-c", str(src), "-o", str(tmp)], log=obj / (src.stem + ".ptxas.log"))
        os.replace(tmp, o)
        _replace_text(st, d)
        return o

    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(one, srcs))
    tmp = LIB / f"{name}.so.tmp{os.getpid()}"
    _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *map(str, objs),
          "-o", str(tmp), "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    os.replace(tmp, LIB / f"{name}.so")
    _replace_text(_stamp_path(name), json.dumps({"digest": digest}))
    return LIB / f"{name}.so"


def build_sanitizer_test(kind: str) -> Path:
    """Executable of csrc/tests/sanitize_main.cpp + the CPU sources under a sanitizer:
    kind = 'address' (with undefined-behaviour checks) or 'thread'."""
    LIB.mkdir(exist_ok=True)
    exe = LIB / f"sanitize_{kind}"
    srcs = _sources("cpu") + [CSRC / "tests" / "sanitize_main.cpp"]
    san = "address,undefined" if kind == "address" else "thread"
    flags = ["-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={san}", "-fno-sanitize-recover=all",
             "-pthread"]
    digest = _digest(srcs + _headers(), flags)
    st = LIB / f"sanitize_{kind}.stamp"
    if exe.exists() and st.exists() and st.read_text() == digest:
        return exe
    inc = [f"-I{CSRC}", f"-I{CSRC / 'codec'}"]
    _run(["g++", *flags, *inc, "-x", "c++", *map(str, srcs), "-o", str(exe)])
    st.write_text(digest)
    return exe


def build_all(force: bool = False) -> None:
    build_cpu(force)
    build_cuda(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", *(p.name for p in sorted(LIB.glob("*.so"))))
