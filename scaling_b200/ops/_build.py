"""Builds the native library of scaling_b200 in-tree with nvcc for sm_100a.

The CUDA sources under ``scaling_b200/csrc`` expose a plain C ABI (``extern "C"``) and are
compiled straight to ``scaling_b200/lib/libsb200.so``; Python loads it with ctypes and passes raw
device pointers plus the current CUDA stream.  No torch headers are involved, so a full rebuild
takes well under a minute and the same library serves callers that are not Python.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libsb200.so"
BUILD_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")
    return cand


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _digest(paths: list[Path]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def needs_build() -> bool:
    stamp = LIB_DIR / "libsb200.sha256"
    if not LIB_PATH.exists() or not stamp.exists():
        return True
    deps = sources() + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    return stamp.read_text().strip() != _digest(deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source for sm_100a and link ``libsb200.so``.  Returns the library path.

    Several ranks of one job may get here at the same time (fresh checkout, changed source): the build runs under
    an exclusive file lock, the check is repeated once the lock is held, and objects and the library are written
    under temporary names and moved into place, so that no process ever maps a half-written file."""
    if not force and not needs_build():
        return LIB_PATH
    import fcntl

    BUILD_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    with open(LIB_DIR / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():  # another process built it while this one waited
                return LIB_PATH
            return _build_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool) -> Path:
    nvcc = _nvcc()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    hdr_digest = _digest(headers)

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        stamp = BUILD_DIR / (src.stem + ".sha256")
        dig = hashlib.sha256((hdr_digest + _digest([src])).encode()).hexdigest()
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
            return obj
        tmp = obj.with_suffix(f".{os.getpid()}.tmp.o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(tmp)]
        if src.suffix == ".cpp":
            cmd.insert(1, "-x")
            cmd.insert(2, "cu")
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        os.replace(tmp, obj)
        stamp.write_text(dig)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    tmp_lib = LIB_DIR / f"libsb200.{os.getpid()}.tmp.so"
    cmd = [nvcc, "-shared", "-o", str(tmp_lib), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp_lib, LIB_PATH)  # a process that has the old file mapped keeps its inode
    deps = sources() + headers
    (LIB_DIR / "libsb200.sha256").write_text(_digest(deps))
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
