"""Ahead-of-time build of the native library (CUDA kernels + C++ runtime) for sm_100a.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into an
object file and linked into ``kraken_b200/_C/libkraken_b200.so`` in the source tree, so the
library travels with the checkout and no JIT cache is involved. A source hash stored next to the
library makes rebuilds incremental. nvcc cross-compiles without a GPU.

``build(debug=True)`` compiles the same sources with ``-DKRAKEN_DEBUG=1`` into
``libkraken_b200_debug.so``: every kernel then checks the indices it derives (tile counters, slab
rows, chunk and slot offsets) and, instead of touching memory out of bounds, records
``KR_ERR_BOUNDS`` in the device status word and skips the access. ``KRAKEN_DEBUG=1`` makes
``kraken_b200.ops.lib`` load that library.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
CSRC = REPO / "csrc"
OUT_DIR = REPO / "kraken_b200" / "_C"
LIB_PATH = OUT_DIR / "libkraken_b200.so"
DEBUG_LIB_PATH = OUT_DIR / "libkraken_b200_debug.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]
INCLUDE_FLAG = f"-I{CSRC / 'include'}"      # absolute path: kept out of the staleness digest


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")


def lib_path(debug: bool = False) -> Path:
    return DEBUG_LIB_PATH if debug else LIB_PATH


def _headers_digest(debug: bool = False) -> str:
    h = hashlib.sha256()
    h.update(b"debug" if debug else b"release")
    for p in sorted((CSRC / "include").rglob("*")):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _source_digest(src: Path, headers: str) -> str:
    h = hashlib.sha256()
    h.update(headers.encode())
    h.update(src.read_bytes())
    return h.hexdigest()


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(verbose: bool = False, force: bool = False, debug: bool = False) -> Path:
    """Compiles what changed and links the shared library. Returns its path. Safe to call from
    several processes at once (ranks of one job): an exclusive file lock serialises them and the
    library is replaced atomically, so nobody ever loads a half-written file."""
    import fcntl

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    with open(OUT_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale(debug):
                return lib_path(debug)
            return _build_locked(verbose, force, debug)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose: bool, force: bool, debug: bool = False) -> Path:
    nvcc = _nvcc()
    headers = _headers_digest(debug)
    tag = ".dbg" if debug else ""
    extra = ["-DKRAKEN_DEBUG=1"] if debug else []
    target = lib_path(debug)
    jobs = []
    objects = []
    for src in sources():
        obj = OUT_DIR / (src.stem + tag + ".o")
        stamp = OUT_DIR / (src.stem + tag + ".hash")
        digest = _source_digest(src, headers)
        objects.append(obj)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == digest:
            continue
        jobs.append((src, obj, stamp, digest))

    def compile_one(job):
        src, obj, stamp, digest = job
        cmd = [nvcc, *NVCC_FLAGS, *extra, INCLUDE_FLAG, "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        stamp.write_text(digest)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not target.exists():
        tmp = target.with_suffix(f".so.tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objects), "-Xcompiler", "-fPIC", "-lpthread"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, target)
    return target


def is_stale(debug: bool = False) -> bool:
    if not lib_path(debug).exists():
        return True
    headers = _headers_digest(debug)
    tag = ".dbg" if debug else ""
    for src in sources():
        stamp = OUT_DIR / (src.stem + tag + ".hash")
        if not stamp.exists() or stamp.read_text() != _source_digest(src, headers):
            return True
    return False


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv, debug="--debug" in sys.argv))
