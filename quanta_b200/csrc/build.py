"""Compile the CUDA sources of this folder for sm_100a into one shared library and load it.

The library is plain C ABI (raw device pointers and a stream), so it compiles in seconds per file
with nvcc alone and is loaded with ctypes.  It is built in-tree under ``csrc/_build`` when that is
writable (an already-built library travels with the folder), else under ``$QUANTA_B200_BUILD_DIR``
or a per-user folder of the temporary directory.  Nothing is fetched; a missing compiler or a
failed build raises: there is no fallback path.

A build is reused while the hash of all sources and flags matches the one stored beside it.
"""

from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
LIB_NAME = "libquanta_b200_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[quanta_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list(SRC_DIR.glob("*.cu")) + list(SRC_DIR.glob("*.cuh")) + list(SRC_DIR.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH, /usr/local/cuda/bin): the CUDA kernels "
                           "cannot be built, and there is no other execution path")


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("QUANTA_B200_BUILD_DIR")
    if env:
        d = Path(env)
        if not _writable(d):
            raise KernelBuildError(f"QUANTA_B200_BUILD_DIR={env} is not writable")
        return d
    d = SRC_DIR / "_build"
    if _writable(d):
        return d
    d = Path(tempfile.gettempdir()) / f"quanta_b200_build_{os.getuid()}"
    if _writable(d):
        return d
    raise KernelBuildError("no writable folder for the kernel build (tried csrc/_build and the temp folder)")


def _up_to_date(d: Path, fp: str) -> bool:
    stamp = d / "fingerprint.txt"
    return (d / LIB_NAME).exists() and stamp.exists() and stamp.read_text().strip() == fp


def build(verbose: bool = True, force: bool = False) -> Path:
    """Build (if needed) and return the path of the shared library."""
    fp = _fingerprint()
    # a library built in-tree is used even when the tree itself is read-only
    intree = SRC_DIR / "_build"
    if not force and _up_to_date(intree, fp):
        return intree / LIB_NAME
    d = build_dir()
    if not force and _up_to_date(d, fp):
        return d / LIB_NAME
    nvcc = _find_nvcc()
    srcs = sources()
    if verbose:
        _log(f"compiling {len(srcs)} CUDA files for sm_100a into {d} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            _log(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()

    def compile_one(src: Path) -> Path:
        obj = d / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _log(f"compiled {src.name} ({time.time() - t0:.0f} s)")
        return obj

    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = d / (LIB_NAME + f".tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, d / LIB_NAME)
        (d / "fingerprint.txt").write_text(fp)
    finally:
        done.set()
    if verbose:
        _log(f"kernels built in {time.time() - t0:.0f} s")
    return d / LIB_NAME


_LIB = None


def load() -> ctypes.CDLL:
    """The loaded kernel library; built on first use."""
    global _LIB
    if _LIB is None:
        path = build()
        try:
            _LIB = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from e
    return _LIB
