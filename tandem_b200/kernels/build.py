"""Compile the CUDA sources under ``tandem_b200/csrc`` for sm_100a and load them.

Each ``.cu`` file becomes one shared library of plain C entry points, built with nvcc at first
use and kept under ``tandem_b200/csrc/_build`` (or, when the checkout is read-only, under a
per-user folder in the system's temporary directory).  The file name carries a hash of the
sources and flags, so an edited kernel is rebuilt and a stale library is never loaded.  There
is no fallback: a missing compiler or a failed build raises.

12vivi/tandem compiles its two ``.cu`` files at first use as well, through
``torch.utils.cpp_extension.load_inline`` (python/tandem/cache/kv_io.py:29-39).
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]

_lock = threading.RLock()
_loaded: dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("TANDEM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $TANDEM_NVCC, PATH and /usr/local/cuda/bin): "
                           "the CUDA kernels cannot be built and there is no other path")


_build_dir = None


def build_dir() -> str:
    """In the tree when it can be written, else a per-user folder in the temporary directory."""
    global _build_dir
    with _lock:
        if _build_dir is None:
            d = os.path.join(CSRC, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(dir=d)
                os.close(fd)
                os.remove(probe)
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"tandem_b200_build_{os.getuid()}")
                os.makedirs(d, exist_ok=True)
            _build_dir = d
        return _build_dir


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(source: str, defines: tuple) -> str:
    h = hashlib.sha256()
    for path in [source] + _headers():
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read())
    h.update(repr((ARCH_FLAGS, BASE_FLAGS, defines)).encode())
    return h.hexdigest()[:16]


def library_path(stem: str, defines: tuple = ()) -> str:
    source = os.path.join(CSRC, stem + ".cu")
    tag = "".join(f"_{d.replace('=', '')}" for d in defines)
    return os.path.join(build_dir(), f"tb_{stem}{tag}_{_digest(source, defines)}.so")


def compile_library(stem: str, defines: tuple = (), verbose: bool = True) -> str:
    """Build ``csrc/<stem>.cu`` (if its library is not there yet) and return the library's path."""
    out = library_path(stem, defines)
    if os.path.isfile(out):
        return out
    source = os.path.join(CSRC, stem + ".cu")
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *[f"-D{d}" for d in defines], "-I", CSRC, "-o", tmp, source]
    if verbose:
        print(f"[tandem_b200] compiling {stem}.cu {' '.join(defines)} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[tandem_b200]   still compiling {stem}.cu ({time.time() - t0:.0f} s)", file=sys.stderr,
                      flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed for {stem}.cu:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    if verbose:
        print(f"[tandem_b200]   built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def compile_many(jobs: list, verbose: bool = True) -> list[str]:
    """jobs: [(stem, defines)] compiled side by side."""
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        return list(pool.map(lambda j: compile_library(j[0], tuple(j[1]), verbose), jobs))


def load_library(stem: str, defines: tuple = ()) -> ctypes.CDLL:
    key = stem + "|" + ",".join(defines)
    lib = _loaded.get(key)
    if lib is None:
        path = compile_library(stem, defines)
        with _lock:
            lib = _loaded.setdefault(key, ctypes.CDLL(path))
    return lib
