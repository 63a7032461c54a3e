"""Compiles the CUDA sources under ``csrc/`` for sm_100a into one shared library and loads it.

The library is built at the first call and kept in ``csrc/_build`` inside the package (or,
when that folder cannot be written, in a per-user folder under the temporary directory).
A hash of the sources and flags beside it says whether it is current, so a copied tree with
new timestamps does not rebuild. There is no CPU fallback: if the library cannot be built
or loaded, the error is raised.
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
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libsmolmoe_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelBuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[smolmoe_c99_b200] {message}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def _source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _build_dir() -> str:
    override = os.environ.get("SMOLMOE_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    local = os.path.join(CSRC, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"smolmoe_c99_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _compile_one(nvcc: str, name: str, out_dir: str, verbose_ptxas: bool) -> str:
    obj = os.path.join(out_dir, name[:-3] + ".o")
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    started = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
    _say(f"compiled {name} in {time.time() - started:.1f} s")
    if verbose_ptxas:
        sys.stderr.write(proc.stderr)
    return obj


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Builds the library if it is missing or stale; returns its path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = lib_path + ".hash"
    want = _source_hash()
    if not force and os.path.exists(lib_path) and os.path.exists(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == want:
                return lib_path
    nvcc = _nvcc()
    names = sources()
    _say(f"building {len(names)} CUDA sources for sm_100a into {out_dir} (first call only)")
    started = time.time()
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as pool:
        objects = list(pool.map(lambda n: _compile_one(nvcc, n, out_dir, verbose_ptxas), names))
    tmp = lib_path + f".{os.getpid()}.tmp"
    # the CUDA runtime is linked statically (nvcc's default); driver entry points are looked
    # up at run time, so the library loads on a machine without a driver too
    link = [nvcc, "-shared", "-o", tmp, *objects]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib_path)
    with open(stamp_path, "w") as f:
        f.write(want + "\n")
    _say(f"built {LIB_NAME} in {time.time() - started:.1f} s")
    return lib_path


def load() -> ctypes.CDLL:
    """The loaded library (built first if needed)."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _lib.sm_last_error.restype = ctypes.c_char_p
        return _lib
