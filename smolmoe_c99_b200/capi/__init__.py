"""The C interface of the library (``engine.h``): built with the machine's C compiler at first use, like the kernels.

    from smolmoe_c99_b200.capi import build
    path = build()          # .../capi/_build/libsmolmoe_engine.so

A C program includes ``engine.h``, links this library and ``libpython`` (``python3-config --embed --ldflags``) and,
if its interpreter is not the one the packages were installed for, sets ``PYTHONPATH`` to their folder."""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libsmolmoe_engine.so"


class CapiBuildError(RuntimeError):
    pass


def header() -> str:
    return os.path.join(HERE, "engine.h")


def _build_dir() -> str:
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"smolmoe_c99_b200_capi_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def build(force: bool = False) -> str:
    """Compiles ``engine_capi.c`` into a shared library (Python symbols are left to the process that loads it: a
    Python program has them, a C program links libpython) and returns its path."""
    out_dir = _build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    h = hashlib.sha256()
    for name in ("engine_capi.c", "engine.h"):
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    include = sysconfig.get_config_var("INCLUDEPY")
    h.update(str(include).encode())
    stamp = lib + ".hash"
    if not force and os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read().strip() == h.hexdigest():
        return lib
    cc = shutil.which("cc") or shutil.which("gcc")
    if not cc:
        raise CapiBuildError("no C compiler (cc or gcc) to build the C interface with")
    if not include or not os.path.exists(os.path.join(include, "Python.h")):
        raise CapiBuildError(f"Python.h not found under {include}: the C interface needs the interpreter's headers")
    tmp = lib + f".{os.getpid()}.tmp"
    cmd = [cc, "-shared", "-fPIC", "-O2", "-std=c11", "-fvisibility=hidden", "-I", include, "-I", HERE,
           os.path.join(HERE, "engine_capi.c"), "-o", tmp, "-ldl"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise CapiBuildError(f"the C compiler failed on engine_capi.c:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(h.hexdigest() + "\n")
    return lib
