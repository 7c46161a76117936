"""Compile the C interface into libstratum_c.so beside its source (the host compiler; no CUDA in this layer)."""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ("stratum_capi.c", "stratum.h")
LIBRARY = os.path.join(HERE, "_build", "libstratum_c.so")


def python_link_flags():
    """(include dir, library dir, library name) of the interpreter that runs this."""
    cfg = sysconfig.get_config_vars()
    if not cfg.get("Py_ENABLE_SHARED"):
        raise RuntimeError("this interpreter has no shared library (libpython) to embed")
    name = "python" + cfg["LDVERSION"]
    return sysconfig.get_paths()["include"], cfg.get("LIBDIR") or "", name


def library(verbose: bool = False) -> str:
    """The path of libstratum_c.so, compiled if it is missing or older than its sources."""
    newest = max(os.path.getmtime(os.path.join(HERE, s)) for s in SOURCES)
    if os.path.exists(LIBRARY) and os.path.getmtime(LIBRARY) >= newest:
        return LIBRARY
    os.makedirs(os.path.dirname(LIBRARY), exist_ok=True)
    include, libdir, name = python_link_flags()
    tmp = LIBRARY + f".{os.getpid()}.tmp"
    cmd = ["gcc", "-O2", "-Wall", "-Wextra", "-shared", "-fPIC", "-I", include, "-I", HERE,
           f'-DSTRATUM_PYTHON_EXE="{sys.executable}"',
           os.path.join(HERE, "stratum_capi.c"), "-o", tmp]
    if libdir:
        cmd += ["-L", libdir, f"-Wl,-rpath,{libdir}"]
    cmd += ["-l" + name, "-ldl"]
    if verbose:
        print("[stratum_b200] compiling the C interface", flush=True)
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError("the C interface did not compile:\n" + " ".join(cmd) + "\n" + done.stderr)
    os.replace(tmp, LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    print(library(verbose=True))
