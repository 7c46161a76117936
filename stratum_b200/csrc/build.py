"""Compiling the CUDA sources for sm_100a and loading them with ctypes.

One shared library per source file, built with nvcc at the first use of that
file's kernels (so a run compiles what its model and dtype need, nothing
else), kept beside the sources in `_build/` when that folder can be written,
else in a per-user folder under the system's temporary directory.  A library
is rebuilt when its source, the shared header or the flags change.  While nvcc
runs, a line goes to stderr every few seconds.  There is no fallback: without a
library the kernels cannot run and the import fails with the compiler's message.
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
from typing import Dict, Iterable, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
                           "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
SOURCES = ("elementwise", "linear_simple", "attention_simple", "sampling", "gemm_skinny", "attention_mma",
           "gemm_tc", "attention_tc", "attention_stream", "attention_static")
HEADERS = ("common.cuh",)
EXTRA_DEPS = {"attention_static": ("attention_mma.cu", "attention_static.h", "mma_common.cuh"),   # files a source includes
              "attention_mma": ("mma_common.cuh",), "attention_stream": ("mma_common.cuh", "tc_common.cuh"),
              "gemm_tc": ("tc_common.cuh",), "attention_tc": ("tc_common.cuh",)}

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    """nvcc is missing or failed; the message carries its output."""


def _say(msg: str) -> None:
    print(f"[stratum_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("STRATUM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $STRATUM_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be compiled and there is no other path")


def build_dir() -> str:
    """`_build/` beside the sources if writable, else a folder of this user's under the temp dir."""
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"stratum_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _fingerprint(name: str, extra_flags: Iterable[str]) -> str:
    h = hashlib.sha256()
    for f in (name + ".cu",) + HEADERS + EXTRA_DEPS.get(name, ()):
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + list(extra_flags)).encode())
    return h.hexdigest()[:24]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libstratum_{name}.so")


def _is_current(name: str, extra_flags: Iterable[str] = ()) -> bool:
    so = library_path(name)
    stamp = so + ".stamp"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _fingerprint(name, extra_flags)


def _start(name: str, nvcc: str, extra_flags: Iterable[str]):
    so = library_path(name)
    tmp = f"{so}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + ["-I", HERE, "-o", tmp, os.path.join(HERE, name + ".cu")]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    return proc, tmp, so


def ensure_built(names: Iterable[str], extra_flags: Iterable[str] = ()) -> None:
    """Compile, in parallel, whichever of `names` are missing or stale."""
    names = [n for n in names if not _is_current(n, extra_flags)]
    if not names:
        return
    nvcc = find_nvcc()
    _say(f"compiling {', '.join(n + '.cu' for n in names)} for sm_100a into {build_dir()} ...")
    t0 = time.time()
    running = {n: _start(n, nvcc, extra_flags) for n in names}
    outputs: Dict[str, str] = {}
    last = t0
    while running:
        for n in list(running):
            proc, tmp, so = running[n]
            try:
                out, _ = proc.communicate(timeout=0.5)
            except subprocess.TimeoutExpired:
                continue
            del running[n]
            outputs[n] = out
            if proc.returncode != 0:
                for other in running.values():
                    other[0].kill()
                raise BuildError(f"nvcc failed on {n}.cu (exit {proc.returncode}):\n{out}")
            os.replace(tmp, so)
            with open(so + ".stamp", "w") as f:
                f.write(_fingerprint(n, extra_flags))
        if running and time.time() - last > 5.0:
            last = time.time()
            _say(f"  still compiling {', '.join(running)} ({last - t0:.0f} s)")
    _say(f"compiled {len(names)} file(s) in {time.time() - t0:.1f} s")


def load(name: str) -> ctypes.CDLL:
    """The shared library of one source file, built first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            ensure_built([name])
            lib = ctypes.CDLL(library_path(name))
            _loaded[name] = lib
        return lib


def build_all(names: Optional[Iterable[str]] = None) -> List[str]:
    """Compile every source (used by the build check); returns the library paths."""
    names = list(names or SOURCES)
    ensure_built(names)
    return [library_path(n) for n in names]
