"""Compile the C interface and the C caller of it (tests/capi_client.c) for the tests."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def build_client(tmp_dir: str):
    """(path of the client program, path of libstratum_c.so)."""
    from stratum_b200.capi.build import library
    lib = library()
    exe = os.path.join(tmp_dir, "capi_client")
    cmd = ["gcc", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "stratum_b200", "capi"),
           os.path.join(HERE, "capi_client.c"), "-o", exe, "-L", os.path.dirname(lib), "-lstratum_c",
           f"-Wl,-rpath,{os.path.dirname(lib)}"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    return exe, lib


def clean_env():
    """The environment a C program has: nothing that points an interpreter at this package."""
    env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH", "PYTHONHOME", "VIRTUAL_ENV")}
    return env
