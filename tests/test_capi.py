"""The C interface without a GPU: it compiles, a C program brings up the interpreter and the package through it,
and failures come back as codes with messages (here: no model can be opened without a CUDA device)."""
import ctypes
import subprocess

from capi_helpers import build_client, clean_env


def test_c_program_gets_codes_and_messages(tmp_path):
    exe, _ = build_client(str(tmp_path))
    done = subprocess.run([exe, "probe", str(tmp_path / "no_such_model")], capture_output=True, text=True,
                          env=clean_env(), cwd=str(tmp_path), timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    lines = done.stdout.splitlines()
    assert lines[0].startswith("open -> -2 ctx null: ") and len(lines[0]) > len("open -> -2 ctx null: ") + 10
    assert lines[1].startswith("open(null) -> -1: stratum_open:")
    assert lines[2] == "vocab(null) -> -1"


def test_inside_a_running_interpreter(tmp_path):
    """Loaded into a process that already runs Python, the layer uses that interpreter."""
    _, lib_path = build_client(str(tmp_path))
    lib = ctypes.CDLL(lib_path)              # (its calls take the interpreter lock themselves)
    lib.stratum_last_error.restype = ctypes.c_char_p
    lib.stratum_open.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_longlong, ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_void_p)]
    ctx = ctypes.c_void_p()
    assert lib.stratum_open(None, b"float32", 64, 0, ctypes.byref(ctx)) == -1
    assert lib.stratum_open(b"x", b"float32", 0, 0, ctypes.byref(ctx)) == -1
    assert lib.stratum_open(str(tmp_path / "none").encode(), b"float32", 64, 0, ctypes.byref(ctx)) == -2
    assert not ctx.value and len(lib.stratum_last_error(None)) > 10
    assert lib.stratum_open(b"x", b"float32", 64, 0, None) == -1
