"""The allocation-free attention entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they need attention (inside a
stream capture, on a thread that must not block in the driver, under a fixed memory budget, or
from a binding that owns no allocator).  `stratum_attention_mma_static` serves them from a scratch
array built into its library.  This test calls it exactly as such a caller would - ctypes on the
shared library, raw pointers, no helper of the package in between - twice in a row with different
shapes, so that what the first call leaves in the shared scratch is there when the second runs, and
compares both results with the regular entry point, which takes its scratch from the caller.

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, c, n_q, n_kv, hd, n_splits, chunk, window=0):
    """The exported symbol, with nothing but pointers and sizes."""
    f = lib.stratum_attention_mma_static
    f.restype = c_int
    f.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                  c_int, c_void_p]
    T = c["T"]
    out = torch.zeros(T, n_q * hd, dtype=torch.bfloat16, device="cuda")
    status = f(c["qkv"].data_ptr(), c["qkv"].stride(0), c["kc"].data_ptr(), c["vc"].data_ptr(),
               c["pos"].data_ptr(), c["seq"].data_ptr(), c["table"].data_ptr(), c["table"].stride(0),
               None, None, None, T, 1, out.data_ptr(), out.stride(0), T, n_q, n_kv, hd, 64, window,
               c_float(1.0 / math.sqrt(hd)), n_splits, chunk, torch.cuda.current_stream().cuda_stream)
    return status, out


def test_static_scratch_entry_point_matches_the_regular_one():
    from stratum_b200.csrc import build
    from test_kernels_gpu import _attention_case, _run_mma, as64, rel_err
    lib = build.load("attention_static")          # a ctypes.CDLL of the shared library; nothing else of the package
    size = lib.stratum_attention_static_scratch_floats
    size.restype = ctypes.c_longlong
    assert size() == 4 * 1024 * 1024

    rng = np.random.default_rng(99)
    # first call: long sequences, many splits; second call: other sizes, fewer splits, so stale partials of
    # the first call lie exactly where the second one's unused slots would be
    cases = [((8, 2, 128), [699, 0, 63, 64, 300, 1023], 8, 128),
             ((6, 1, 64), [200, 511, 5], 3, 192)]
    for (n_q, n_kv, hd), lens, n_splits, chunk in cases:
        c = _attention_case(rng, lens, [1] * len(lens), n_q, n_kv, hd, "bfloat16")
        want = _run_mma(c, [1] * len(lens), n_q, n_kv, hd, n_splits=n_splits, chunk=chunk)
        status, got = _call_static(lib, c, n_q, n_kv, hd, n_splits, chunk)
        torch.cuda.synchronize()
        assert status == 0
        assert rel_err(as64(got), as64(want)) < 8e-3           # the tolerance of the attention tests
        assert rel_err(as64(got), c["ref"]) < 8e-3             # and against the plain reference itself
        assert torch.equal(got, want)                           # same kernels, same inputs: the same bits

    # one split uses no scratch, so a step far beyond the scratch's size is taken as the regular entry point
    # takes it: 1,100 sequences x 32 heads x 130 floats would be 4.6 M floats, more than the array holds
    lens = [int(x) for x in rng.integers(0, 3, size=1100)]
    c = _attention_case(rng, lens, [1] * len(lens), 32, 8, 128, "bfloat16")
    want = _run_mma(c, [1] * len(lens), 32, 8, 128, n_splits=1, chunk=64)
    status, got = _call_static(lib, c, 32, 8, 128, 1, 64)
    torch.cuda.synchronize()
    assert status == 0 and torch.equal(got, want)
    assert rel_err(as64(got), c["ref"]) < 8e-3
    status, _ = _call_static(lib, c, 32, 8, 128, 2, 64)        # the same step in two splits does need it
    assert status == -4

    # beyond the built-in scratch: refused before anything is launched
    c = _attention_case(rng, [10] * 4, [1] * 4, 8, 2, 128, "bfloat16")
    status, _ = _call_static(lib, c, 8, 2, 128, 40000, 64)
    assert status == -4
    torch.cuda.synchronize()
