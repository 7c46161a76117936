"""The tensor-core matrix product's extra epilogue work, each alone against its plain restatement, in every form
of the kernel (k shared inside clusters, stream-K with its second pass, tiles, tiles on pairs of CTAs):
rows scaled by a norm that was handed over, the residual add that also hands on to the next norm, and the
query/key/value epilogue that rotates and writes the paged cache."""
import math

import numpy as np
import pytest
import torch

from plain import llama_plain as P
from test_kernels_gpu import as64, dev, rel_err

pytestmark = pytest.mark.gpu
ROWS = [1, 5, 16, 24, 48, 100, 300, 700]      # clusters / stream-K of 16, 32, 64, 128 columns / tiles / pairs of CTAs


def _bf(a):
    return dev(a, torch.bfloat16)


@pytest.mark.parametrize("M", ROWS)
@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 520), (4096, 14336)])
def test_residual_add_hands_on_to_the_next_norm(M, N, K):
    from stratum_b200 import kernels as Kn
    if K == 14336 and M not in (5, 48, 300):
        pytest.skip("the long k is tried with three row counts")
    rng = np.random.default_rng(M + N + K)
    x, w = _bf(rng.standard_normal((M, K)) * 0.5), _bf(rng.standard_normal((N, K)) * 0.05)
    bias = dev(rng.standard_normal(N) * 0.1)
    res = dev(rng.standard_normal((M, N)))
    gain = dev(rng.random(N) + 0.5)
    want = as64(res) + P.linear(as64(x), as64(w), as64(bias))
    xb = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    ss = torch.full((64, M), float("nan"), dtype=torch.float32, device="cuda")
    parts = Kn.gemm_tc(x, w, bias, res, Kn.EPI_ADD_F32_EMIT, Kn.GemmExtra().emit(xb, gain, ss))
    torch.cuda.synchronize()
    Kn.check_status()
    assert 1 <= parts <= 64
    got = as64(res)
    assert rel_err(got, want) < 6e-3
    # what was handed on belongs to the values that were written, exactly
    assert torch.equal(xb, (res * gain).to(torch.bfloat16))
    sums = as64(ss[:parts]).sum(axis=0)
    assert np.isfinite(sums).all() and torch.isnan(ss[parts:]).all()
    assert np.max(np.abs(sums - (got ** 2).sum(axis=1)) / (got ** 2).sum(axis=1)) < 1e-5


@pytest.mark.parametrize("M", ROWS)
@pytest.mark.parametrize("mode,K,N", [("store", 1024, 2048 + 128), ("swiglu", 1024, 2048 + 128),
                                      ("store", 4096 + 64, 4096)])   # the last: k shared inside clusters up to 64 rows
def test_rows_scaled_by_a_handed_over_norm(M, mode, K, N):
    from stratum_b200 import kernels as Kn
    rng = np.random.default_rng(M)
    H, eps, parts = 1024, 1e-5, 7
    x, w = _bf(rng.standard_normal((M, K)) * 0.5), _bf(rng.standard_normal((N, K)) * 0.05)
    bias = dev(rng.standard_normal(N) * 0.1)
    ss = dev(rng.random((parts + 2, M)) * H / parts)                 # two rows more than are used
    scale = 1.0 / np.sqrt(as64(ss[:parts]).sum(axis=0) / H + eps)
    y = P.linear(as64(x), as64(w)) * scale[:, None] + as64(bias)
    extra = Kn.GemmExtra().scaled_rows(ss, parts, H, eps)
    if mode == "store":
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        Kn.gemm_tc(x, w, bias, out, Kn.EPI_STORE, extra)
        want = y
        if N == 4096 and M <= 64:
            assert Kn.gemm_tc_last_form()[0] == "cluster-k"
    else:
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
        Kn.gemm_tc(x, w, bias, out, Kn.EPI_SWIGLU, extra)
        want = P.silu(y[:, 0::2]) * y[:, 1::2]
    torch.cuda.synchronize()
    Kn.check_status()
    assert rel_err(as64(out), want) < 8e-3


@pytest.mark.parametrize("M", ROWS)
@pytest.mark.parametrize("n_q,n_kv,hd,pairs,K", [(8, 2, 128, 64, 512), (6, 3, 64, 16, 512), (4, 4, 32, 16, 512),
                                                 (24, 4, 128, 64, 4096)])   # the last: clusters up to 64 rows
def test_query_key_value_epilogue_rotates_and_writes_the_cache(M, n_q, n_kv, hd, pairs, K):
    from stratum_b200 import kernels as Kn
    rng = np.random.default_rng(M * hd)
    N = (n_q + 2 * n_kv) * hd
    x, w = _bf(rng.standard_normal((M, K)) * 0.5), _bf(rng.standard_normal((N, K)) * 0.05)
    bias = dev(rng.standard_normal(N) * 0.1)
    # rows are tokens of sequences of unequal lengths with pages in an order of their own; some rows are padding
    n_seqs = max(1, M // 3)
    seq = rng.integers(0, n_seqs, size=M)
    pos = np.zeros(M, dtype=np.int64)
    count = {}
    for i in range(M):
        base = 61 * (int(seq[i]) % 3)
        pos[i] = base + count.get(int(seq[i]), 0)
        count[int(seq[i])] = count.get(int(seq[i]), 0) + 1
    pad = rng.random(M) < 0.15
    seq_dev = np.where(pad, -1, seq).astype(np.int32)
    width = int(pos.max()) // 64 + 1
    table = rng.permutation(n_seqs * width).reshape(n_seqs, width).astype(np.int32)
    n_pages = n_seqs * width
    kc = torch.full((n_pages, n_kv, 64, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full((n_pages, n_kv, 64, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    inv = dev(1.0 / (10000.0 ** (np.arange(pairs) * 2.0 / (2 * pairs))))
    cs = torch.empty(M, pairs, 2, dtype=torch.float32, device="cuda")
    Kn.rope_table(dev(pos, torch.int32), inv, 1.25, cs)
    ang = pos[:, None].astype(np.float32) * as64(inv).astype(np.float32)[None, :]
    assert rel_err(as64(cs), 1.25 * np.stack([np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))], axis=2)) < 1e-6
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device="cuda")
    extra = Kn.GemmExtra().qkv_rope(cs, dev(pos, torch.int32), dev(seq_dev, torch.int32), dev(table, torch.int32), kc,
                                    vc, n_q, n_kv, hd, 64, True)
    Kn.gemm_tc(x, w, bias, out, Kn.EPI_QKV_ROPE, extra)
    torch.cuda.synchronize()
    Kn.check_status()
    if K == 4096 and M <= 64:
        assert Kn.gemm_tc_last_form()[0] == "cluster-k"
    y = P.linear(as64(x), as64(w), as64(bias))
    q = y[:, :n_q * hd].reshape(M, n_q, hd)
    k = y[:, n_q * hd:(n_q + n_kv) * hd].reshape(M, n_kv, hd)
    v = y[:, (n_q + n_kv) * hd:].reshape(M, n_kv, hd)
    inv64 = as64(inv).astype(np.float32)
    q = P.apply_rope(q, pos, inv64, True, 1.25)
    k = P.apply_rope(k, pos, inv64, True, 1.25)
    assert rel_err(as64(out[:, :n_q * hd]), q.reshape(M, -1)) < 8e-3
    kc64, vc64 = as64(kc), as64(vc)
    written = np.zeros((n_pages, 64), dtype=bool)
    for i in range(M):
        if pad[i]:
            continue
        pg, at = table[seq[i], pos[i] // 64], pos[i] % 64
        written[pg, at] = True
        assert rel_err(kc64[pg, :, at], k[i]) < 8e-3, i
        assert rel_err(vc64[pg, :, at], v[i]) < 8e-3, i
    untouched = ~written                                                       # [pages, places]: nothing else was touched
    assert np.all(kc64.transpose(0, 2, 1, 3)[untouched] == 7.0) and np.all(vc64.transpose(0, 2, 1, 3)[untouched] == 7.0)
    # without the cache (a layer that reads another layer's): queries only
    kc.fill_(7.0)
    extra = Kn.GemmExtra().qkv_rope(cs, dev(pos, torch.int32), dev(seq_dev, torch.int32), None, None, None, n_q, n_kv,
                                    hd, 64, False)
    out2 = torch.full((M, N), 9.0, dtype=torch.bfloat16, device="cuda")
    Kn.gemm_tc(x, w, bias, out2, Kn.EPI_QKV_ROPE, extra)
    torch.cuda.synchronize()
    assert torch.equal(out2[:, :n_q * hd], out[:, :n_q * hd]) and bool((kc == 7.0).all())


def test_extras_are_refused_where_they_cannot_hold():
    from stratum_b200 import kernels as Kn
    x, w = _bf(np.zeros((4, 64))), _bf(np.zeros((200, 64)))
    res = torch.zeros(4, 200, device="cuda")
    with pytest.raises(Kn.KernelError):                 # N no multiple of 128: the sums' parts would not tile it
        Kn.gemm_tc(x, w, None, res, Kn.EPI_ADD_F32_EMIT,
                   Kn.GemmExtra().emit(torch.zeros(4, 200, dtype=torch.bfloat16, device="cuda"),
                                       torch.ones(200, device="cuda"), torch.zeros(8, 4, device="cuda")))
    with pytest.raises(Kn.KernelError):
        Kn.gemm_tc(x, w, None, res, Kn.EPI_ADD_F32_EMIT)                        # needs its GemmExtra
