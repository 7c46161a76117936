"""Each kernel alone against its plain reference, at sizes other than the engine tests use."""
import math

import numpy as np
import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def as64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rel_err(got, ref):
    return float(np.max(np.abs(got - ref)) / (np.max(np.abs(ref)) + 1e-30))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [100, 4096, 5120 + 8])
def test_rmsnorm(dtype, hidden):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(hidden)
    x = dev(rng.standard_normal((7, hidden)) * 3.0)
    gain = dev(rng.random(hidden) + 0.5)
    out = torch.empty(7, hidden, dtype=DT[dtype], device="cuda")
    K.rmsnorm(x, gain, 1e-5, out)
    ref = P.rms_norm(as64(x), as64(gain), 1e-5)
    assert rel_err(as64(out), ref) < (2e-6 if dtype == "float32" else 5e-3)
    rows = dev([5, 0, 5], torch.int32)
    out2 = torch.empty(3, hidden, dtype=DT[dtype], device="cuda")
    K.rmsnorm(x, gain, 1e-5, out2, rows)
    assert torch.equal(out2, out[[5, 0, 5]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [1024, 1544, 4096, 8192])
def test_rmsnorm_many_rows(dtype, hidden):
    """Prompts take other block shapes than decode steps (more values per thread)."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(hidden + 1)
    x = dev(rng.standard_normal((300, hidden)) * 2.0)
    gain = dev(rng.random(hidden) + 0.5)
    out = torch.empty(300, hidden, dtype=DT[dtype], device="cuda")
    K.rmsnorm(x, gain, 1e-6, out)
    assert rel_err(as64(out), P.rms_norm(as64(x), as64(gain), 1e-6)) < (2e-6 if dtype == "float32" else 5e-3)
    few = torch.empty(5, hidden, dtype=DT[dtype], device="cuda")
    K.rmsnorm(x[:5], gain, 1e-6, few)
    assert rel_err(as64(few), as64(out[:5])) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,head_dim,first", [(5, 48, 0), (2, 128, 640), (7, 20, 8)])
def test_rmsnorm_heads_in_place(dtype, n_heads, head_dim, first):
    """The per-head norm of queries or keys: only the named stretch of each row changes."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(n_heads * head_dim)
    width = first + n_heads * head_dim + 24
    x = dev(rng.standard_normal((9, width)) * 2.0, DT[dtype])
    gain = dev(rng.random(head_dim) + 0.5)
    before = as64(x)
    K.rmsnorm_heads(x, first, n_heads, head_dim, gain, 1e-6)
    got = as64(x)
    heads = before[:, first:first + n_heads * head_dim].reshape(9, n_heads, head_dim)
    ref = P.head_rms_norm(heads, as64(gain), 1e-6).reshape(9, -1)
    assert rel_err(got[:, first:first + n_heads * head_dim], ref) < (2e-6 if dtype == "float32" else 5e-3)
    assert np.array_equal(got[:, :first], before[:, :first])
    assert np.array_equal(got[:, first + n_heads * head_dim:], before[:, first + n_heads * head_dim:])
    one = dev(before[4:5], DT[dtype])                      # a row alone gives the bits it gave in the batch
    K.rmsnorm_heads(one, first, n_heads, head_dim, gain, 1e-6)
    assert torch.equal(one[0], x[4])
    with pytest.raises(K.KernelError):
        K.rmsnorm_heads(x, first, n_heads + 2, head_dim, gain, 1e-6)      # would run past the row


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed_gather(dtype):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(1)
    table = dev(rng.standard_normal((1000, 72)), DT[dtype])
    ids = dev([999, 0, 17, 17], torch.int32)
    out = torch.empty(4, 72, dtype=torch.float32, device="cuda")
    K.embed_gather(table, ids, out)
    assert torch.equal(out, table[[999, 0, 17, 17]].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(2)
    g, u = rng.standard_normal((5, 176)) * 4, rng.standard_normal((5, 176))
    gu = dev(np.stack([g, u], axis=2).reshape(5, 352), DT[dtype])
    out = torch.empty(5, 176, dtype=DT[dtype], device="cuda")
    K.swiglu(gu, out)
    g64, u64 = as64(gu)[:, 0::2], as64(gu)[:, 1::2]
    assert rel_err(as64(out), P.silu(g64) * u64) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K_", [(1, 50, 24), (70, 130, 96), (3, 1000, 176), (129, 64, 520)])
def test_linear_simple(dtype, M, N, K_):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(M * N)
    x = dev(rng.standard_normal((M, K_)), DT[dtype])
    w = dev(rng.standard_normal((N, K_)) * 0.1, DT[dtype])
    b = dev(rng.standard_normal(N))
    ref = P.linear(as64(x), as64(w), as64(b))
    tol = 1e-5 if dtype == "float32" else 6e-3
    out = torch.empty(M, N, dtype=DT[dtype], device="cuda")
    K.linear_simple(x, w, b, out, K.EPI_STORE)
    assert rel_err(as64(out), ref) < tol
    res = dev(rng.standard_normal((M, N)))
    keep = as64(res)
    K.linear_simple(x, w, None, res, K.EPI_ADD_F32)
    assert rel_err(as64(res), keep + P.linear(as64(x), as64(w))) < 1e-5
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    K.linear_simple(x, w, b, out32, K.EPI_STORE_F32)
    assert rel_err(as64(out32), ref) < 1e-5
    # a row's value does not depend on the rows beside it
    one = torch.empty(1, N, dtype=torch.float32, device="cuda")
    K.linear_simple(x[M - 1:M], w, b, one, K.EPI_STORE_F32)
    assert torch.equal(one[0], out32[M - 1])


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16, 32])
@pytest.mark.parametrize("N,K_", [(48, 64), (1000, 200), (4096 + 16, 4096), (2 * 177, 96)])
def test_gemm_skinny(M, N, K_):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(M + N)
    x = dev(rng.standard_normal((M, K_)), torch.bfloat16)
    w = dev(rng.standard_normal((N, K_)) * 0.1, torch.bfloat16)
    b = dev(rng.standard_normal(N))
    ref = P.linear(as64(x), as64(w), as64(b))
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.gemm_skinny(x, w, b, out, K.EPI_STORE)
    assert rel_err(as64(out), ref) < 6e-3
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    K.gemm_skinny(x, w, b, out32, K.EPI_STORE_F32)
    assert rel_err(as64(out32), ref) < 2e-5
    res = dev(rng.standard_normal((M, N)))
    keep = as64(res)
    K.gemm_skinny(x, w, None, res, K.EPI_ADD_F32)
    assert rel_err(as64(res), keep + P.linear(as64(x), as64(w))) < 2e-5
    act = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
    K.gemm_skinny(x, w, b, act, K.EPI_SWIGLU)
    r16 = as64(dev(ref, torch.bfloat16))
    assert rel_err(as64(act), P.silu(r16[:, 0::2]) * r16[:, 1::2]) < 2e-2
    # the same row alone gives the same bits
    one = torch.empty(1, N, dtype=torch.float32, device="cuda")
    K.gemm_skinny(x[M - 1:M], w, b, one, K.EPI_STORE_F32)
    assert torch.equal(one[0], out32[M - 1])


# shapes of test_gemm_tc that take the cluster form on 148 SMs (clusters of 4, 3, 5, 5, 2, 4 and 4 CTAs when this
# was written; how many clusters of a size fit at once is the driver's answer)
CLUSTER_FORMS = {(8, 4096, 4096), (40, 4096, 4096 + 72), (30, 5000, 3080), (24, 3072, 6144), (13, 3000, 6152),
                 (64, 8192 + 8, 2048 + 16), (17, 4096, 14336), (64, 4096 + 64, 14336)}


PAIRS_SHARED = {(512, 4096, 14336), (256, 6144, 4096 + 64), (400, 4096, 14336 + 8)}
# 129 to 256 rows, few tiles of W, long k: clusters again, x as one block of 256 rows
WIDE_CLUSTERS = {(200, 4096, 4096), (256, 4096 + 64, 4096), (250, 4100, 14344), (129, 4096, 4096 + 8)}


@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (33, 48, 64), (64, 1000, 200), (100, 256, 4096), (300, 4096 + 16, 512),
                                     (2048, 2 * 177, 96), (129, 6144, 1024), (1, 128, 128), (17, 130, 72),
                                     (8, 4096, 4096), (5, 28672, 1024), (64, 4096 + 64, 14336), (16, 6144, 4096),
                                     (40, 50000, 512), (8, 128256, 1024), (9, 1002, 1096), (64, 260, 2048),
                                     # more tiles than SMs with a partly filled last wave: its tiles are shared along k
                                     (2048, 4096, 512), (1024, 6144, 1280), (4096, 1024, 640), (2000, 4100, 520),
                                     # fewer tiles than SMs: all of them are shared
                                     (200, 4096, 4096), (100, 1000, 8192), (65, 2304, 2048), (128, 4096, 1024), (97, 6146, 328),
                                     # a full wave of whole tiles, then shared ones
                                     (1280, 4608, 8192),
                                     # pairs of CTAs on 256 x 256 tiles: rows and columns that end inside a tile, more
                                     # tiles than pairs of SMs, one row of tiles
                                     (1000, 2100, 264), (256, 28672, 128), (2304, 9000, 72),
                                     # a few hundred rows, few tiles of 256 x 256: all pairs of CTAs share them along k
                                     (512, 4096, 14336), (256, 4096 + 64, 4096), (520, 4100, 14344), (130, 2048 + 8, 1096), (700, 4100, 2048),
                                     (256, 6144, 4096 + 64), (200, 2048, 8192), (400, 4096, 14336 + 8), (250, 4100, 14344), (129, 4096, 4096 + 8),
                                     # few rows, no more tiles than SMs: too little k for clusters to share
                                     (40, 4096, 2048), (30, 5120, 1000), (3, 2304, 1032), (8, 16000, 520),
                                     # k shared inside clusters, rows dealt out to the ranks
                                     (40, 4096, 4096 + 72), (30, 5000, 3080), (24, 3072, 6144), (13, 3000, 6152),
                                     (64, 8192 + 8, 2048 + 16), (17, 4096, 14336)])
def test_gemm_tc(M, N, K_):
    """(The forms the few-row cases take on 148 SMs are checked too; see CLUSTER_FORMS.)"""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(M + N + K_)
    x = dev(rng.standard_normal((M, K_)), torch.bfloat16)
    w = dev(rng.standard_normal((N, K_)) * 0.1, torch.bfloat16)
    b = dev(rng.standard_normal(N))
    ref = as64(x) @ as64(w).T + as64(b)
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    K.gemm_tc(x, w, b, out32, K.EPI_STORE_F32)
    K.check_status()
    assert rel_err(as64(out32), ref) < 2e-5
    if (M, N, K_) in CLUSTER_FORMS:
        form, size = K.gemm_tc_last_form()
        assert form == "cluster-k" and 2 <= size <= 8
    elif M <= 64:
        assert K.gemm_tc_last_form()[0] == "stream-k"
    elif (M, N, K_) in PAIRS_SHARED:
        assert K.gemm_tc_last_form()[0] == "pairs-shared"
    elif (M, N, K_) in WIDE_CLUSTERS:
        assert K.gemm_tc_last_form()[0] == "cluster-k"
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc(x, w, b, out, K.EPI_STORE)
    assert rel_err(as64(out), ref) < 6e-3
    res = dev(rng.standard_normal((M, N)))
    keep = as64(res)
    K.gemm_tc(x, w, None, res, K.EPI_ADD_F32)
    assert rel_err(as64(res), keep + as64(x) @ as64(w).T) < 2e-5
    act = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc(x, w, b, act, K.EPI_SWIGLU)
    K.check_status()
    r16 = as64(dev(ref, torch.bfloat16))
    assert rel_err(as64(act), P.silu(r16[:, 0::2]) * r16[:, 1::2]) < 2e-2
    # the split over SMs depends on the shapes only: a second run gives the same bits
    again = torch.empty(M, N, dtype=torch.float32, device="cuda")
    K.gemm_tc(x, w, b, again, K.EPI_STORE_F32)
    K.check_status()
    assert torch.equal(again, out32)
    if M <= 16:
        # and a row alone gives the same bits as the row in its batch
        one = torch.empty(1, N, dtype=torch.float32, device="cuda")
        K.gemm_tc(x[M - 1:M], w, b, one, K.EPI_STORE_F32)
        assert torch.equal(one[0], out32[M - 1])


def test_gemm_skinny_refuses_what_it_cannot_do():
    from stratum_b200 import kernels as K
    x = torch.zeros(2, 20, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(2, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(K.KernelError, match="shape"):
        K.gemm_skinny(x, w, None, out, K.EPI_STORE)            # K = 20 is no multiple of 8
    x = torch.zeros(40, 16, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 16, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(40, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(K.KernelError, match="limit"):
        K.gemm_skinny(x, w, None, out, K.EPI_STORE)


# ------------------------------------------------------------------ rope + cache write, attention
def _paged(rng, n_pages, n_kv, hd, dtype):
    return (torch.zeros(n_pages, n_kv, 64, hd, dtype=DT[dtype], device="cuda"),
            torch.zeros(n_pages, n_kv, 64, hd, dtype=DT[dtype], device="cuda"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_store_rotates_and_lands_in_the_right_rows(dtype, interleaved):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(4)
    n_q, n_kv, hd, rope_dim = 6, 2, 48, 32
    # two sequences: the first continues at position 130 with 3 tokens, the second starts with 2
    pos = [130, 131, 132, 0, 1]
    seq = [0, 0, 0, 1, 1]
    table = np.array([[7, 3, 9], [5, -1, -1]], dtype=np.int32)       # pages in an order of their own
    qkv = dev(rng.standard_normal((5, (n_q + 2 * n_kv) * hd)), DT[dtype])
    before = as64(qkv)
    inv = P.rope_inv_freq(rope_dim, 10000.0).astype(np.float32)
    kc, vc = _paged(rng, 10, n_kv, hd, dtype)
    K.rope_store(qkv, dev(pos, torch.int32), dev(seq, torch.int32), dev(table, torch.int32), dev(inv), interleaved,
                 1.0, kc, vc, n_q, n_kv, hd, 64, True)
    heads = before.reshape(5, n_q + 2 * n_kv, hd)
    q_ref = P.apply_rope(heads[:, :n_q], np.array(pos), inv.astype(np.float64), interleaved)
    k_ref = P.apply_rope(heads[:, n_q:n_q + n_kv], np.array(pos), inv.astype(np.float64), interleaved)
    v_ref = heads[:, n_q + n_kv:]
    tol = 2e-6 if dtype == "float32" else 5e-3
    assert rel_err(as64(qkv).reshape(5, -1, hd)[:, :n_q], q_ref) < tol
    assert np.array_equal(as64(qkv).reshape(5, -1, hd)[:, n_q:], heads[:, n_q:])       # k and v stay as projected
    for t in range(5):
        page = table[seq[t], pos[t] // 64]
        assert rel_err(as64(kc[page, :, pos[t] % 64]), k_ref[t]) < tol
        assert np.array_equal(as64(vc[page, :, pos[t] % 64]), v_ref[t])
    written = {(int(table[s, p // 64]), p % 64) for s, p in zip(seq, pos)}
    mask = torch.ones(10, 64, dtype=torch.bool)
    for pg, r in written:
        mask[pg, r] = False
    assert float(kc.float().abs().sum(dim=(1, 3)).cpu()[mask].sum()) == 0.0            # nothing else was touched


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (3, 3, 48), (5, 1, 16)])
def test_rope_store_prompt_kernel(interleaved, n_q, n_kv, hd):
    """Prompts of 64 tokens or more with fully rotated heads take the 16-byte kernel; a continuation lands beside
    what the cache already holds, and the same tokens one by one give the same rows up to rounding."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(hd + n_q)
    n0, n1 = 70, 90                                                   # sequence 0 continues at 50; sequence 1 starts
    pos = list(range(50, 50 + n0)) + list(range(n1))
    seq = [0] * n0 + [1] * n1
    table = np.array([[4, 1], [0, 5]], dtype=np.int32)
    T = n0 + n1
    qkv = dev(rng.standard_normal((T, (n_q + 2 * n_kv) * hd)), torch.bfloat16)
    before = as64(qkv)
    inv = P.rope_inv_freq(hd, 500000.0).astype(np.float32)
    kc, vc = _paged(rng, 6, n_kv, hd, "bfloat16")
    single = qkv.clone()
    kc1, vc1 = _paged(rng, 6, n_kv, hd, "bfloat16")
    K.rope_store(qkv, dev(pos, torch.int32), dev(seq, torch.int32), dev(table, torch.int32), dev(inv), interleaved,
                 1.0, kc, vc, n_q, n_kv, hd, 64, True)
    for t in range(0, T, 40):                                         # fewer than 64 tokens: the general kernel
        K.rope_store(single[t:t + 40], dev(pos[t:t + 40], torch.int32), dev(seq[t:t + 40], torch.int32),
                     dev(table, torch.int32), dev(inv), interleaved, 1.0, kc1, vc1, n_q, n_kv, hd, 64, True)
    heads = before.reshape(T, n_q + 2 * n_kv, hd)
    q_ref = P.apply_rope(heads[:, :n_q], np.array(pos), inv.astype(np.float64), interleaved)
    k_ref = P.apply_rope(heads[:, n_q:n_q + n_kv], np.array(pos), inv.astype(np.float64), interleaved)
    assert rel_err(as64(qkv).reshape(T, -1, hd)[:, :n_q], q_ref) < 5e-3
    assert np.array_equal(as64(qkv).reshape(T, -1, hd)[:, n_q:], heads[:, n_q:])
    for t in range(T):
        page = table[seq[t], pos[t] // 64]
        assert rel_err(as64(kc[page, :, pos[t] % 64]), k_ref[t]) < 5e-3
        assert np.array_equal(as64(vc[page, :, pos[t] % 64]), heads[t, n_q + n_kv:])
    assert rel_err(as64(qkv), as64(single)) < 5e-3 and rel_err(as64(kc), as64(kc1)) < 5e-3
    assert torch.equal(vc, vc1)
    # rows nobody wrote stay zero: sequence 0 holds positions 50..119, sequence 1 0..89
    untouched = kc.clone()
    for s_, lo, hi in ((0, 50, 120), (1, 0, 90)):
        for p_ in range(lo, hi):
            untouched[table[s_, p_ // 64], :, p_ % 64] = 0
    assert float(untouched.float().abs().sum()) == 0.0


def _attention_case(rng, lens_before, n_new, n_q, n_kv, hd, dtype, window=0, spike=None):
    """Build a paged cache holding random keys/values and run the kernel for the new tokens."""
    from stratum_b200 import kernels as K
    B = len(lens_before)
    total = [a + b for a, b in zip(lens_before, n_new)]
    n_pages = sum((t + 63) // 64 for t in total)
    order = rng.permutation(n_pages).tolist()
    kc, vc = _paged(rng, n_pages, n_kv, hd, dtype)
    width = max((t + 63) // 64 for t in total)
    table = np.full((B, width), -1, dtype=np.int32)
    ks, vs, qs = [], [], []
    for s in range(B):
        k = rng.standard_normal((total[s], n_kv, hd))
        v = rng.standard_normal((total[s], n_kv, hd))
        q = rng.standard_normal((n_new[s], n_q, hd))
        if spike is not None:
            spike(s, q, k, v)
        k = as64(dev(k, DT[dtype])); v = as64(dev(v, DT[dtype])); q = as64(dev(q, DT[dtype]))
        for p in range((total[s] + 63) // 64):
            pg = order.pop()
            table[s, p] = pg
            n = min(64, total[s] - 64 * p)
            kc[pg, :, :n] = dev(k[64 * p:64 * p + n].transpose(1, 0, 2), DT[dtype])
            vc[pg, :, :n] = dev(v[64 * p:64 * p + n].transpose(1, 0, 2), DT[dtype])
        ks.append(k); vs.append(v); qs.append(q)
    T = sum(n_new)
    qkv = torch.zeros(T, (n_q + 2 * n_kv) * hd, dtype=DT[dtype], device="cuda")
    pos, seq, r = [], [], 0
    for s in range(B):
        qkv[r:r + n_new[s], :n_q * hd] = dev(qs[s].reshape(n_new[s], -1), DT[dtype])
        pos += list(range(lens_before[s], total[s])); seq += [s] * n_new[s]; r += n_new[s]
    ref = []
    for s in range(B):
        scale = 1.0 / math.sqrt(hd)
        for i in range(n_new[s]):
            p = lens_before[s] + i
            lo = 0 if window <= 0 else max(0, p - window + 1)
            row = np.zeros((n_q, hd))
            for h in range(n_q):
                kv = h // (n_q // n_kv)
                sc = ks[s][lo:p + 1, kv] @ qs[s][i, h] * scale
                row[h] = P.softmax(sc) @ vs[s][lo:p + 1, kv]
            ref.append(row.reshape(-1))
    return dict(qkv=qkv, kc=kc, vc=vc, pos=dev(pos, torch.int32), seq=dev(seq, torch.int32),
                table=dev(table, torch.int32), ref=np.stack(ref), T=T)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (5, 5, 48), (6, 1, 16), (2, 1, 256)])
def test_attention_simple(dtype, n_q, n_kv, hd):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(hd)
    c = _attention_case(rng, [0, 130, 63, 700], [70, 1, 3, 1], n_q, n_kv, hd, dtype)
    out = torch.empty(c["T"], n_q * hd, dtype=DT[dtype], device="cuda")
    K.attention_simple(c["qkv"], c["kc"], c["vc"], c["pos"], c["seq"], c["table"], out, n_q, n_kv, hd, 64, 0,
                       1.0 / math.sqrt(hd))
    assert rel_err(as64(out), c["ref"]) < (3e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """Scale one query and one key so that a single far score dominates: the output must be that key's value."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(11)
    n_q, n_kv, hd = 4, 2, 64
    far = {0: 3, 1: 517}                      # sequence -> position of the key to find

    def spike(s, q, k, v):
        d = rng.standard_normal(hd)
        d /= np.linalg.norm(d)
        k[far[s], :, :] = d * 12.0
        q[-1, :, :] = d * 12.0                # the last new token looks for it

    c = _attention_case(rng, [699, 600], [1, 2], n_q, n_kv, hd, dtype, spike=spike)
    out = torch.empty(c["T"], n_q * hd, dtype=DT[dtype], device="cuda")
    K.attention_simple(c["qkv"], c["kc"], c["vc"], c["pos"], c["seq"], c["table"], out, n_q, n_kv, hd, 64, 0,
                       1.0 / math.sqrt(hd))
    assert rel_err(as64(out), c["ref"]) < (3e-6 if dtype == "float32" else 8e-3)
    # and the reference itself is (almost) that one value row: the case does test the far key
    v_far = as64(c["vc"][c["table"][0, far[0] // 64].item(), 0, far[0] % 64])
    assert np.max(np.abs(c["ref"][0][:hd] - v_far)) < 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(dtype):
    """With a window of W keys the key at p-W+1 counts and the key at p-W does not."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(12)
    n_q, n_kv, hd, W = 2, 1, 32, 100
    p = 299

    def spike(s, q, k, v):
        d = rng.standard_normal(hd)
        d /= np.linalg.norm(d)
        q[-1, :, :] = d * 10.0
        k[p - W + 1 if s == 0 else p - W, :, :] = d * 10.0       # just inside / just outside

    c = _attention_case(rng, [p, p], [1, 1], n_q, n_kv, hd, dtype, window=W, spike=spike)
    out = torch.empty(c["T"], n_q * hd, dtype=DT[dtype], device="cuda")
    K.attention_simple(c["qkv"], c["kc"], c["vc"], c["pos"], c["seq"], c["table"], out, n_q, n_kv, hd, 64, W,
                       1.0 / math.sqrt(hd))
    assert rel_err(as64(out), c["ref"]) < (3e-6 if dtype == "float32" else 8e-3)
    inside = as64(c["vc"][c["table"][0, (p - W + 1) // 64].item(), 0, (p - W + 1) % 64])
    outside = as64(c["vc"][c["table"][1, (p - W) // 64].item(), 0, (p - W) % 64])
    assert np.max(np.abs(c["ref"][0][:hd] - inside)) < 1e-2          # found
    assert np.max(np.abs(c["ref"][1][:hd] - outside)) > 0.1          # not seen


def _run_mma(c, n_new, n_q, n_kv, hd, window=0, n_splits=1, chunk=0):
    from stratum_b200 import kernels as K
    out = torch.zeros(c["T"], n_q * hd, dtype=torch.bfloat16, device="cuda")
    gs = n_q // n_kv
    if all(n == 1 for n in n_new):
        qblocks, per_block = None, 1
    else:
        per_block = 16 // min(gs, 16)
        seqs, rows, counts, r = [], [], [], 0
        for i, n in enumerate(n_new):
            for b in range(0, n, per_block):
                seqs.append(i); rows.append(r + b); counts.append(min(per_block, n - b))
            r += n
        qblocks = tuple(dev(a, torch.int32) for a in (seqs, rows, counts))
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.full((c["T"] * n_q * n_splits * hd,), float("nan"), dtype=torch.float32, device="cuda")
        part_ml = torch.full((c["T"] * n_q * n_splits * 2,), float("nan"), dtype=torch.float32, device="cuda")
    K.attention_mma(c["qkv"], c["kc"], c["vc"], c["pos"], c["seq"], c["table"], qblocks, per_block, out, part_o,
                    part_ml, n_q, n_kv, hd, 64, window, 1.0 / math.sqrt(hd), n_splits, chunk)
    return out


@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (5, 5, 48), (6, 1, 16), (32, 8, 64), (40, 2, 32), (3, 1, 96)])
def test_attention_mma_prompts_and_continuations(n_q, n_kv, hd):
    rng = np.random.default_rng(hd + n_q)
    n_new = [70, 1, 3, 130]
    c = _attention_case(rng, [0, 130, 63, 200], n_new, n_q, n_kv, hd, "bfloat16")
    out = _run_mma(c, n_new, n_q, n_kv, hd)
    assert rel_err(as64(out), c["ref"]) < 8e-3


@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (4, 4, 64), (40, 2, 32), (16, 2, 128), (6, 2, 48), (2, 1, 16)])
@pytest.mark.parametrize("n_splits,chunk", [(1, 0), (4, 256), (11, 64)])
def test_attention_mma_decode_with_splits(n_q, n_kv, hd, n_splits, chunk):
    rng = np.random.default_rng(hd)
    lens = [699, 0, 63, 64, 300]                # one sequence has a single key, some fill only the first split
    c = _attention_case(rng, lens, [1] * 5, n_q, n_kv, hd, "bfloat16")
    out = _run_mma(c, [1] * 5, n_q, n_kv, hd, n_splits=n_splits, chunk=chunk)
    assert rel_err(as64(out), c["ref"]) < 8e-3


def test_attention_mma_far_key_and_window_edge():
    rng = np.random.default_rng(21)
    n_q, n_kv, hd = 4, 2, 64
    far = {0: 3, 1: 517}

    def spike(s, q, k, v):
        d = rng.standard_normal(hd); d /= np.linalg.norm(d)
        k[far[s], :, :] = d * 12.0
        q[-1, :, :] = d * 12.0

    c = _attention_case(rng, [699, 600], [1, 1], n_q, n_kv, hd, "bfloat16", spike=spike)
    for n_splits, chunk in ((1, 0), (6, 128)):
        out = _run_mma(c, [1, 1], n_q, n_kv, hd, n_splits=n_splits, chunk=chunk)
        assert rel_err(as64(out), c["ref"]) < 8e-3
    W, p = 100, 299

    def edge(s, q, k, v):
        d = rng.standard_normal(hd); d /= np.linalg.norm(d)
        q[-1, :, :] = d * 10.0
        k[p - W + 1 if s == 0 else p - W, :, :] = d * 10.0

    c = _attention_case(rng, [p, p], [1, 1], n_q, n_kv, hd, "bfloat16", window=W, spike=edge)
    for n_splits, chunk in ((1, 0), (5, 64)):
        out = _run_mma(c, [1, 1], n_q, n_kv, hd, window=W, n_splits=n_splits, chunk=chunk)
        assert rel_err(as64(out), c["ref"]) < 8e-3
    c = _attention_case(rng, [250, 0], [60, 140], n_q, n_kv, hd, "bfloat16", window=W)     # prompts under a window
    out = _run_mma(c, [60, 140], n_q, n_kv, hd, window=W)
    assert rel_err(as64(out), c["ref"]) < 8e-3


def _run_tile(c, n_new, n_q, n_kv, hd, window=0):
    from stratum_b200 import kernels as K
    out = torch.zeros(c["T"], n_q * hd, dtype=torch.bfloat16, device="cuda")
    per_warp = 16 // min(n_q // n_kv, 16)
    seqs, rows, counts, r = [], [], [], 0
    for i, n in enumerate(n_new):
        for b in range(0, n, 4 * per_warp):
            seqs.append(i); rows.append(r + b); counts.append(min(4 * per_warp, n - b))
        r += n
    qblocks = tuple(dev(a, torch.int32) for a in (seqs, rows, counts))
    K.attention_tile(c["qkv"], c["kc"], c["vc"], c["pos"], c["seq"], c["table"], qblocks, per_warp, out, n_q, n_kv, hd,
                     64, window, 1.0 / math.sqrt(hd))
    return out


@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (5, 5, 48), (6, 1, 16), (32, 8, 64), (40, 2, 32), (3, 1, 96),
                                         (4, 4, 112)])
def test_attention_tile_prompts_and_continuations(n_q, n_kv, hd):
    rng = np.random.default_rng(hd + n_q + 1)
    n_new = [70, 1, 3, 130, 17]
    c = _attention_case(rng, [0, 130, 63, 200, 0], n_new, n_q, n_kv, hd, "bfloat16")
    out = _run_tile(c, n_new, n_q, n_kv, hd)
    assert rel_err(as64(out), c["ref"]) < 8e-3
    W = 100
    c = _attention_case(rng, [250, 0, 5], [60, 140, 1], n_q, n_kv, hd, "bfloat16", window=W)
    assert rel_err(as64(_run_tile(c, [60, 140, 1], n_q, n_kv, hd, window=W)), c["ref"]) < 8e-3


def test_attention_tile_far_key():
    rng = np.random.default_rng(31)
    n_q, n_kv, hd = 4, 2, 64

    def spike(s, q, k, v):
        d = rng.standard_normal(hd); d /= np.linalg.norm(d)
        k[3 if s == 0 else 517, :, :] = d * 12.0
        q[-1, :, :] = d * 12.0

    c = _attention_case(rng, [600, 0], [100, 700], n_q, n_kv, hd, "bfloat16", spike=spike)
    assert rel_err(as64(_run_tile(c, [100, 700], n_q, n_kv, hd)), c["ref"]) < 8e-3


def _run_tc(c, n_new, n_q, n_kv, hd, window=0, halves=1):
    from stratum_b200 import kernels as K
    out = torch.zeros(c["T"], n_q * hd, dtype=torch.bfloat16, device="cuda")
    per_tile = halves * (128 // (n_q // n_kv))
    seqs, rows, counts, r = [], [], [], 0
    for i, n in enumerate(n_new):
        for b in range(0, n, per_tile):
            seqs.append(i); rows.append(r + b); counts.append(min(per_tile, n - b))
        r += n
    qblocks = tuple(dev(a, torch.int32) for a in (seqs, rows, counts))
    K.attention_tc(c["qkv"], c["kc"], c["vc"], c["pos"], c["table"], qblocks, out, n_q, n_kv, hd, 64, window,
                   1.0 / math.sqrt(hd), halves)
    K.check_status()
    return out


@pytest.mark.parametrize("halves", [1, 2])
@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (4, 4, 64), (32, 8, 128), (16, 1, 64), (2, 1, 128)])
def test_attention_tc_prompts_and_continuations(n_q, n_kv, hd, halves):
    """halves 2: a CTA's two halves of 128 rows share the key and value tiles; runs that fill one half only, that
    end inside the second half, and that make the second half walk one tile more than the first."""
    rng = np.random.default_rng(hd + n_q + 2)
    n_new = [70, 1, 3, 200, 17, 300]
    c = _attention_case(rng, [0, 130, 63, 200, 0, 40], n_new, n_q, n_kv, hd, "bfloat16")
    out = _run_tc(c, n_new, n_q, n_kv, hd, halves=halves)
    assert rel_err(as64(out), c["ref"]) < 8e-3
    W = 100
    c = _attention_case(rng, [250, 0, 5], [60, 140, 1], n_q, n_kv, hd, "bfloat16", window=W)
    assert rel_err(as64(_run_tc(c, [60, 140, 1], n_q, n_kv, hd, window=W, halves=halves)), c["ref"]) < 8e-3


@pytest.mark.parametrize("halves", [1, 2])
def test_attention_tc_far_key(halves):
    rng = np.random.default_rng(41)
    n_q, n_kv, hd = 4, 2, 64

    def spike(s, q, k, v):
        d = rng.standard_normal(hd); d /= np.linalg.norm(d)
        k[3 if s == 0 else 517, :, :] = d * 12.0
        q[-1, :, :] = d * 12.0

    c = _attention_case(rng, [600, 0], [100, 700], n_q, n_kv, hd, "bfloat16", spike=spike)
    assert rel_err(as64(_run_tc(c, [100, 700], n_q, n_kv, hd, halves=halves)), c["ref"]) < 8e-3


@pytest.mark.parametrize("halves", [1, 2])
@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (4, 2, 64)])
def test_attention_tc_long_walk(n_q, n_kv, hd, halves):
    """Three hundred new tokens behind 5,900 cached ones: every query tile walks some ninety key tiles (the K and V
    rings go round forty times), one key near the beginning stands out for the last query, and with a window of
    1,000 the walk begins in the middle of the cache."""
    rng = np.random.default_rng(hd + halves)

    def spike(s, q, k, v):
        if s == 0:
            d = rng.standard_normal(hd); d /= np.linalg.norm(d)
            k[3, :, :] = d * 12.0
            q[-1, :, :] = d * 12.0

    c = _attention_case(rng, [5900, 0], [300, 64], n_q, n_kv, hd, "bfloat16", spike=spike)
    assert rel_err(as64(_run_tc(c, [300, 64], n_q, n_kv, hd, halves=halves)), c["ref"]) < 8e-3
    c = _attention_case(rng, [5900], [300], n_q, n_kv, hd, "bfloat16", window=1000, spike=spike)
    assert rel_err(as64(_run_tc(c, [300], n_q, n_kv, hd, window=1000, halves=halves)), c["ref"]) < 8e-3


def _run_stream(c, n_q, n_kv, hd, window=0, pad_rows=0, whole_pages=False):
    """attention_stream on the case's new tokens (one per sequence), optionally with padding rows appended."""
    from stratum_b200 import kernels as K
    T = c["T"]
    qkv, pos, seq = c["qkv"], c["pos"], c["seq"]
    if pad_rows:
        qkv = torch.cat([qkv, torch.full((pad_rows, qkv.shape[1]), 7.0, dtype=qkv.dtype, device="cuda")])
        pos = torch.cat([pos, torch.zeros(pad_rows, dtype=torch.int32, device="cuda")])
        seq = torch.cat([seq, torch.full((pad_rows,), -1, dtype=torch.int32, device="cuda")])
    out = torch.zeros(T + pad_rows, n_q * hd, dtype=torch.bfloat16, device="cuda")
    K.attention_stream(qkv, c["kc"], c["vc"], pos, seq, c["table"], out, n_q, n_kv, hd, 64, window,
                       1.0 / math.sqrt(hd), whole_pages=whole_pages)
    K.check_status()
    # when the kernels after it may start changes nothing in the result
    early = torch.zeros_like(out)
    K.attention_stream(qkv, c["kc"], c["vc"], pos, seq, c["table"], early, n_q, n_kv, hd, 64, window,
                       1.0 / math.sqrt(hd), late_trigger=False, whole_pages=whole_pages)
    K.check_status()
    assert torch.equal(early, out)
    return out


@pytest.mark.parametrize("n_q,n_kv,hd,whole", [(8, 2, 128, False), (4, 4, 64, False), (32, 8, 128, False),
                                               (8, 1, 64, False), (3, 1, 128, False), (12, 2, 128, False),
                                               (4, 4, 64, True), (8, 1, 64, True), (32, 8, 64, True), (6, 2, 64, True)])
def test_attention_stream_decode_steps(n_q, n_kv, hd, whole):
    """whole: eight warps that take whole pages in turn (heads of 64), else four warps a quarter of every page."""
    from functools import partial
    _run_stream = partial(globals()["_run_stream"], whole_pages=whole)
    rng = np.random.default_rng(hd + n_q + 3)
    # unequal sequences: one short of a page end, one just past it, a long one, a single key, a few pages
    lens = [63, 64, 1500, 0, 300, 129]
    c = _attention_case(rng, lens, [1] * len(lens), n_q, n_kv, hd, "bfloat16")
    out = _run_stream(c, n_q, n_kv, hd, pad_rows=2)
    assert rel_err(as64(out[:c["T"]]), c["ref"]) < 8e-3
    assert float(out[c["T"]:].float().abs().sum()) == 0.0                 # padding rows are left alone
    # one long sequence alone: every (sequence, kv head) is shared by many CTAs
    c = _attention_case(rng, [5000], [1], n_q, n_kv, hd, "bfloat16")
    assert rel_err(as64(_run_stream(c, n_q, n_kv, hd)), c["ref"]) < 8e-3
    # many short sequences: many whole (sequence, kv head) runs per CTA
    lens = [int(x) for x in rng.integers(0, 200, size=70)]
    c = _attention_case(rng, lens, [1] * len(lens), n_q, n_kv, hd, "bfloat16")
    assert rel_err(as64(_run_stream(c, n_q, n_kv, hd)), c["ref"]) < 8e-3
    if whole and n_kv == 8:
        # many long sequences: every SM streams a hundred pages or more, its warps far apart in the ring
        lens = [int(x) for x in rng.integers(2500, 3000, size=48)]
        c = _attention_case(rng, lens, [1] * len(lens), n_q, n_kv, hd, "bfloat16")
        for _ in range(3):
            assert rel_err(as64(_run_stream(c, n_q, n_kv, hd)), c["ref"]) < 8e-3


@pytest.mark.parametrize("whole", [False, True])
def test_attention_stream_far_key_and_window_edge(whole):
    from functools import partial
    _run_stream = partial(globals()["_run_stream"], whole_pages=whole)
    rng = np.random.default_rng(43)
    n_q, n_kv, hd = 4, 2, 64
    far = {0: 3, 1: 517}

    def spike(s, q, k, v):
        d = rng.standard_normal(hd); d /= np.linalg.norm(d)
        k[far[s], :, :] = d * 12.0
        q[-1, :, :] = d * 12.0

    c = _attention_case(rng, [699, 600], [1, 1], n_q, n_kv, hd, "bfloat16", spike=spike)
    out = _run_stream(c, n_q, n_kv, hd)
    assert rel_err(as64(out), c["ref"]) < 8e-3
    W, p = 100, 400

    def edge(s, q, k, v):                     # sequence 0: the spiked key is the last one inside the window;
        d = rng.standard_normal(hd); d /= np.linalg.norm(d)          # sequence 1: the first one outside
        k[p - W + 1 if s == 0 else p - W, :, :] = d * 12.0
        q[-1, :, :] = d * 12.0

    c = _attention_case(rng, [p, p], [1, 1], n_q, n_kv, hd, "bfloat16", window=W, spike=edge)
    out = _run_stream(c, n_q, n_kv, hd, window=W)
    assert rel_err(as64(out), c["ref"]) < 8e-3


def test_attention_stream_refuses_what_it_cannot_do():
    from stratum_b200 import kernels as K
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device="cuda")   # noqa: E731
    with pytest.raises(K.KernelError, match="shape"):                       # head size 96
        K.attention_stream(z(1, 3 * 96), z(1, 1, 64, 96), z(1, 1, 64, 96), z(1, dt=torch.int32), z(1, dt=torch.int32),
                           z(1, 1, dt=torch.int32), z(1, 96), 1, 1, 96, 64, 0, 1.0)
    with pytest.raises(K.KernelError, match="shape"):                       # 16 heads per kv head
        K.attention_stream(z(1, 18 * 64), z(1, 1, 64, 64), z(1, 1, 64, 64), z(1, dt=torch.int32),
                           z(1, dt=torch.int32), z(1, 1, dt=torch.int32), z(1, 16 * 64), 16, 1, 64, 64, 0, 1.0)
    with pytest.raises(K.KernelError, match="shape"):                       # whole pages per warp: heads of 64 only
        K.attention_stream(z(1, 3 * 128), z(1, 1, 64, 128), z(1, 1, 64, 128), z(1, dt=torch.int32),
                           z(1, dt=torch.int32), z(1, 1, dt=torch.int32), z(1, 128), 1, 1, 128, 64, 0, 1.0,
                           whole_pages=True)


def test_attention_mma_refuses_head_sizes_it_cannot_do():
    from stratum_b200 import kernels as K
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device="cuda")   # noqa: E731
    with pytest.raises(K.KernelError, match="shape"):
        K.attention_mma(z(1, 3 * 256), z(1, 1, 64, 256), z(1, 1, 64, 256), z(1, dt=torch.int32), z(1, dt=torch.int32),
                        z(1, 1, dt=torch.int32), None, 1, z(1, 256), None, None, 1, 1, 256, 64, 0, 1.0, 1, 0)


def test_fill_normal_is_seeded_and_normal():
    from stratum_b200 import kernels as K
    a = torch.empty(1 << 20, dtype=torch.float32, device="cuda")
    b = torch.empty(1 << 20, dtype=torch.float32, device="cuda")
    K.fill_normal(a, 5, 0.02); K.fill_normal(b, 5, 0.02)
    assert torch.equal(a, b)
    K.fill_normal(b, 6, 0.02)
    assert not torch.equal(a, b)
    assert abs(float(a.mean())) < 1e-4 and abs(float(a.std()) - 0.02) < 2e-4
    c = torch.empty(1 << 20, dtype=torch.bfloat16, device="cuda")
    K.fill_normal(c, 5, 0.02)
    assert torch.equal(c, a.bfloat16())
