"""Which kernel a call is given to: the rules of parts/gemm_dispatch.py and parts/attention_dispatch.py, with the
launchers replaced by recorders (no GPU needed)."""
import types

import pytest
import torch


@pytest.fixture
def recorded(monkeypatch):
    from stratum_b200 import kernels as K
    calls = []

    def recorder(name):
        def f(*args, **kwargs):
            calls.append((name, args, kwargs))
        return f

    for name in ("gemm_skinny", "gemm_tc", "linear_simple", "swiglu", "attention_simple", "attention_stream",
                 "attention_mma", "attention_tc", "attention_tile"):
        monkeypatch.setattr(K, name, recorder(name))
    return calls


def _xw(rows, n, k, dtype=torch.bfloat16):
    return torch.zeros(rows, k, dtype=dtype), torch.zeros(n, k, dtype=dtype), torch.zeros(rows, n, dtype=dtype)


def test_matrix_product_rules(recorded):
    from stratum_b200.parts import gemm_dispatch as G
    small, large = (4096, 4096), (28672, 4096)                  # 16.8 M and 117 M weights
    assert small[0] * small[1] < G.STREAMK_MIN_WEIGHTS <= large[0] * large[1]
    for rows, shape, want in ((1, small, "gemm_skinny"), (G.SKINNY_MAX_ROWS, small, "gemm_skinny"),
                              (G.SKINNY_MAX_ROWS + 1, small, "gemm_tc"), (1, large, "gemm_tc"),
                              (2048, small, "gemm_tc")):
        recorded.clear()
        x, w, out = _xw(rows, *shape)
        G.run(x, w, None, out, G.STORE)
        assert [c[0] for c in recorded] == [want], (rows, shape)
    # float32 is the true 32-bit path whatever the shape; so is a row pitch that no 16-byte copy can start on
    for x, w, out in (_xw(8, 4096, 4096, torch.float32), _xw(8, 64, 20)):
        recorded.clear()
        G.run(x, w, None, out, G.ADD_TO_F32)
        assert [c[0] for c in recorded] == ["linear_simple"]
    # SwiGLU without a tensor-core kernel: the product, then the activation
    recorded.clear()
    x, w, _ = _xw(3, 64, 20)
    G.run(x, w, None, torch.zeros(3, 32, dtype=torch.bfloat16), G.SWIGLU)
    assert [c[0] for c in recorded] == ["linear_simple", "swiglu"]


def _attention_call(recorded, dtype, head_dim, n_heads, n_kv, n_tokens, all_single):
    from stratum_b200.parts import attention_dispatch as A
    recorded.clear()
    att = types.SimpleNamespace(head_dim=head_dim, n_heads=n_heads, n_kv_heads=n_kv, window=0, scale=1.0,
                                runtime=types.SimpleNamespace(scratch=lambda name, n, dt: torch.zeros(n, dtype=dt)))
    width = (n_heads + 2 * n_kv) * head_dim
    qkv = torch.zeros(n_tokens, width, dtype=dtype)
    cache = types.SimpleNamespace(k=None, v=None, block_table=None)
    step = types.SimpleNamespace(all_single=all_single, n_tokens=n_tokens, max_len=300, token_pos=None,
                                 token_seq=None, query_blocks=lambda n: None)
    A.run(att, qkv, cache, step, torch.zeros(n_tokens, n_heads * head_dim, dtype=dtype))
    assert len(recorded) == 1
    return recorded[0]


def test_attention_rules(recorded):
    bf, f32 = torch.bfloat16, torch.float32
    assert _attention_call(recorded, f32, 128, 32, 8, 8, True)[0] == "attention_simple"
    assert _attention_call(recorded, bf, 256, 4, 2, 8, True)[0] == "attention_simple"        # head size above 128
    name, _, kw = _attention_call(recorded, bf, 128, 32, 8, 8, True)
    assert name == "attention_stream" and kw["late_trigger"] is True
    assert _attention_call(recorded, bf, 64, 8, 2, 2, True)[2]["late_trigger"] is False     # one or two sequences
    # heads of 64: whole pages per warp once an SM gets more than a few pages (here 5 pages a sequence and kv head)
    assert _attention_call(recorded, bf, 64, 8, 2, 100, True)[2]["whole_pages"] is False    # 1,000 pages
    assert _attention_call(recorded, bf, 64, 32, 8, 64, True)[2]["whole_pages"] is True     # 2,560 pages
    assert _attention_call(recorded, bf, 128, 32, 8, 64, True)[2]["whole_pages"] is False
    assert _attention_call(recorded, bf, 80, 6, 2, 8, True)[0] == "attention_mma"            # head size 80
    assert _attention_call(recorded, bf, 128, 12, 1, 8, True)[0] == "attention_mma"          # 12 heads per kv head
    assert _attention_call(recorded, bf, 128, 32, 8, 300, False)[0] == "attention_tc"
    assert _attention_call(recorded, bf, 128, 3, 1, 300, False)[0] == "attention_tile"       # 128 % 3 != 0
    assert _attention_call(recorded, bf, 96, 8, 2, 300, False)[0] == "attention_tile"


def test_extra_epilogue_rules(recorded, monkeypatch):
    """Where a product carries more than its basic epilogue: rows of a handed-over norm and the query/key/value
    epilogue go to the tensor-core kernel or are refused; a Handover is honoured where the product's tiles fill the SMs
    (hands_over); prompt attention gets query tiles of 256 rows."""
    from stratum_b200 import kernels as K
    from stratum_b200.parts import gemm_dispatch as G
    from stratum_b200.parts.base import Handover, NormedRows, Runtime
    from stratum_b200.parts.linear import ADD_TO_F32, STORE, Linear
    small = (4096, 4096)
    x, w, out = _xw(4, *small)
    assert not G.takes_tensor_cores(x, w, extras=False) and G.takes_tensor_cores(x, w, extras=True)
    G.run(x, w, None, out, G.STORE, extra=object())               # few rows, small matrix: still the tensor cores
    assert [c[0] for c in recorded] == ["gemm_tc"]
    with pytest.raises(K.KernelError, match="only the tensor-core kernel"):
        G.run(*_xw(4, 64, 20)[:2], None, torch.zeros(4, 64, dtype=torch.bfloat16), G.STORE, extra=object())
    # Linear: the residual add honours a Handover only with enough rows
    monkeypatch.setattr(K, "_need", lambda *a, **k: None)        # (the tensors of this test live on the host)
    monkeypatch.setattr(K, "gemm_tc", lambda *a, **k: (recorded.append(("gemm_tc", a, k)), 7)[1])
    rt = types.SimpleNamespace(dtype=torch.bfloat16, device="cpu",
                               empty=lambda *shape, dtype=torch.bfloat16: torch.zeros(shape, dtype=dtype))
    lin = Linear(rt, torch.zeros(4096, 4096, dtype=torch.bfloat16))
    gain = torch.ones(4096)
    assert not G.hands_over(768, 4096) and G.hands_over(769, 4096)          # 48 and 64 tiles of 256 x 256
    assert not G.hands_over(1024, 2048) and G.hands_over(2048, 2048)
    monkeypatch.setattr(G, "HANDOVER_MIN_TILES", 1)
    for rows, honoured in ((G.HANDOVER_MIN_ROWS - 1, False), (G.HANDOVER_MIN_ROWS, True)):
        recorded.clear()
        ask = Handover(gain, 4096, 1e-5)
        lin(torch.zeros(rows, 4096, dtype=torch.bfloat16), out=torch.zeros(rows, 4096), mode=ADD_TO_F32, emit=ask)
        assert (ask.result is not None) == honoured
        assert [c[0] for c in recorded] == ["gemm_tc"]
        assert recorded[0][1][4] == (K.EPI_ADD_F32_EMIT if honoured else K.EPI_ADD_F32)
        if honoured:
            r = ask.result
            assert isinstance(r, NormedRows) and r.parts == 7 and r.x.shape == (rows, 4096) and r.size == 4096
            # and the product behind the norm takes them as rows to be scaled
            recorded.clear()
            lin(r, mode=STORE)
            assert recorded[0][1][4] == K.EPI_STORE and recorded[0][1][5].c.norm_parts == 7
    # prompt attention: a CTA's query tile is 256 rows (2 x 128 / group size tokens), 128 when asked for
    from stratum_b200.parts import attention_dispatch as A
    sizes = []
    att = types.SimpleNamespace(head_dim=128, n_heads=32, n_kv_heads=8, window=0, scale=1.0, runtime=None)
    step = types.SimpleNamespace(all_single=False, n_tokens=300, max_len=300, token_pos=None, token_seq=None,
                                 query_blocks=lambda n: sizes.append(n))
    cache = types.SimpleNamespace(k=None, v=None, block_table=None)
    for env, tokens in ((None, 64), ("1", 32)):
        if env:
            monkeypatch.setenv("STRATUM_ATTENTION_HALVES", env)
        recorded.clear()
        A.run(att, torch.zeros(300, 48 * 128, dtype=torch.bfloat16), cache, step, torch.zeros(300, 4096, dtype=torch.bfloat16))
        assert recorded[0][0] == "attention_tc" and sizes[-1] == tokens
