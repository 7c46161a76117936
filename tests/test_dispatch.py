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
    assert _attention_call(recorded, bf, 80, 6, 2, 8, True)[0] == "attention_mma"            # head size 80
    assert _attention_call(recorded, bf, 128, 12, 1, 8, True)[0] == "attention_mma"          # 12 heads per kv head
    assert _attention_call(recorded, bf, 128, 32, 8, 300, False)[0] == "attention_tc"
    assert _attention_call(recorded, bf, 128, 3, 1, 300, False)[0] == "attention_tile"       # 128 % 3 != 0
    assert _attention_call(recorded, bf, 96, 8, 2, 300, False)[0] == "attention_tile"
