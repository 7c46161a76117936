"""The engine against the plain oracle at the layer sizes of Llama-3.1-8B, Llama-3.2-1B and Llama-2-7B (one or two layers, a small vocabulary so that
the float64 oracle stays quick): the kernels meet K = 4096 and 14336, 32 heads of 128 in groups of 4, and every
form of the matrix product (one and two rows, 3 to 16, 17 to 32, 33 to 64, prompts) in both dtypes."""
import numpy as np
import pytest
import torch

from helpers import assert_close, load_plain, make_model_dir, plain_logits, rand_tokens

pytestmark = pytest.mark.gpu

REAL_LAYERS = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 4096, "intermediate_size": 14336,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 2048,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False, "hidden_act": "silu",
}


# the same for the layer sizes of Llama-3.2-1B (heads of 64, tied head) and Llama-2-7B (as many kv heads as heads)
REAL_LAYERS_1B = dict(REAL_LAYERS, hidden_size=2048, intermediate_size=8192, head_dim=64, tie_word_embeddings=True,
                      rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                    "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})
REAL_LAYERS_7B = dict(REAL_LAYERS, num_hidden_layers=1, intermediate_size=11008, num_key_value_heads=32,
                      rope_theta=10000.0, rope_scaling=None, max_position_embeddings=4096)
SHAPES = {"llama3.1-8b": REAL_LAYERS, "llama3.2-1b": REAL_LAYERS_1B, "llama2-7b": REAL_LAYERS_7B}


@pytest.fixture(scope="module", params=sorted(SHAPES))
def model(request, tmp_path_factory):
    raw = {k: v for k, v in SHAPES[request.param].items() if v is not None}
    path = make_model_dir(str(tmp_path_factory.mktemp("real_layers")), raw, seed=21, dtype="bfloat16")
    cfg, w = load_plain(path)
    return path, cfg, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_in_every_cut(model, dtype):
    from stratum_b200.engine import Engine, StepEntry, load_model
    path, cfg, w = model
    m, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    engine = Engine(m, max_tokens=8192)
    rng = np.random.default_rng(5)
    V = cfg["vocab_size"]
    # one request whole, then its last tokens one by one
    n, tail = 150, 12
    toks = rand_tokens(rng, n, V)
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks, [0, 63, 64, n - 1])]).cpu().numpy()
    engine.release(slot)
    assert_close(got, ref[[0, 63, 64, n - 1]], dtype, "whole")
    slot = engine.acquire()
    got = [engine.step([StepEntry(slot, toks[:n - tail], [n - tail - 1])]).cpu().numpy()]
    for i in range(n - tail, n):
        got.append(engine.step([StepEntry(slot, [toks[i]], [0])]).cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref[n - tail - 1:], dtype, "token by token")
    # batches of unequal lengths, of 2, 5, 20 and 40 requests: shorter requests end earlier, slots are reused
    for batch_no, count in enumerate((2, 5, 20, 40)):
        lens = [int(x) for x in rng.integers(1, 30, size=count)]
        lens[0] = 70                                          # one prompt longer than a page
        extra_n = [1 + (i % 3) for i in range(count)]
        prompts = [rand_tokens(rng, k, V) for k in lens]
        extra = [rand_tokens(rng, k, V) for k in extra_n]
        refs = [plain_logits(cfg, w, p + e) for p, e in zip(prompts, extra)]
        slots = [engine.acquire() for _ in lens]
        out = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
        for i, p in enumerate(prompts):
            assert_close(out[i], refs[i][len(p) - 1], dtype, f"batch {batch_no} prompt {i}")
        live, step = list(range(count)), 0
        while live:
            out = engine.step([StepEntry(slots[i], [extra[i][step]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                assert_close(out[row], refs[i][lens[i] + step], dtype, f"batch {batch_no} seq {i} decode {step}")
            step += 1
            for i in list(live):
                if step >= extra_n[i]:
                    engine.release(slots[i])
                    live.remove(i)
        engine.cache.check()
    assert engine.cache.tokens_held() == 0


@pytest.mark.parametrize("forced", [False, True])
def test_fused_epilogues_at_model_level(model, forced, monkeypatch):
    """The matrix products' extra epilogue work inside a model (bfloat16): rotation and cache write on the
    projection's epilogue, and norms handed over to the product in front of them.  By default the first serves
    decode steps and the second prompts whose tiles fill the SMs (from 769 rows on at these widths); `forced` turns both on for every step, so that
    every form of the kernel meets them (prompts of 300 and 40 tokens, batches of 3 and 20 single tokens)."""
    from stratum_b200 import kernels as K
    from stratum_b200.engine import Engine, StepEntry, load_model
    from stratum_b200.parts import gemm_dispatch
    path, cfg, w = model
    if forced:
        monkeypatch.setenv("STRATUM_FUSE_ROPE", "2")
        monkeypatch.setattr(gemm_dispatch, "HANDOVER_MIN_ROWS", 1)
        monkeypatch.setattr(gemm_dispatch, "HANDOVER_MIN_TILES", 1)
        monkeypatch.setattr(gemm_dispatch, "SKINNY_MAX_ROWS", 0)        # every product on the tensor-core kernel
    m, _ = load_model(path, torch.bfloat16, "cuda")
    engine = Engine(m, max_tokens=4096)
    rng = np.random.default_rng(11)
    V = cfg["vocab_size"]
    calls = {"rope_store": 0, "rmsnorm": 0}
    for name in calls:
        orig = getattr(K, name)
        monkeypatch.setattr(K, name, (lambda o, n: lambda *a, **k: (calls.__setitem__(n, calls[n] + 1), o(*a, **k))[1])(orig, name))
    lens = [300, 40, 7] + [int(x) for x in rng.integers(1, 20, size=17)]
    seqs = [rand_tokens(rng, n + 3, V) for n in lens]
    refs = [plain_logits(cfg, w, s) for s in seqs[:3]]
    slots = [engine.acquire() for _ in lens]
    got = engine.step([StepEntry(slots[0], seqs[0][:300], [0, 150, 299])]).cpu().numpy()      # 300 rows: pairs of CTAs
    assert_close(got, refs[0][[0, 150, 299]], "bfloat16", "prompt of 300")
    n_layers = cfg["num_hidden_layers"]
    if forced:
        assert calls["rope_store"] == 0                       # rotation rode on the projection
    # handed over: only the first layer's first norm and the final one run a kernel of their own
    assert calls["rmsnorm"] == (2 if forced else 2 * n_layers + 1)
    got = engine.step([StepEntry(s, q[:n], [n - 1]) for s, q, n in zip(slots[1:], seqs[1:], lens[1:])]).cpu().numpy()
    assert_close(got[:2], np.stack([refs[1][39], refs[2][6]]), "bfloat16", "prompts of 40 and 7 among others")
    before = dict(calls)
    for k in range(3):                                         # three tokens each for three sequences, then for all
        live = range(3) if k < 2 else range(len(lens))
        ropes = calls["rope_store"]
        got = engine.step([StepEntry(slots[i], [seqs[i][lens[i] + k]], [0]) for i in live]).cpu().numpy()
        assert_close(got[:3], np.stack([refs[i][lens[i] + k] for i in range(3)]), "bfloat16", f"decode {k}")
        if forced or k == 2:          # decode steps whose projection the tensor-core kernel takes (here: 20 rows)
            assert calls["rope_store"] == ropes                # rotation rode on the projection
    if forced:
        assert calls["rmsnorm"] == before["rmsnorm"] + 3 * 2
    else:
        assert calls["rmsnorm"] == before["rmsnorm"] + 3 * (2 * n_layers + 1)
    for s in slots:
        engine.release(s)
    engine.cache.check()
