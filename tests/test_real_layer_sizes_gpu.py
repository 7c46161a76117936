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
