"""Random tiny Llama configurations (a fixed seed) through the engine against the plain oracle: head sizes from 16
to 256 in steps of 16, one to four kv heads in groups of 1 to 12, widths and vocabularies that are no power of two,
every rope scaling, pair layout and partial rotation, biases, a tied head; now and then sizes that reach the
wide-matrix kernels.  Each: a prompt whole and its tail token by token, then an unequal batch of up to 70 requests
whose shorter ones end earlier."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_close, load_plain, make_model_dir, plain_logits, rand_tokens

pytestmark = pytest.mark.gpu

SEED, COUNT = 7, 12


def _random_config(rng):
    hd = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256]))
    n_kv = int(rng.integers(1, 5))
    group = int(rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 12]))
    if hd >= 160:
        group = min(group, 4)
    n_q = n_kv * group
    hidden = int(rng.choice([64, 72, 96, 102, 136, 192, 200, 264, 320]))
    inter = int(rng.choice([96, 112, 150, 176, 200, 328, 520, 1032]))
    vocab = int(rng.choice([97, 200, 256, 331, 517, 1000, 2049]))
    if rng.integers(0, 4) == 0:      # sizes that reach the wide-matrix kernels
        hidden = int(rng.choice([1024, 2048, 2056, 1536]))
        inter = int(rng.choice([2816, 4096, 2200, 1032]))
        vocab = int(rng.choice([4099, 2304, 8200]))
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": int(rng.integers(1, 4)), "hidden_size": hidden, "intermediate_size": inter,
        "num_attention_heads": n_q, "num_key_value_heads": n_kv, "head_dim": hd, "vocab_size": vocab,
        "rms_norm_eps": float(rng.choice([1e-4, 1e-5, 1e-6])), "rope_theta": float(rng.choice([1000.0, 10000.0, 500000.0])),
        "max_position_embeddings": 2048,
        "tie_word_embeddings": bool(rng.integers(0, 2)), "attention_bias": bool(rng.integers(0, 2)),
        "mlp_bias": bool(rng.integers(0, 2)), "hidden_act": "silu",
    }
    kind = rng.choice(["none", "linear", "llama3", "yarn"])
    if kind == "linear":
        cfg["rope_scaling"] = {"rope_type": "linear", "factor": 2.0}
    elif kind == "llama3":
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 64}
    elif kind == "yarn":
        cfg["rope_scaling"] = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32,
                               "beta_fast": 8.0, "beta_slow": 0.5}
    if rng.integers(0, 3) == 0:
        cfg["rope_interleaved"] = True
    if rng.integers(0, 3) == 0 and hd >= 32:
        cfg["rope_dim"] = hd // 2 if (hd // 2) % 2 == 0 else hd
    return cfg


def _run_one(idx, cfg, dtype, rng, tmp):
    from stratum_b200.engine import Engine, StepEntry, load_model
    path = make_model_dir(os.path.join(tmp, f"m{idx}_{dtype}"), cfg, seed=idx, dtype=dtype)
    c, w = load_plain(path)
    m, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    engine = Engine(m, max_tokens=16384)
    V = c["vocab_size"]
    # whole + tail
    n = int(rng.choice([1, 2, 17, 63, 64, 65, 100, 129, 200, 300, 420]))
    tail = min(n - 1, int(rng.integers(0, 6)))
    toks = rand_tokens(rng, n, V)
    ref = plain_logits(c, w, toks)
    slot = engine.acquire()
    head = n - tail
    want = sorted(set([0, head - 1, head // 2]))
    got = engine.step([StepEntry(slot, toks[:head], want)]).cpu().numpy()
    assert_close(got, ref[want], dtype, f"whole n={n}")
    for i in range(head, n):
        got = engine.step([StepEntry(slot, [toks[i]], [0])]).cpu().numpy()
        assert_close(got[0], ref[i], dtype, f"tail {i}")
    engine.release(slot)
    # unequal batch
    count = int(rng.choice([2, 3, 5, 9, 17, 33, 70]))
    lens = [int(x) for x in rng.integers(1, 40, size=count)]
    lens[0] = int(rng.choice([64, 70, 128, 150]))
    extra_n = [1 + int(x) for x in rng.integers(0, 3, size=count)]
    prompts = [rand_tokens(rng, k, V) for k in lens]
    extra = [rand_tokens(rng, k, V) for k in extra_n]
    check = sorted(set([0, count - 1] + [int(x) for x in rng.integers(0, count, size=3)]))
    refs = {i: plain_logits(c, w, prompts[i] + extra[i]) for i in check}
    slots = [engine.acquire() for _ in lens]
    out = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
    for i in check:
        assert_close(out[i], refs[i][lens[i] - 1], dtype, f"batch prompt {i} of {count}")
    live, step = list(range(count)), 0
    while live:
        out = engine.step([StepEntry(slots[i], [extra[i][step]], [0]) for i in live]).cpu().numpy()
        for row, i in enumerate(live):
            if i in refs:
                assert_close(out[row], refs[i][lens[i] + step], dtype, f"batch seq {i} of {count} decode {step}")
        step += 1
        for i in list(live):
            if step >= extra_n[i]:
                engine.release(slots[i])
                live.remove(i)
    engine.cache.check()
    assert engine.cache.tokens_held() == 0


@pytest.mark.parametrize("idx", range(COUNT))
def test_random_configuration(idx, tmp_path):
    rng = np.random.default_rng(SEED)
    for _ in range(idx + 1):                       # the idx-th configuration of the seed's sequence
        cfg = _random_config(rng)
    for dtype in ("float32", "bfloat16"):
        _run_one(idx, cfg, dtype, np.random.default_rng(SEED * 1000 + idx), str(tmp_path))
