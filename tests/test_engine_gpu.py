"""The engine against the plain oracle on the GPU: whole prompts, token by token, unequal batches."""
import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, load_plain, make_model_dir, plain_logits, rand_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def _engine(path, dtype, max_tokens=2048):
    from stratum_b200.engine import Engine, load_model
    model, cfg = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    return Engine(model, max_tokens=max_tokens), cfg


@pytest.fixture(scope="module", params=[(n, d) for n in "ABCDEFG" for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    path = make_model_dir(str(tmp_path_factory.mktemp(f"tiny{name}_{dtype}")), TINY[name], seed=ord(name),
                          dtype=dtype)
    cfg, w = load_plain(path)
    engine, _ = _engine(path, dtype)
    return name, dtype, cfg, w, engine


def test_whole_prompt_all_positions(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine = setup
    rng = np.random.default_rng(1)
    for n in (1, 5, 64, 65, 150):
        toks = rand_tokens(rng, n, cfg["vocab_size"])
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        engine.release(slot)
        assert_close(got, plain_logits(cfg, w, toks), dtype, f"{name} whole n={n}")
    engine.cache.check()


def test_last_tokens_one_by_one(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine = setup
    rng = np.random.default_rng(2)
    n, tail = 100, 32
    toks = rand_tokens(rng, n, cfg["vocab_size"])
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([StepEntry(slot, toks[:n - tail], [n - tail - 1])]).cpu().numpy()]
    for i in range(n - tail, n):
        got.append(engine.step([StepEntry(slot, [toks[i]], [0])]).cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref[n - tail - 1:], dtype, f"{name} token by token")


def test_unequal_batches_slots_reused(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine = setup
    rng = np.random.default_rng(3)
    V = cfg["vocab_size"]
    for batch_no, lens in enumerate([(5, 9, 12), (1, 17), (70, 3, 33, 64)]):
        prompts = [rand_tokens(rng, n, V) for n in lens]
        extra = [rand_tokens(rng, k, V) for k in (3 + 2 * i for i in range(len(lens)))]   # unequal decode lengths
        refs = [plain_logits(cfg, w, p + e) for p, e in zip(prompts, extra)]
        slots = [engine.acquire() for _ in lens]
        out = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
        for i, p in enumerate(prompts):
            assert_close(out[i], refs[i][len(p) - 1], dtype, f"{name} batch {batch_no} prompt {i}")
        live = list(range(len(lens)))
        step = 0
        while live:
            entries = [StepEntry(slots[i], [extra[i][step]], [0]) for i in live]
            out = engine.step(entries).cpu().numpy()
            for row, i in enumerate(live):
                assert_close(out[row], refs[i][len(prompts[i]) + step], dtype,
                             f"{name} batch {batch_no} seq {i} decode {step}")
            step += 1
            for i in list(live):
                if step >= len(extra[i]):          # shorter requests end earlier
                    engine.release(slots[i])
                    live.remove(i)
        engine.cache.check()
    assert engine.cache.tokens_held() == 0


def test_long_decoding_crosses_pages_and_buckets(setup):
    """A short prompt, then some hundreds of tokens one by one: positions cross several pages."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine = setup
    rng = np.random.default_rng(4)
    n = 330 if name != "C" else 200
    toks = rand_tokens(rng, n, cfg["vocab_size"])
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([StepEntry(slot, toks[:3], [2])]).cpu().numpy()]
    check = set(range(3, n, 37)) | {63, 64, 65, 127, 128, 129, n - 1}
    for i in range(3, n):
        out = engine.step([StepEntry(slot, [toks[i]], [0] if i in check else [])])
        if i in check:
            got.append(out.cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref[[2] + sorted(check)], dtype, f"{name} long decode")


def test_first_tokens_of_a_sequence(setup):
    """Position 0 alone, then 1, 2, 3: the first tokens see the least context and have no page behind them."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine = setup
    rng = np.random.default_rng(6)
    toks = rand_tokens(rng, 4, cfg["vocab_size"])
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = np.concatenate([engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks])
    engine.release(slot)
    assert_close(got, ref, dtype, f"{name} first tokens")


def test_errors_leave_the_engine_unchanged(setup):
    from stratum_b200.cache import CacheFull
    from stratum_b200.engine import StepEntry, StepError
    name, dtype, cfg, w, engine = setup
    slot = engine.acquire()
    with pytest.raises(StepError, match="outside the vocabulary"):
        engine.step([StepEntry(slot, [cfg["vocab_size"]], [0])])
    with pytest.raises(StepError, match="wanted place"):
        engine.step([StepEntry(slot, [1, 2], [2])])
    with pytest.raises(StepError, match="not held"):
        engine.step([StepEntry(slot + 7, [1], [0])])
    with pytest.raises(CacheFull):
        engine.step([StepEntry(slot, [1] * (64 * 33), [])])      # beyond the 2048 tokens this engine holds
    assert engine.length(slot) == 0
    engine.release(slot)
    engine.cache.check()
