"""Prompt steps replayed as captured graphs against the same steps launch by launch and against the plain oracle:
batches of unequal prompts padded in tokens and in sequences, a shape used again by another batch, chunks that
continue sequences, decoding afterwards from the cache the replayed steps wrote."""
import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, load_plain, make_model_dir, plain_logits, rand_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("G", "float32"), ("B", "bfloat16"), ("D", "bfloat16"),
                                        ("E", "bfloat16"), ("F", "bfloat16")])
def test_replayed_prompt_steps(tmp_path, name, dtype):
    from stratum_b200 import StepEntry, Stratum
    path = make_model_dir(str(tmp_path / "m"), TINY[name], seed=41, dtype=dtype)
    cfg, w = load_plain(path)
    V = cfg["vocab_size"]
    replayed = Stratum(path, dtype=dtype, max_tokens=4096)
    by_hand = Stratum(path, dtype=dtype, max_tokens=4096, use_graphs=False)
    assert replayed.prompt_graphs is not None and replayed.prompt_graphs.enabled and by_hand.prompt_graphs is None
    replayed.prompt_graphs.capture_after = 0             # (by default a shape is captured at its second sighting)
    rng = np.random.default_rng(7)
    # (5, 70, 130) and (70, 4, 131) share a shape (256 tokens, 4 sequences); 64 tokens fill theirs exactly
    batches = [(5, 70, 130), (64,), (1, 200, 3, 17, 40), (70, 4, 131), (2, 1)]
    steps = 0
    for lens in batches:
        seqs = [rand_tokens(rng, n + 12, V) for n in lens]
        refs = [plain_logits(cfg, w, s) for s in seqs]
        both = []
        for llm in (replayed, by_hand):
            slots = [llm.acquire() for _ in lens]
            out = [llm.step([StepEntry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)])]
            # a chunk that continues every sequence, then two single tokens
            out.append(llm.step([StepEntry(s, q[n:n + 10], [9]) for s, q, n in zip(slots, seqs, lens)]))
            for k in (10, 11):
                ids, _, lg = llm.decode_step(slots, [q[n + k] for q, n in zip(seqs, lens)], with_logits=True)
                out.append(lg.clone())
            both.append([o.cpu().numpy() for o in out])
            for s in slots:
                llm.release(s)
            llm.engine.cache.check()
        steps += 2
        (p_r, c_r, d0_r, d1_r), (p_h, c_h, d0_h, d1_h) = both
        for i, n in enumerate(lens):
            assert_close(p_r[i], refs[i][n - 1], dtype, f"{lens} prompt {i}")
            assert_close(c_r[i], refs[i][n + 9], dtype, f"{lens} chunk {i}")
            assert_close(d0_r[i], refs[i][n + 10], dtype, f"{lens} decode {i}")
            assert_close(d1_r[i], refs[i][n + 11], dtype, f"{lens} decode {i}")
        if dtype == "float32":              # the same kernels on the same rows in the same order: the same bits
            assert np.array_equal(p_r, p_h) and np.array_equal(c_r, c_h)
            assert np.array_equal(d0_r, d0_h) and np.array_equal(d1_r, d1_h)
    pg = replayed.prompt_graphs
    assert pg.replays == steps
    # seven shapes in ten steps (a shape is captured again when a scratch buffer it points into was regrown)
    assert len(pg.graphs) == 7 and pg.captures < steps
    assert replayed.engine.cache.tokens_held() == 0


def test_what_is_replayed_and_what_is_not(tmp_path):
    from stratum_b200 import StepEntry, Stratum
    from stratum_b200.engine.graphs import padded_seqs, padded_tokens
    assert [padded_tokens(n, 2048) for n in (1, 64, 65, 512, 513, 2048, 2049)] == [64, 64, 128, 512, 640, 2048, None]
    assert [padded_seqs(n) for n in (1, 2, 3, 8, 9)] == [1, 2, 4, 8, 16]
    path = make_model_dir(str(tmp_path / "m"), TINY["A"], seed=3, dtype="float32")
    llm = Stratum(path, dtype="float32", max_tokens=8192)
    pg = llm.prompt_graphs
    a, b = llm.acquire(), llm.acquire()
    toks = list(range(1, 40))
    # a shape is replayed from its second sighting on: one that never comes back is not captured
    assert pg.shape_of([StepEntry(a, toks, [38]), StepEntry(b, toks[:3], [2])]) is None
    assert pg.shape_of([StepEntry(a, toks, [38]), StepEntry(b, toks[:3], [2])]) == (64, 2, 1)
    assert pg.shape_of([StepEntry(a, toks, list(range(39)))]) is None          # every position wanted: by hand
    assert pg.shape_of([StepEntry(a, [1], [0]), StepEntry(b, [2], [0])]) is None   # one token each: a decode step
    assert pg.shape_of([StepEntry(a, [1] * 1025, [0])]) is None                # too long
    # errors are the step function's, and leave everything as it was
    with pytest.raises(ValueError, match="vocabulary"):
        llm.step([StepEntry(a, [1, 2, 10 ** 6], [2])])
    with pytest.raises(ValueError, match="not held"):
        llm.step([StepEntry(77, [1, 2, 3], [2])])
    assert llm.engine.length(a) == 0 and pg.replays == 0
    out = llm.step([StepEntry(a, toks, [38]), StepEntry(b, toks[:3], [2])])
    assert out.shape == (2, TINY["A"]["vocab_size"]) and pg.replays == 1 and llm.engine.length(a) == 39
