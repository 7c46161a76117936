"""Generation through the Python entry point, the command line and trace replay, against the plain oracle."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, assert_close, load_plain, make_model_dir, plain_logits, rand_tokens
from plain import llama_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in "AB":
        for dtype in ("float32", "bfloat16"):
            out[name, dtype] = make_model_dir(str(tmp_path_factory.mktemp(f"g{name}{dtype}")), TINY[name],
                                              seed=10 + ord(name), dtype=dtype)
    return out


def _check_greedy(cfg, w, prompt, tokens, dtype):
    seq = list(prompt)
    for tok in tokens:
        ref = plain_logits(cfg, w, seq)[-1]
        slack = TOL[dtype] * float(np.max(np.abs(ref)))
        assert ref[tok] >= ref.max() - 2 * slack, (prompt, tokens, tok, int(ref.argmax()))
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_batch_of_unequal_prompts(folders, dtype):
    """Three sequences, prompts 5/9/12, 8 greedy tokens each, through Stratum.generate."""
    from stratum_b200 import Stratum
    path = folders["A", dtype]
    cfg, w = load_plain(path)
    rng = np.random.default_rng(0)
    prompts = [rand_tokens(rng, n, cfg["vocab_size"]) for n in (5, 9, 12)]
    llm = Stratum(path, dtype=dtype, max_tokens=512)
    res = llm.generate(prompts, max_new_tokens=8, stop_ids=())
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 8 and r.finish_reason == "length"
        _check_greedy(cfg, w, p, r.tokens, dtype)
        if dtype == "float32":
            assert r.tokens == P.greedy_generate(cfg, w, p, 8)
    # alone or together, and in batches one after another: the same tokens
    alone = [llm.generate([p], max_new_tokens=8, stop_ids=())[0].tokens for p in prompts]
    serial = llm.generate(prompts, max_new_tokens=8, stop_ids=(), max_batch=2)
    if dtype == "float32":
        assert alone == [r.tokens for r in res] == [r.tokens for r in serial]
    llm.engine.cache.check()
    assert llm.engine.cache.tokens_held() == 0


def test_stop_token_ends_one_sequence_early(folders):
    from stratum_b200 import Stratum
    path = folders["A", "float32"]
    cfg, w = load_plain(path)
    prompts = [[3, 1, 4, 1, 5], [9, 2, 6]]
    full = [P.greedy_generate(cfg, w, p, 10) for p in prompts]
    stop = full[0][3]
    expect = [P.greedy_generate(cfg, w, p, 10, stop_ids=[stop]) for p in prompts]
    llm = Stratum(path, dtype="float32", max_tokens=512)
    res = llm.generate(prompts, max_new_tokens=10, stop_ids=[stop])
    assert [r.tokens for r in res] == expect
    assert res[0].finish_reason == "stop" and res[0].tokens[-1] == stop
    assert llm.engine.cache.tokens_held() == 0


def test_temperature_sampling_matches_plain_draws(folders):
    """Two sequences, prompts 1/17, 6 tokens at temperature 0.8 with a fixed seed (float32)."""
    from stratum_b200 import SamplingParams, Stratum
    path = folders["B", "float32"]
    cfg, w = load_plain(path)
    rng = np.random.default_rng(5)
    prompts = [rand_tokens(rng, n, cfg["vocab_size"]) for n in (1, 17)]
    params = SamplingParams(temperature=0.8, seed=1234)
    llm = Stratum(path, dtype="float32", max_tokens=512)
    res = llm.generate(prompts, max_new_tokens=6, stop_ids=(), sampling=params)
    again = llm.generate(prompts, max_new_tokens=6, stop_ids=(), sampling=params)
    assert [r.tokens for r in res] == [r.tokens for r in again]            # same seed, same tokens
    # a request keeps its draws when its batch changes, as long as it keeps its stream
    alone = llm.generate([prompts[1]], max_new_tokens=6, stop_ids=(), sampling=params, stream_ids=[1])[0]
    assert alone.tokens == res[1].tokens
    swapped = llm.generate(prompts[::-1], max_new_tokens=6, stop_ids=(), sampling=params, stream_ids=[1, 0])
    assert [r.tokens for r in swapped] == [res[1].tokens, res[0].tokens]
    for i, (p, r) in enumerate(zip(prompts, res)):
        stream = P.Pcg32(1234, i)
        seq = list(p)
        for tok in r.tokens:
            ids, probs = P.filtered_distribution(plain_logits(cfg, w, seq)[-1], 0.8, 0, 1.0)
            u = stream.uniform()
            cum = np.cumsum(probs)
            # the picked id's stretch of the cumulative distribution holds u, up to float32 noise
            below = cum[tok - 1] if tok > 0 else 0.0
            assert below - 4e-6 <= u < cum[tok] + 4e-6, (i, seq, tok, P.sample_inverse_cdf(ids, probs, u))
            seq.append(tok)


def test_command_line_prints_the_reference_lines(folders):
    path = folders["A", "float32"]
    cfg, w = load_plain(path)
    prompt = [1, 2, 3, 4, 5, 6, 7, 8]
    expect = P.greedy_generate(cfg, w, prompt, 5)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "stratum"), path, "4", *map(str, prompt), "--fp32",
                        "--timing"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == [str(t) for t in expect]
    assert f"after prefill, stratum_argmax = {expect[0]}" in r.stderr
    for g in range(4):
        assert f"step {g:2d}  in={expect[g]}  stratum_argmax={expect[g + 1]}  logit=" in r.stderr
    assert "[timing] prefill 8 tok" in r.stderr
    # --profile: the same tokens launch by launch, and device time per kind of kernel
    r = subprocess.run([sys.executable, os.path.join(ROOT, "stratum"), path, "4", *map(str, prompt), "--fp32",
                        "--profile"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == [str(t) for t in expect]
    prof = r.stderr[r.stderr.index("[profile]"):]
    for name in ("linear_simple", "attention_simple", "rmsnorm", "rope_store", "embed_gather", "argmax"):
        assert f"    {name} " in prof and " calls (" in prof, prof
    # errors: id outside the vocabulary, prompt beyond capacity; nonzero exit, as the reference
    r = subprocess.run([sys.executable, os.path.join(ROOT, "stratum"), path, "2", "999"], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode != 0 and "outside the vocabulary" in r.stderr
    r = subprocess.run([sys.executable, os.path.join(ROOT, "stratum"), path, "40", "1", "2", "--max-kv", "32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "exceeds KV capacity" in r.stderr


def test_command_line_batch_file(folders, tmp_path):
    """--batch-file: one prompt per line, run as one batch of unequal lengths; every request's ids on its own line."""
    path = folders["A", "float32"]
    cfg, w = load_plain(path)
    prompts = [[1, 2, 3], [9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 11], [42]]
    bf = tmp_path / "prompts.txt"
    bf.write_text("\n".join(" ".join(map(str, q)) for q in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "stratum"), path, "3", "--fp32", "--batch-file", str(bf)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [ln.split() for ln in r.stdout.strip().splitlines()]
    assert lines == [[str(t) for t in P.greedy_generate(cfg, w, q, 4)] for q in prompts]
    assert "request 1: prompt 11 tok, 4 generated, ended by length" in r.stderr


def _run_trace(model, dtype, out, max_tokens, steps):
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype,
                          "--out", out, "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE,
                         stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {s['step']}"
    p.stdin.close()
    assert p.wait(timeout=600) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(folders, dtype, tmp_path):
    path = folders["B", dtype]
    cfg, w = load_plain(path)
    rng = np.random.default_rng(8)
    V = cfg["vocab_size"]
    a, b, c = (rand_tokens(rng, n, V) for n in (70, 9, 33))
    ra, rb, rc = (plain_logits(cfg, w, t) for t in (a, b, c))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]},
                                     {"id": "b", "tokens": b[:5], "want": []}], "end": []}]
    for i in range(10):
        ents = [{"id": "a", "tokens": [a[60 + i]], "want": [0]}]
        end = ["a"] if i == 9 else []
        if i < 4:
            ents.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
            if i == 3:
                end.append("b")
        steps.append({"step": 1 + i, "entries": ents, "end": end})
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": c, "want": list(range(33))}], "end": ["c"]})
    out = str(tmp_path / "out")
    _run_trace(path, dtype, out, 64 * 3, steps)       # a: 2 pages, b: 1 page; c reuses what they gave back
    read = lambda n: np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V)   # noqa: E731
    assert_close(read(0), ra[[0, 59]], dtype, "trace step 0")
    for i in range(10):
        got = read(1 + i)
        assert_close(got[0], ra[60 + i], dtype, f"trace a {i}")
        if i < 4:
            assert_close(got[1], rb[5 + i], dtype, f"trace b {i}")
        else:
            assert got.shape[0] == 1
    assert_close(read(11), rc, dtype, "trace c")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_launch_by_launch(folders, dtype):
    """Decode steps as replayed CUDA graphs (padded rows, bucketed page tables) give what eager steps give."""
    from stratum_b200 import SamplingParams, Stratum
    path = folders["B", dtype]
    cfg, w = load_plain(path)
    rng = np.random.default_rng(21)
    prompts = [rand_tokens(rng, n, cfg["vocab_size"]) for n in (3, 60, 17, 9, 64, 2, 30, 5, 11, 70)]
    budgets = [70, 9, 30, 12, 5, 66, 8, 20, 3, 15]          # sequences leave at different times; pages are crossed
    eager = Stratum(path, dtype=dtype, max_tokens=4096, use_graphs=False)
    graphed = Stratum(path, dtype=dtype, max_tokens=4096, use_graphs=True)
    for params in (SamplingParams(), SamplingParams(temperature=0.9, top_k=20, seed=5)):
        a = eager.generate(prompts, max_new_tokens=budgets, stop_ids=(), sampling=params)
        b = graphed.generate(prompts, max_new_tokens=budgets, stop_ids=(), sampling=params)
        assert [r.tokens for r in a] == [r.tokens for r in b]
    assert graphed.graphs.captures >= 3
    _check_greedy(cfg, w, prompts[1], eager.generate([prompts[1]], 9, stop_ids=())[0].tokens, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_after_slots_change_pages(folders, dtype):
    """A captured graph is used again by a batch with the same slots, rows, width and sampling mode whose
    sequences hold other pages: the page tables must be written again, not remembered.  The first call's middle
    request ends first, so slots 0 and 2 stay live with pages 0 and 2; in the second call the same live slots
    own pages 0 and 3."""
    from stratum_b200 import Stratum
    path = folders["A", dtype]
    cfg, w = load_plain(path)
    rng = np.random.default_rng(4)
    V = cfg["vocab_size"]
    eager = Stratum(path, dtype=dtype, max_tokens=1024, use_graphs=False)
    graphed = Stratum(path, dtype=dtype, max_tokens=1024, use_graphs=True)
    for lens in ((10, 10, 10), (10, 70, 10), (3, 64, 9), (10, 10, 10)):
        prompts = [rand_tokens(rng, n, V) for n in lens]
        budgets = [12, 2, 12]
        a = eager.generate(prompts, max_new_tokens=budgets, stop_ids=())
        b = graphed.generate(prompts, max_new_tokens=budgets, stop_ids=())
        assert [r.tokens for r in a] == [r.tokens for r in b], lens
        for p, r in zip(prompts, b):
            _check_greedy(cfg, w, p, r.tokens, dtype)
    # the same few graphs served all four calls (bfloat16: a graph is captured again after the split-key
    # attention's scratch has grown, because it recorded the old buffer's address)
    assert graphed.graphs.captures <= (3 if dtype == "float32" else 6)
    graphed.engine.cache.check()


def test_a_given_up_wait_is_an_error_and_changes_nothing(folders):
    """The status word of the kernels' bounded waits is read on the product path.  No wait is made to run out
    on the device: the word is written from the host before a step, as a kernel that gave up would have."""
    from stratum_b200 import StepEntry, Stratum, kernels
    from stratum_b200.kernels import KernelError
    path = folders["A", "bfloat16"]
    llm = Stratum(path, dtype="bfloat16", max_tokens=512)
    slot = llm.acquire()
    llm.step([StepEntry(slot, [1, 2, 3], [2])])
    ids, _ = llm.decode_step([slot], [4])                      # captures the graph; the word is clean
    assert llm.engine.length(slot) == 4
    for run in (lambda: llm.decode_step([slot], [5]),                       # a replayed graph
                lambda: llm.step([StepEntry(slot, [5], [0])]),               # launch by launch
                lambda: llm.generate([[7, 8, 9]], max_new_tokens=3, stop_ids=())):
        kernels.status_word().fill_(103)
        with pytest.raises(KernelError, match="wait ran out"):
            run()
        assert llm.engine.length(slot) == 4                   # nothing advanced
        assert int(kernels.status_word().item()) == 0         # cleared for the next run
    llm.engine.cache.check()
    ids2, _ = llm.decode_step([slot], [5])                     # and the engine still works
    assert llm.engine.length(slot) == 5
    llm.release(slot)
    assert llm.engine.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_one_step_ahead_gives_the_same_tokens(folders, dtype):
    """Decode steps launched before the host has read the step before (ids fed back on the device) against the
    same steps read one by one: greedy with a stop id that ends requests at different steps, and sampling, in
    batches that follow one another so that slots given back late (after their ride along) are used again."""
    from stratum_b200 import SamplingParams, Stratum
    path = folders["B", dtype]
    cfg, w = load_plain(path)
    rng = np.random.default_rng(31)
    V = cfg["vocab_size"]
    prompts = [rand_tokens(rng, n, V) for n in (3, 60, 17, 9, 64, 2, 30)]
    budgets = [70, 9, 30, 12, 5, 66, 8]
    llm = Stratum(path, dtype=dtype, max_tokens=64 * 6, max_seqs=3)      # three requests at a time: three batches
    base = llm.generate(prompts, max_new_tokens=budgets, stop_ids=(), run_ahead=False)
    # a stop id that some requests meet early, others never
    counts = {}
    for r in base:
        for t in r.tokens[2:20]:
            counts[t] = counts.get(t, 0) + 1
    stop = max(counts, key=counts.get)
    for params in (SamplingParams(), SamplingParams(temperature=0.9, top_k=20, seed=5)):
        a = llm.generate(prompts, max_new_tokens=budgets, stop_ids=[stop], sampling=params, run_ahead=False)
        b = llm.generate(prompts, max_new_tokens=budgets, stop_ids=[stop], sampling=params, run_ahead=True)
        assert [(r.tokens, r.finish_reason) for r in a] == [(r.tokens, r.finish_reason) for r in b]
        assert any(r.finish_reason == "stop" for r in a) and any(r.finish_reason == "length" for r in a)
    _check_greedy(cfg, w, prompts[1], llm.generate([prompts[1]], 9, stop_ids=())[0].tokens, dtype)
    llm.engine.cache.check()
    assert llm.engine.cache.tokens_held() == 0
