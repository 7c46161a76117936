"""Decode steps as replayed CUDA graphs at the layer sizes of Llama-3.1-8B, Llama-3.2-1B and Llama-2-7B.

This is the schedule that generation uses by default and that the benchmark times: the stream-K and
cluster forms of the matrix product with their second pass, the TMA-fed decode attention with its late
launch trigger, padded rows and page tables of a bucketed width, all overlapping through programmatic
dependent launch.  Every replayed step's logits are compared with the launch-by-launch engine's (the same
bits in float32) and, for some requests of every batch, with the float64 oracle; the picked ids with the
logits they were picked from.  Batches of 1 to 64 requests of unequal lengths run one after another on the
same cache, long requests cross pages so that the width bucket doubles twice, short ones leave early and
their slots and pages are taken again.
"""
import numpy as np
import pytest
import torch

from helpers import TOL, assert_close, load_plain, make_model_dir, plain_logits, rand_tokens
from plain import llama_plain as P
from test_real_layer_sizes_gpu import SHAPES

pytestmark = pytest.mark.gpu

BATCHES = (1, 2, 3, 8, 9, 40, 64)
LONG_STEPS = 72                      # a prompt of 60 tokens then holds 132: pages 1 -> 2 -> 3, widths 1 -> 2 -> 4


def _workload(rng, V):
    """Per batch: prompts, forced continuations (unequal), and which requests the oracle checks."""
    work = []
    for count in BATCHES:
        lens = [int(x) for x in rng.integers(1, 40, size=count)]
        steps = [int(x) for x in rng.integers(1, 24, size=count)]
        lens[0], steps[0] = 60, LONG_STEPS
        if count <= 3:
            steps = [LONG_STEPS] * count                     # every sequence crosses a page
            lens = [60 - 7 * i for i in range(count)]
        else:
            lens[-1], steps[-1] = 5, LONG_STEPS - 8           # a second long one, at the batch's far end
        seqs = [rand_tokens(rng, n + k, V) for n, k in zip(lens, steps)]
        checked = sorted({0, count - 1, count // 2})
        work.append((lens, steps, seqs, checked))
    return work


@pytest.fixture(scope="module", params=sorted(SHAPES))
def setup(request, tmp_path_factory):
    raw = {k: v for k, v in SHAPES[request.param].items() if v is not None}
    path = make_model_dir(str(tmp_path_factory.mktemp("graph_layers")), raw, seed=33, dtype="bfloat16")
    cfg, w = load_plain(path)
    work = _workload(np.random.default_rng(17), cfg["vocab_size"])
    refs = {}                         # (batch, request) -> oracle logits of the whole sequence; shared by both dtypes
    for b, (lens, steps, seqs, checked) in enumerate(work):
        for i in checked:
            refs[b, i] = plain_logits(cfg, w, seqs[i])
    return path, cfg, w, work, refs


def _check_picks(logits, picked, sampling, uniforms):
    for row, tok in enumerate(picked):
        lg = logits[row]
        if sampling.greedy:
            assert tok == int(np.argmax(lg)), (row, tok, int(np.argmax(lg)))     # numpy: the lowest index among equals
        else:
            ids, probs = P.filtered_distribution(lg, sampling.temperature, sampling.top_k, sampling.top_p)
            at = list(ids).index(tok)                                            # must be a candidate at all
            cum = np.cumsum(probs)
            below = cum[at - 1] if at > 0 else 0.0
            assert below - 4e-6 <= uniforms[row] < cum[at] + 4e-6, (row, tok, uniforms[row])


@pytest.mark.parametrize("mode", ["greedy", "sampling"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_at_real_layer_sizes(setup, dtype, mode):
    from stratum_b200 import SamplingParams, StepEntry, Stratum
    from stratum_b200.engine import Engine
    from stratum_b200.sampling import Pcg32
    path, cfg, w, work, refs = setup
    sampling = SamplingParams() if mode == "greedy" else SamplingParams(temperature=0.9, top_k=20, seed=5)
    llm = Stratum(path, dtype=dtype, max_tokens=64 * 256, max_seqs=64, use_graphs=True)
    eager = Engine(llm.model, max_tokens=64 * 256, max_seqs=64)      # the same weights, a cache of its own
    for b, (lens, steps, seqs, checked) in enumerate(work):
        count = len(lens)
        slots = [llm.acquire() for _ in range(count)]
        eslots = [eager.acquire() for _ in range(count)]
        llm.step([StepEntry(s, q[:n], []) for s, q, n in zip(slots, seqs, lens)])
        eager.step([StepEntry(s, q[:n], []) for s, q, n in zip(eslots, seqs, lens)])
        streams = [Pcg32(sampling.seed, i) for i in range(count)]
        mirror = [Pcg32(sampling.seed, i) for i in range(count)]
        live, k = list(range(count)), 0
        while live:
            toks = [seqs[i][lens[i] + k] for i in live]
            uniforms = None if sampling.greedy else [mirror[i].uniform() for i in live]
            ids, vals, logits = llm.decode_step([slots[i] for i in live], toks, sampling,
                                                [streams[i] for i in live], with_logits=True)
            got = logits.cpu().numpy()
            want = eager.step([StepEntry(eslots[i], [t], [0]) for i, t in zip(live, toks)]).cpu().numpy()
            if dtype == "float32":
                assert np.array_equal(got, want), f"batch {count} step {k}: replayed and launched logits differ"
            else:
                assert np.max(np.abs(got - want)) <= 1e-2 * np.max(np.abs(want)), f"batch {count} step {k}"
            for row, i in enumerate(live):
                if (b, i) in refs:
                    assert_close(got[row], refs[b, i][lens[i] + k], dtype, f"batch {count} request {i} step {k}")
                assert abs(vals[row] - got[row][ids[row]]) <= 1e-6 * max(1.0, abs(vals[row]))
            _check_picks(got, ids, sampling, uniforms)
            k += 1
            for i in list(live):
                if k >= steps[i]:                              # shorter requests end earlier; their slots go back
                    llm.release(slots[i]); eager.release(eslots[i]); live.remove(i)
        llm.engine.cache.check()
    assert llm.engine.cache.tokens_held() == 0
    assert llm.graphs.captures >= 8                             # rows 1, 2, 3, 8, 16, 40, 64 and three widths


def test_generate_with_graphs_at_real_layer_sizes(setup):
    """The same through Stratum.generate (bfloat16): two calls, the second taking the slots the first gave
    back; the logits of every step, by the hook, against the oracle; the tokens against launch-by-launch."""
    from stratum_b200 import Stratum
    path, cfg, w, work, _ = setup
    rng = np.random.default_rng(3)
    V = cfg["vocab_size"]
    graphed = Stratum(path, dtype="bfloat16", max_tokens=64 * 64, use_graphs=True)
    eager = Stratum(path, dtype="bfloat16", max_tokens=64 * 64, use_graphs=False)
    for lens, budgets in (((10, 10, 10), (20, 3, 20)), ((10, 70, 10, 3), (12, 9, 12, 30))):
        prompts = [rand_tokens(rng, n, V) for n in lens]
        seen = []
        out = graphed.generate(prompts, max_new_tokens=list(budgets), stop_ids=(),
                               on_logits=lambda lg, ids: seen.append((lg.cpu().numpy().copy(), list(ids))))
        ref_out = eager.generate(prompts, max_new_tokens=list(budgets), stop_ids=())
        oracle = [plain_logits(cfg, w, p + r.tokens) for p, r in zip(prompts, out)]
        live = list(range(len(prompts)))
        for step, (lg, ids) in enumerate(seen):
            assert len(ids) == len(live)
            for row, i in enumerate(live):
                assert_close(lg[row], oracle[i][len(prompts[i]) - 1 + step], "bfloat16", f"request {i} step {step}")
                assert ids[row] == out[i].tokens[step]
            live = [i for i in live if step + 1 < budgets[i]]
        for i, (a, e) in enumerate(zip(out, ref_out)):
            if a.tokens != e.tokens:                           # only where the oracle itself sees a near tie
                j = next(j for j, (x, y) in enumerate(zip(a.tokens, e.tokens)) if x != y)
                row = oracle[i][len(prompts[i]) - 1 + j]
                assert abs(row[a.tokens[j]] - row[e.tokens[j]]) <= 2 * TOL["bfloat16"] * np.max(np.abs(row))
        graphed.engine.cache.check()
        assert graphed.engine.cache.tokens_held() == 0
