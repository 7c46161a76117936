"""The same requests cut into steps in three ways (whole; last 32 tokens one by one; unequal batches one after
another in a cache so small that slots and pages are reused) give the same logits at every position: the same
bits on the float32 path, whose every reduction has one order whatever the step holds; within the stated bound
on the bfloat16 path, where prompts and single tokens run through different kernels.  Tiny A, tiny B and the
layer sizes of Llama-3.1-8B; and once through the programs, bin/trace_run and bin/logit_compare."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, assert_close, load_plain, make_model_dir, plain_logits, rand_tokens
from test_real_layer_sizes_gpu import REAL_LAYERS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENS = (150, 70, 33, 9, 100, 1, 64, 65, 20)
MAX_TOKENS = 6 * 64                   # mode 3 needs three batches; the second and third take what the first gave back


@pytest.fixture(scope="module", params=["A", "B", "llama3.1-8b-layers"])
def model(request, tmp_path_factory):
    raw = TINY[request.param] if request.param in TINY else REAL_LAYERS
    path = make_model_dir(str(tmp_path_factory.mktemp("modes")), raw, seed=5, dtype="bfloat16")
    cfg, w = load_plain(path)
    rng = np.random.default_rng(9)
    requests = [(f"r{i}", rand_tokens(rng, n, cfg["vocab_size"])) for i, n in enumerate(LENS)]
    return request.param, path, cfg, w, requests


def _records(path, dtype, requests, mode):
    from stratum_b200 import replay
    from stratum_b200.engine import Engine, load_model
    m, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    engine = Engine(m, max_tokens=MAX_TOKENS)
    index = {rid: i for i, (rid, _) in enumerate(requests)}
    out = {}
    player = replay.Player(engine, lambda rid, pos, row: out.__setitem__((index[rid], pos), row.copy()))
    steps = replay.plan_steps(requests, mode, MAX_TOKENS)
    for rec in steps:
        player.play_step(rec)
    engine.cache.check()
    assert engine.cache.tokens_held() == 0
    return out, steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_three_cuts_give_the_same_logits(model, dtype):
    from stratum_b200 import replay
    name, path, cfg, w, requests = model
    runs = {mode: _records(path, dtype, requests, mode) for mode in (1, 2, 3)}
    whole = runs[1][0]
    assert len(whole) == sum(LENS)
    # mode 3 really batches and really reuses: more than one batch, requests ending at different steps
    steps3 = runs[3][1]
    assert sum(1 for s in steps3 if len(s["entries"]) > 1 and any(len(e["tokens"]) > 1 for e in s["entries"])) == 3
    assert len({len(s["entries"]) for s in steps3}) >= 4           # batches shrink as their requests end
    # the whole cut against the oracle, for two requests (the others are tied to it by the comparison below)
    for i in (0, 3):
        ref = plain_logits(cfg, w, requests[i][1])
        got = np.stack([whole[i, p] for p in range(LENS[i])])
        assert_close(got, ref, dtype, f"{name} request {i} whole")
    for mode in (2, 3):
        rows, s = replay.compare_records(whole, runs[mode][0])
        assert s["records"] == sum(LENS) and s["only_in_base"] == 0 and s["only_in_other"] == 0
        if dtype == "float32":
            differ = [r[0] for r in rows if not r[4]]
            assert not differ, f"{name} mode {mode}: {len(differ)} rows differ in some bit, first {differ[:3]}"
        else:
            bound = TOL["bfloat16"] * s["max_abs_logit"]
            assert s["max_abs_diff"] <= bound, (name, mode, s)
            assert s["max_kl"] <= bound * bound, (name, mode, s)
            for key, kl, maxd, agree, same in rows:
                if not agree:                               # the best ids may differ only where the base has a near tie
                    b = whole[key]
                    assert b.max() - b[int(np.argmax(runs[mode][0][key]))] <= 2 * bound, (name, mode, key)
            print(f"{name} mode {mode} vs whole (bfloat16): max|dl|={s['max_abs_diff']:.4g} of "
                  f"{s['max_abs_logit']:.4g}, max KL={s['max_kl']:.3g}, top-1 {s['top1_agree']}/{s['records']}, "
                  f"identical {s['identical']}")


def test_replay_programs_modes_and_compare(tmp_path):
    """bin/trace_run --requests/--mode/--records and bin/logit_compare --require-identical, float32."""
    path = make_model_dir(str(tmp_path / "m"), TINY["A"], seed=2, dtype="float32")
    rng = np.random.default_rng(1)
    reqs = tmp_path / "requests.jsonl"
    reqs.write_text("".join(json.dumps({"id": f"q{i}", "tokens": rand_tokens(rng, n, 256)}) + "\n"
                            for i, n in enumerate((40, 70, 5, 66))))
    files = []
    for mode in (1, 2, 3):
        out = str(tmp_path / f"mode{mode}.slog")
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype",
                            "float32", "--max-tokens", "192", "--requests", str(reqs), "--mode", str(mode),
                            "--records", out], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        assert r.stdout.splitlines()[0] == "done 0"
        files.append(out)
    for other in files[1:]:
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "logit_compare"), files[0], other,
                            "--require-identical", "--quiet"], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "records=181" in r.stdout and "identical=181/181" in r.stdout
