"""The C interface on the GPU: a program written in C (tests/capi_client.c) steps prompts of unequal lengths and
single tokens, generates, and makes calls that must fail; what it wrote is compared with the plain oracle."""
import os
import subprocess

import numpy as np
import pytest

from capi_helpers import build_client, clean_env
from helpers import TINY, assert_close, load_plain, make_model_dir, plain_logits, rand_tokens
from plain import llama_plain as P

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_c_program_steps_and_generates(tmp_path, name, dtype):
    path = make_model_dir(str(tmp_path / "model"), TINY[name], seed=31, dtype=dtype)
    cfg, w = load_plain(path)
    V = cfg["vocab_size"]
    rng = np.random.default_rng(4)
    lens = [7, 70, 3, 19]                                        # one prompt longer than a page
    prompts = [rand_tokens(rng, n, V) for n in lens]
    n = len(lens)
    np.asarray([n] + lens + [t for p in prompts for t in p], dtype="<i4").tofile(str(tmp_path / "in.i32"))
    out = tmp_path / "out"
    out.mkdir()
    exe, _ = build_client(str(tmp_path))
    done = subprocess.run([exe, "run", path, dtype, str(tmp_path / "in.i32"), str(out)], capture_output=True,
                          text=True, env=clean_env(), cwd=str(tmp_path), timeout=900)
    assert done.returncode == 0 and done.stdout.strip().endswith("ok"), done.stdout + done.stderr

    picked = np.fromfile(str(out / "picked.i32"), dtype="<i4").reshape(4, 64)[:, :n]
    prompt_logits = np.fromfile(str(out / "prompt_logits.f32"), dtype="<f4").reshape(n, V)
    decode_logits = np.fromfile(str(out / "decode_logits.f32"), dtype="<f4").reshape(3, n, V)
    for i, p in enumerate(prompts):
        ref = plain_logits(cfg, w, p + picked[:3, i].tolist())
        assert_close(prompt_logits[i], ref[len(p) - 1], dtype, f"prompt {i}")
        for k in range(3):
            assert_close(decode_logits[k, i], ref[len(p) + k], dtype, f"seq {i} decode {k}")
    gen = np.fromfile(str(out / "generated.i32"), dtype="<i4")
    counts, ids = gen[:n], gen[n:].reshape(n, 4)
    assert counts.tolist() == [4] * n
    if dtype == "float32":
        assert ids.tolist() == picked.T.tolist()                 # generation and stepping by hand agree
        assert ids.tolist() == [P.greedy_generate(cfg, w, p, 4) for p in prompts]
    sampled = np.fromfile(str(out / "sampled.i32"), dtype="<i4")
    assert sampled[:n].tolist() == [4] * n and np.all((sampled[n:] >= 0) & (sampled[n:] < V))
    from stratum_b200 import SamplingParams, Stratum             # the Python entry point draws the same tokens
    llm = Stratum(path, dtype=dtype, max_tokens=2048)
    same = llm.generate(prompts, max_new_tokens=4, stop_ids=(), sampling=SamplingParams(0.8, 5, 1.0, 7))
    assert [r.tokens for r in same] == sampled[n:].reshape(n, 4).tolist()

    notes = (out / "notes.txt").read_text().splitlines()
    slots = [int(x.split()[1]) for x in notes if x.startswith("slot ") and "again" not in x]
    assert len(set(slots)) == n
    assert [int(x.split()[1]) for x in notes if x.startswith("length ") and "after" not in x] == [k + 3 for k in lens]
    by = {x.split(" -> ")[0]: x.split(" -> ")[1] for x in notes if " -> " in x}
    assert by["bad token"].startswith("-2: ") and "vocabulary" in by["bad token"]
    assert by["bad slot"].startswith("-2: ") and by["released twice"].startswith("-2: ")
    assert by["null tokens"].startswith("-1: ")
    assert f"length after {lens[0] + 3}" in notes                # the refused step changed nothing
    assert int([x for x in notes if x.startswith("slot again")][0].split()[2]) in slots    # a slot is used again
    stop, row = int(picked[1, 0]), ids[0].tolist()               # the second id found by hand was the stop id
    assert f"stopped after {row.index(stop) + 1 if stop in row else 4}" in notes
