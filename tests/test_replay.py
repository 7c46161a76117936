"""Replay planning, record files and the comparison (no GPU): every position is wanted exactly once in each
mode, capacity is respected, mode 3 lets requests end at different steps and reuses what they gave back."""
import os
import subprocess
import sys

import numpy as np
import pytest

from stratum_b200 import replay
from stratum_b200.cache.pages import PAGE_TOKENS, pages_for

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _requests(lens):
    rng = np.random.default_rng(0)
    return [(f"r{i}", rng.integers(0, 100, size=n).tolist()) for i, n in enumerate(lens)]


def _simulate(requests, steps, max_tokens):
    """Play the plan on paper: positions seen per request, pages held, joins and endings."""
    toks = dict(requests)
    held, seen, ended = {}, {rid: [] for rid in toks}, set()
    n_pages = pages_for(max_tokens)
    most_live = 0
    for s in steps:
        lens = [len(e["tokens"]) for e in s["entries"]]
        assert all(n == 1 for n in lens) or all(e["id"] not in held for e in s["entries"])   # start together or go on by one
        for e in s["entries"]:
            rid = e["id"]
            assert rid not in ended
            before = held.get(rid, 0)
            assert list(e["tokens"]) == toks[rid][before:before + len(e["tokens"])]
            for w in e["want"]:
                seen[rid].append(before + w)
            held[rid] = before + len(e["tokens"])
        assert sum(pages_for(n) for n in held.values()) <= n_pages
        most_live = max(most_live, len(held))
        for rid in s["end"]:
            assert held.pop(rid) == len(toks[rid])
            ended.add(rid)
    assert not held and ended == set(toks)
    for rid, t in toks.items():
        assert sorted(seen[rid]) == list(range(len(t))), rid
    return most_live


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_every_position_once_and_capacity_kept(mode):
    reqs = _requests([1, 2, 33, 64, 65, 100, 7, 130, 40, 3])
    steps = replay.plan_steps(reqs, mode, max_tokens=5 * PAGE_TOKENS, tail=32)
    assert [s["step"] for s in steps] == list(range(len(steps)))
    most = _simulate(reqs, steps, 5 * PAGE_TOKENS)
    if mode == 3:
        assert most >= 3                                   # real batches
        ends = [len(s["end"]) for s in steps if s["end"]]
        assert len(ends) > 4                               # requests of one batch end at different steps
        first_steps = [s for s in steps if any(len(e["tokens"]) > 1 for e in s["entries"]) or len(s["entries"]) > 1]
        assert len([s for s in steps if len(s["entries"]) > 1 and len(s["entries"][0]["tokens"]) >= 1]) > 0
        assert first_steps
    else:
        assert most == 1
    if mode == 2:
        singles = [s for s in steps if len(s["entries"][0]["tokens"]) == 1 and s["entries"][0]["id"] == "r5"]
        assert len(singles) == 32                          # the last 32 tokens go one by one


def test_plan_refuses_what_cannot_fit():
    with pytest.raises(ValueError, match="do not fit"):
        replay.plan_steps(_requests([200]), 1, max_tokens=128)
    with pytest.raises(ValueError, match="mode"):
        replay.plan_steps(_requests([5]), 4, max_tokens=128)


def test_record_files_and_comparison(tmp_path):
    rng = np.random.default_rng(1)
    V = 50
    rows = {(r, p): rng.standard_normal(V).astype(np.float32) for r in range(3) for p in range(4)}
    a, b = str(tmp_path / "a.slog"), str(tmp_path / "b.slog")
    for path, shift in ((a, 0.0), (b, 1e-3)):
        w = replay.RecordWriter(path, V)
        for (r, p), row in (rows.items() if shift == 0.0 else reversed(list(rows.items()))):
            noisy = row + (shift * rng.standard_normal(V)).astype(np.float32)
            w.write(r, p, noisy)
        w.close()
    va, ra = replay.read_records(a)
    assert va == V and set(ra) == set(rows) and all(np.array_equal(ra[k], rows[k]) for k in rows)
    _, rb = replay.read_records(b)
    per, s = replay.compare_records(ra, rb)                # pairs by (request, position), whatever the order
    assert s["records"] == 12 and s["identical"] == 0 and 0 < s["max_abs_diff"] < 1e-2 and 0 <= s["max_kl"] < 1e-4
    _, same = replay.compare_records(ra, ra)
    assert same["identical"] == 12 and same["max_kl"] == 0.0 and same["top1_agree"] == 12
    # KL against a hand computation on one row
    key = (1, 2)
    p = np.exp(ra[key].astype(np.float64)); p /= p.sum()
    q = np.exp(rb[key].astype(np.float64)); q /= q.sum()
    kl = float(np.sum(p * np.log(p / q)))
    got = [r for r in per if r[0] == key][0][1]
    assert abs(got - kl) < 1e-12
    # the tool, as a program
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "logit_compare"), a, b], capture_output=True,
                       text=True)
    assert r.returncode == 0 and "summary: records=12" in r.stdout and "identical=0/12" in r.stdout
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "logit_compare"), a, b, "--require-identical",
                        "--quiet"], capture_output=True, text=True)
    assert r.returncode == 1
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "logit_compare"), a, a, "--require-identical",
                        "--quiet"], capture_output=True, text=True)
    assert r.returncode == 0 and "identical=12/12" in r.stdout
    # malformed files are errors
    with open(a, "rb") as f:
        blob = f.read()
    bad = str(tmp_path / "bad.slog")
    with open(bad, "wb") as f:
        f.write(blob[:-5])
    with pytest.raises(ValueError, match="truncated"):
        replay.read_records(bad)
    with open(bad, "wb") as f:
        f.write(b"SLOG0001" + blob[8:])
    with pytest.raises(ValueError, match="magic"):
        replay.read_records(bad)
