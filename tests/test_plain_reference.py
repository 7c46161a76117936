"""The plain oracle against the reference's own tools (outputs committed under tests/golden)."""
import json
import os

import numpy as np

from plain import llama_plain as P

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_llama_reference.npz")


def _load():
    z = np.load(GOLD)
    cfg = json.loads(bytes(z["config_json"]).decode())
    w = {k[2:]: z[k].astype(np.float32) for k in z.files if k.startswith("w:")}
    return z, cfg, w


def test_hidden_states_match_reference_oracle():
    z, cfg, w = _load()
    for ri in range(2):
        prompt = z[f"run{ri}:prompt"].tolist()
        greedy = z[f"run{ri}:greedy"].tolist()
        seq = prompt + greedy
        ref_hidden = z[f"run{ri}:hidden_last"]          # one row per processed token
        last = cfg["num_hidden_layers"] - 1
        _, caps = P.forward_hidden(cfg, w, seq, capture_layers=[last])
        assert ref_hidden.shape == caps[last].shape
        # the reference's tolerance between its engine and its oracle is 5e-3
        # (stratum/tools/hidden_oracle.py:272); float32-vs-float64 noise is far below it.
        assert np.max(np.abs(caps[last] - ref_hidden)) < 2e-4


def test_greedy_ids_match_reference_pins():
    """prompt 1..8 -> 70 118 22 60 (.github/workflows/ci.yml:141); prompt 1 2 3 4 ->
    22 then 142 22 185 32 22 22 22 (stratum/tools/campaign_tiny_test.py:33)."""
    z, cfg, w = _load()
    assert z["run0:greedy"].tolist() == [70, 118, 22, 60]
    assert z["run1:greedy"].tolist() == [22, 142, 22, 185, 32, 22, 22, 22]
    for ri in range(2):
        prompt = z[f"run{ri}:prompt"].tolist()
        greedy = z[f"run{ri}:greedy"].tolist()
        assert P.greedy_generate(cfg, w, prompt, len(greedy)) == greedy


def test_rotation_frequencies_match_the_reference_header():
    """no scaling, linear and YaRN (ramp, clamps, derived and explicit magnitude) against what the reference's
    stratum/native/stratum_rope.h computes (tests/golden/make_rope_golden.py compiled and ran it)."""
    with open(os.path.join(os.path.dirname(GOLD), "rope_reference.json")) as f:
        cases = json.load(f)
    assert len(cases) == 5
    for name, c in cases.items():
        scaling = None
        if c["type"] != "none":
            scaling = {"rope_type": c["type"], "factor": c["factor"],
                       "original_max_position_embeddings": c["original_max_position"],
                       "beta_fast": c["beta_fast"], "beta_slow": c["beta_slow"]}
            if c["attention_factor"] > 0:
                scaling["attention_factor"] = c["attention_factor"]
        inv = P.rope_inv_freq(2 * c["pairs"], c["theta"], scaling)
        ref = np.asarray(c["inv_freq"])
        assert inv.shape == ref.shape
        assert np.max(np.abs(inv - ref) / ref) < 2e-6, name          # float32 powf/logf against float64
        assert abs(P.rope_magnitude(scaling) - c["mscale"]) < 1e-6, name
    yarn = np.asarray(cases["yarn_f4_orig32_80"]["inv_freq"])
    plain = P.rope_inv_freq(80, 50000.0)
    ratio = plain / yarn
    assert np.isclose(ratio[0], 1.0) and np.isclose(ratio[-1], 4.0) and np.any((ratio > 1.05) & (ratio < 3.9))
