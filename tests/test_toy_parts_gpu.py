"""Toy parts defined here, in the test, are registered, built and stepped without a change to the library's files:
a feed-forward that routes every token to one of several experts, a position encoding of another kind
(a learned vector per absolute position, added to the embedded tokens), and arrangements that own other
parts than the built-in one (one norm shared by a parallel mixer and feed-forward; a norm before and after
each part; a layer without a feed-forward).  They are no model of anyone's."""
import json
import os
from dataclasses import dataclass
from typing import Any, Dict

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _define_toy():
    from stratum_b200.config import Architecture, ModelConfig, register_architecture
    from stratum_b200.config.base import KeyReader
    from stratum_b200.parts import (FeedForward, LayerSpec, ModelSpec, PartSpec, PositionEncoding, ScheduleEntry,
                                    TensorSpec, register_part)

    @register_part("feed_forward", "toy_routed", replace=True)
    class Routed(FeedForward):
        """Router logits in float32; the token goes to its best expert (lowest index among equals) and the expert's
        output is weighted by the softmax weight of that expert: residual += p_e * W2_e relu(W1_e xn)."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.hidden, self.inner, self.experts = spec["hidden"], spec["inner"], spec["experts"]

        def tensors(self):
            p = self.prefix
            return {p + "router.weight": TensorSpec((self.experts, self.hidden), role="keep"),
                    p + "w1": TensorSpec((self.experts, self.inner, self.hidden)),
                    p + "w2": TensorSpec((self.experts, self.hidden, self.inner))}

        def bind(self, weights):
            p = self.prefix
            self.router = weights[p + "router.weight"].float()
            self.w1, self.w2 = weights[p + "w1"].float(), weights[p + "w2"].float()

        def forward(self, xn, residual, step):
            x = xn.float()
            logits = x @ self.router.T                                   # float32
            prob = torch.softmax(logits, dim=-1)
            best = torch.argmax(logits, dim=-1)                          # first maximum = lowest index
            for e in range(self.experts):
                rows = torch.nonzero(best == e).flatten()
                if rows.numel():
                    h = torch.relu(x[rows] @ self.w1[e].T)
                    residual[rows] += prob[rows, e:e + 1] * (h @ self.w2[e].T)

    @register_part("position", "toy_learned_absolute", replace=True)
    class LearnedAbsolute(PositionEncoding):
        """x[t] += table[position of t]; nothing rotates."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.max_positions, self.hidden = spec["max_positions"], spec["hidden"]

        def tensors(self):
            return {self.prefix + "table": TensorSpec((self.max_positions, self.hidden), role="keep")}

        def bind(self, weights):
            self.table = weights[self.prefix + "table"].float()

        def add_to_embedding(self, x, step):
            x += self.table[step.token_pos.long()]

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        n_layers: int
        hidden: int
        inner: int
        experts: int
        max_positions: int
        vocab: int
        eps: float
        torch_dtype: str = "float32"
        architecture = "ToyRoutedForCausalLM"

        @classmethod
        def from_dict(cls, raw: Dict[str, Any]):
            r = KeyReader(raw)
            out = cls(r.integer("layers"), r.integer("hidden"), r.integer("inner"), r.integer("experts"),
                      r.integer("max_positions"), r.integer("vocab"), r.number("eps", 1e-5))
            r.finish()
            return out

        def to_dict(self):
            return {"architectures": [self.architecture], "layers": self.n_layers, "hidden": self.hidden,
                    "inner": self.inner, "experts": self.experts, "max_positions": self.max_positions,
                    "vocab": self.vocab, "eps": self.eps}

    def describe(cfg):
        norm = lambda p: PartSpec("rmsnorm", {"size": cfg.hidden, "eps": cfg.eps, "prefix": p})   # noqa: E731
        layers = []
        for i in range(cfg.n_layers):
            # attention without any position part of its own: positions come from the learned table alone
            mixer = PartSpec("gqa_attention", {"hidden": cfg.hidden, "n_heads": 3, "n_kv_heads": 3, "head_dim": 16,
                                               "bias": False, "window": 0, "scale": None, "position": None,
                                               "prefix": "attn."})
            # even layers route, odd layers are dense: one model, two kinds of feed-forward
            ff = PartSpec("toy_routed", {"hidden": cfg.hidden, "inner": cfg.inner, "experts": cfg.experts,
                                         "prefix": "moe."}) if i % 2 == 0 else \
                PartSpec("swiglu", {"hidden": cfg.hidden, "intermediate": cfg.inner, "bias": False, "prefix": "ff."})
            layers.append(LayerSpec("prenorm_residual", {"mixer_norm": norm("n1."), "mixer": mixer,
                                                         "feed_forward_norm": norm("n2."), "feed_forward": ff},
                                    f"l.{i}."))
        return ModelSpec(cfg.hidden, cfg.vocab,
                         PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.hidden, "prefix": "emb."}),
                         tuple(layers), tuple(ScheduleEntry(i) for i in range(cfg.n_layers)), norm("nf."),
                         PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.hidden, "tied": False,
                                                  "prefix": "head."}),
                         position=PartSpec("toy_learned_absolute", {"max_positions": cfg.max_positions,
                                                                    "hidden": cfg.hidden, "prefix": "pos."}))

    register_architecture(Architecture(("ToyRoutedForCausalLM",), "test-only: routed experts, learned positions",
                                       ToyConfig, describe), replace=True)
    return ToyConfig


def _plain_toy(cfg, w, toks):
    """Whole sequence, float64, no cache."""
    from plain import llama_plain as P
    T = len(toks)
    x = P.embed(w["emb.weight"], toks) + w["pos.table"][:T]
    used = set()
    for i in range(cfg["layers"]):
        p = f"l.{i}."
        xn = P.rms_norm(x, w[p + "n1.weight"], cfg["eps"])
        q = P.linear(xn, w[p + "attn.q_proj.weight"]).reshape(T, 3, 16)
        k = P.linear(xn, w[p + "attn.k_proj.weight"]).reshape(T, 3, 16)
        v = P.linear(xn, w[p + "attn.v_proj.weight"]).reshape(T, 3, 16)
        x = x + P.linear(P.causal_gqa_attention(q, k, v).reshape(T, 48), w[p + "attn.o_proj.weight"])
        xn = P.rms_norm(x, w[p + "n2.weight"], cfg["eps"])
        if i % 2 == 0:
            logits = xn @ w[p + "moe.router.weight"].T
            prob = P.softmax(logits)
            for t in range(T):
                e = int(np.argmax(logits[t]))
                used.add(e)
                h = np.maximum(xn[t] @ w[p + "moe.w1"][e].T, 0.0)
                x[t] = x[t] + prob[t, e] * (h @ w[p + "moe.w2"][e].T)
        else:
            x = x + P.linear(P.silu(P.linear(xn, w[p + "ff.gate_proj.weight"])) *
                             P.linear(xn, w[p + "ff.up_proj.weight"]), w[p + "ff.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["nf.weight"], cfg["eps"]), w["head.weight"]), used


def test_routed_feed_forward_and_learned_positions_register_build_and_step(tmp_path):
    from helpers import load_plain
    from stratum_b200 import Stratum, StepEntry
    from stratum_b200.weights import write_random_model
    ToyConfig = _define_toy()
    raw = {"architectures": ["ToyRoutedForCausalLM"], "layers": 3, "hidden": 40, "inner": 56, "experts": 5,
           "max_positions": 96, "vocab": 77, "eps": 1e-6}
    cfg = ToyConfig.from_dict(raw)
    path = write_random_model(str(tmp_path / "toy"), cfg, seed=9, std=0.3, dtype="float32")
    with open(os.path.join(path, "config.json")) as f:
        assert json.load(f)["architectures"] == ["ToyRoutedForCausalLM"]
    llm = Stratum(path, dtype="float32", max_tokens=1024, use_graphs=False)        # chosen by config.json
    c, w = load_plain(path)
    rng = np.random.default_rng(1)
    seqs = [rng.integers(0, 77, size=n).tolist() for n in (50, 9, 80)]
    refs, used = [], set()
    for s in seqs:
        r, u = _plain_toy(c, w, s)
        refs.append(r); used |= u
    assert len(used) >= 3                                # the router really sends tokens to different experts
    tol = lambda r: 3e-5 * np.max(np.abs(r))                                                      # noqa: E731
    slots = [llm.acquire() for _ in seqs]
    cut = [33, 2, 70]
    out = llm.step([StepEntry(s, q[:n], [0, n - 1]) for s, q, n in zip(slots, seqs, cut)]).cpu().numpy()
    for i in range(3):
        assert np.max(np.abs(out[2 * i] - refs[i][0])) < tol(refs[i])
        assert np.max(np.abs(out[2 * i + 1] - refs[i][cut[i] - 1])) < tol(refs[i])
    live, k = [0, 1, 2], 0
    while live:                                          # one token each; the shorter sequences end earlier
        out = llm.step([StepEntry(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live]).cpu().numpy()
        for row, i in enumerate(live):
            assert np.max(np.abs(out[row] - refs[i][cut[i] + k])) < tol(refs[i]), (i, k)
        k += 1
        for i in list(live):
            if cut[i] + k >= len(seqs[i]):
                llm.release(slots[i]); live.remove(i)
    llm.engine.cache.check()
    # the same positions matter: a sequence shifted by one token is another sequence
    a = llm.generate([seqs[1]], max_new_tokens=4, stop_ids=())[0].tokens
    seq = list(seqs[1])
    for tok in a:
        ref = _plain_toy(c, w, seq)[0][-1]
        assert ref[tok] >= ref.max() - 1e-4 * np.max(np.abs(ref))
        seq.append(tok)


def _define_arranged():
    """Three test-only arrangements and an architecture whose layers use one each, beside the built-in one."""
    from stratum_b200.config import Architecture, ModelConfig, register_architecture
    from stratum_b200.config.base import KeyReader
    from stratum_b200.parts import Arrangement, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_part

    @register_part("arrangement", "toy_parallel_shared_norm", replace=True)
    class ParallelSharedNorm(Arrangement):
        """x += mixer(n(x)) + feed_forward(n(x)): one norm, both parts read the same normed rows."""
        slots = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def forward(self, layer, x, step, cache):
            xn = layer.part("norm").forward(x)
            layer.part("mixer").forward(xn, x, step, cache)
            layer.part("feed_forward").forward(xn, x, step)

    @register_part("arrangement", "toy_sandwich", replace=True)
    class Sandwich(Arrangement):
        """x += post_a(mixer(pre_a(x))); x += post_b(feed_forward(pre_b(x))): four norms.  The feed-forward
        and its two norms may be left out."""
        slots = {"pre_mixer": "norm", "mixer": "mixer", "post_mixer": "norm",
                 "pre_feed_forward": "norm", "feed_forward": "feed_forward", "post_feed_forward": "norm"}
        optional = ("pre_feed_forward", "feed_forward", "post_feed_forward")

        def forward(self, layer, x, step, cache):
            out = torch.zeros_like(x)                      # parts add their result into what they are given
            layer.part("mixer").forward(layer.part("pre_mixer").forward(x), out, step, cache)
            x += layer.part("post_mixer").forward(out).float()
            if layer.part("feed_forward") is not None:
                out = torch.zeros_like(x)
                layer.part("feed_forward").forward(layer.part("pre_feed_forward").forward(x), out, step)
                x += layer.part("post_feed_forward").forward(out).float()

    @dataclass(frozen=True)
    class ArrangedConfig(ModelConfig):
        hidden: int
        inner: int
        vocab: int
        eps: float
        torch_dtype: str = "float32"
        architecture = "ToyArrangedForCausalLM"

        @classmethod
        def from_dict(cls, raw: Dict[str, Any]):
            r = KeyReader(raw)
            out = cls(r.integer("hidden"), r.integer("inner"), r.integer("vocab"), r.number("eps", 1e-5))
            r.finish()
            return out

        def to_dict(self):
            return {"architectures": [self.architecture], "hidden": self.hidden, "inner": self.inner,
                    "vocab": self.vocab, "eps": self.eps}

    def describe(cfg):
        norm = lambda p, n=cfg.hidden: PartSpec("rmsnorm", {"size": n, "eps": cfg.eps, "prefix": p})   # noqa: E731
        rope = PartSpec("rope", {"rope_dim": 16, "theta": 10000.0, "interleaved": False, "scaling": None})

        def att(qk_norm):
            return PartSpec("gqa_attention", {
                "hidden": cfg.hidden, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16, "bias": False, "window": 0,
                "scale": None, "position": rope, "prefix": "attn.",
                "q_norm": norm("q_norm.", 16) if qk_norm else None,
                "k_norm": norm("k_norm.", 16) if qk_norm else None})

        ff = PartSpec("swiglu", {"hidden": cfg.hidden, "intermediate": cfg.inner, "bias": False, "prefix": "ff."})
        layers = (
            LayerSpec("toy_parallel_shared_norm", {"norm": norm("n."), "mixer": att(False), "feed_forward": ff},
                      "l.0."),
            LayerSpec("toy_sandwich", {"pre_mixer": norm("n1."), "mixer": att(True), "post_mixer": norm("n2."),
                                       "pre_feed_forward": norm("n3."), "feed_forward": ff,
                                       "post_feed_forward": norm("n4.")}, "l.1."),
            LayerSpec("toy_sandwich", {"pre_mixer": norm("n1."), "mixer": att(False), "post_mixer": norm("n2.")},
                      "l.2."),                                                     # no feed-forward at all
            LayerSpec("prenorm_residual", {"mixer_norm": norm("n1."), "mixer": att(True),
                                           "feed_forward_norm": norm("n2."), "feed_forward": ff}, "l.3."))
        return ModelSpec(cfg.hidden, cfg.vocab,
                         PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.hidden, "prefix": "emb."}),
                         layers, tuple(ScheduleEntry(i) for i in range(4)), norm("nf."),
                         PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.hidden, "tied": True,
                                                  "prefix": "head."}))

    register_architecture(Architecture(("ToyArrangedForCausalLM",), "test-only: arrangements that own other parts",
                                       ArrangedConfig, describe), replace=True)
    return ArrangedConfig


def _plain_arranged(cfg, w, toks):
    from plain import llama_plain as P
    T, eps = len(toks), cfg["eps"]
    pos = np.arange(T)
    inv = P.rope_inv_freq(16, 10000.0)

    def att(xn, p, qk_norm):
        q = P.linear(xn, w[p + "attn.q_proj.weight"]).reshape(T, 4, 16)
        k = P.linear(xn, w[p + "attn.k_proj.weight"]).reshape(T, 2, 16)
        v = P.linear(xn, w[p + "attn.v_proj.weight"]).reshape(T, 2, 16)
        if qk_norm:
            q = P.head_rms_norm(q, w[p + "attn.q_norm.weight"], eps)
            k = P.head_rms_norm(k, w[p + "attn.k_norm.weight"], eps)
        q, k = P.apply_rope(q, pos, inv, False), P.apply_rope(k, pos, inv, False)
        return P.linear(P.causal_gqa_attention(q, k, v).reshape(T, 64), w[p + "attn.o_proj.weight"])

    ffn = lambda xn, p: P.swiglu_mlp(xn, w, p + "ff.")      # noqa: E731
    n = lambda x, name: P.rms_norm(x, w[name + "weight"], eps)   # noqa: E731
    x = P.embed(w["emb.weight"], toks)
    xn = n(x, "l.0.n.")
    x = x + att(xn, "l.0.", False) + ffn(xn, "l.0.")
    x = x + n(att(n(x, "l.1.n1."), "l.1.", True), "l.1.n2.")
    x = x + n(ffn(n(x, "l.1.n3."), "l.1."), "l.1.n4.")
    x = x + n(att(n(x, "l.2.n1."), "l.2.", False), "l.2.n2.")
    x = x + att(n(x, "l.3.n1."), "l.3.", True)
    x = x + ffn(n(x, "l.3.n2."), "l.3.")
    return P.linear(n(x, "nf."), w["emb.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_arrangements_that_own_other_parts(tmp_path, dtype):
    from helpers import TOL, load_plain
    from stratum_b200 import StepEntry, Stratum
    from stratum_b200.weights import write_random_model
    ArrangedConfig = _define_arranged()
    raw = {"architectures": ["ToyArrangedForCausalLM"], "hidden": 64, "inner": 96, "vocab": 90, "eps": 1e-5}

    def gains(tensors):                                     # norm gains other than one, so that every norm counts
        g = torch.Generator().manual_seed(1)
        for name, t in tensors.items():
            if name.endswith("weight") and t.dim() == 1:
                t.copy_((0.5 + torch.rand(t.shape, generator=g)).to(t.dtype))

    from stratum_b200.engine.model import expected_tensors
    from stratum_b200.weights.random_init import random_tensors, _TORCH_DTYPES
    from stratum_b200.weights.safetensors_io import write_safetensors
    cfg = ArrangedConfig.from_dict(raw)
    names = expected_tensors(cfg)
    assert "l.1.attn.q_norm.weight" in names and "l.0.attn.q_norm.weight" not in names
    assert "l.2.n1.weight" in names and not any(n.startswith("l.2.ff.") for n in names)
    tensors = random_tensors(names, 3, 0.2, _TORCH_DTYPES[dtype])
    gains(tensors)
    path = str(tmp_path / "arranged")
    os.makedirs(path)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(dict(cfg.to_dict(), torch_dtype=dtype), f)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors)
    c, w = load_plain(path)
    llm = Stratum(path, dtype=dtype, max_tokens=1024)
    rng = np.random.default_rng(6)
    seqs = [rng.integers(0, 90, size=n).tolist() for n in (70, 12)]
    refs = [_plain_arranged(c, w, s) for s in seqs]
    tol = lambda r: TOL[dtype] * np.max(np.abs(r))          # noqa: E731
    slots = [llm.acquire() for _ in seqs]
    cut = [60, 5]
    out = llm.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, cut)]).cpu().numpy()
    assert np.max(np.abs(out[:60] - refs[0][:60])) < tol(refs[0])
    assert np.max(np.abs(out[60:] - refs[1][:5])) < tol(refs[1])
    for k in range(7):                                      # one token each, from the cache
        out = llm.step([StepEntry(slots[i], [seqs[i][cut[i] + k]], [0]) for i in (0, 1)]).cpu().numpy()
        for i in (0, 1):
            assert np.max(np.abs(out[i] - refs[i][cut[i] + k])) < tol(refs[i]), (i, k)
    # a spec that does not give an arrangement its parts is refused with the names
    from stratum_b200.engine.model import Layer
    from stratum_b200.parts import LayerSpec, PartSpec
    with pytest.raises(ValueError, match="missing \\['mixer'\\].*not known to it \\['mixr'\\]"):
        Layer(LayerSpec("toy_parallel_shared_norm", {"norm": PartSpec("rmsnorm", {"size": 8, "eps": 1e-5}),
                                                     "mixr": PartSpec("rmsnorm", {"size": 8, "eps": 1e-5}),
                                                     "feed_forward": PartSpec("swiglu", {"hidden": 8,
                                                                                         "intermediate": 8})},
                        "x."), None)
