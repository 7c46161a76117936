"""A toy mixer with fixed-size state of its own, defined here, is registered, built and stepped
without a change to the library's files."""
import json
import os
from dataclasses import dataclass
from typing import Any, Dict

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _define_toy():
    """Registers (once) a mixer, a configuration and an architecture that live only in this test."""
    from stratum_b200.cache import StateSpec
    from stratum_b200.config import Architecture, ModelConfig, register_architecture
    from stratum_b200.config.base import KeyReader
    from stratum_b200.parts import LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry, TensorSpec, register_part

    @register_part("mixer", "toy_decay_state", replace=True)
    class DecayState(Mixer):
        """state <- decay * state + xn W_in per token, in order; residual += state W_out.
        The state is one float32 vector of `width` per sequence: no keys, no values, no pages."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.hidden, self.width, self.decay = spec["hidden"], spec["width"], spec["decay"]

        def tensors(self):
            return {self.prefix + "in.weight": TensorSpec((self.width, self.hidden)),
                    self.prefix + "out.weight": TensorSpec((self.hidden, self.width))}

        def bind(self, weights):
            self.w_in = weights[self.prefix + "in.weight"].float()
            self.w_out = weights[self.prefix + "out.weight"].float()

        def cache_spec(self):
            return StateSpec((self.width,), "float32")

        def forward(self, xn, residual, step, cache):
            u = xn.float() @ self.w_in.T                           # a test may use library operators
            slots = step.seq_slot.tolist()
            start = step.seq_start.tolist()
            for i, slot in enumerate(slots):
                s = cache.state[slot]
                for r in range(start[i], start[i + 1]):
                    s = self.decay * s + u[r]
                    residual[r] += s @ self.w_out.T
                if cache.writes:
                    cache.state[slot] = s

    @register_part("mixer", "toy_decay_state_on_device", replace=True)
    class DecayStateOnDevice(DecayState):
        """The same mixer written so that a decode step can be captured in a CUDA graph: device operators on
        the current stream only, nothing copied to or from the host, loop counts from the step's host numbers.  Padding
        rows of a captured step carry the spare state row (slot number = max_seqs), so they need no mask."""

        def forward(self, xn, residual, step, cache):
            u = xn.float() @ self.w_in.T
            slot = step.seq_slot.long()
            s = cache.state.index_select(0, slot)                                  # [sequences, width]
            first = step.seq_start[:-1].long()
            n_new = step.seq_start[1:] - step.seq_start[:-1]                       # stays on the device
            last_row = xn.shape[0] - 1
            for t in range(step.max_new):
                live = (n_new > t).unsqueeze(1)
                rows = (first + t).clamp(max=last_row)
                s = torch.where(live, self.decay * s + u.index_select(0, rows), s)
                residual.index_add_(0, rows, (s @ self.w_out.T) * live)
            if cache.writes:
                cache.state.index_copy_(0, slot, s)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        n_layers: int
        hidden: int
        width: int
        decay: float
        vocab: int
        eps: float
        mixer: str = "toy_decay_state"
        torch_dtype: str = "float32"
        architecture = "ToyStateForCausalLM"

        @classmethod
        def from_dict(cls, raw: Dict[str, Any]):
            r = KeyReader(raw)
            out = cls(r.integer("layers"), r.integer("hidden"), r.integer("width"), r.number("decay"),
                      r.integer("vocab"), r.number("eps", 1e-5), r.string("mixer", "toy_decay_state"))
            r.finish()
            return out

        def to_dict(self):
            return {"architectures": [self.architecture], "layers": self.n_layers, "hidden": self.hidden,
                    "width": self.width, "decay": self.decay, "vocab": self.vocab, "eps": self.eps,
                    "mixer": self.mixer}

    def describe(cfg):
        norm = lambda p: PartSpec("rmsnorm", {"size": cfg.hidden, "eps": cfg.eps, "prefix": p})   # noqa: E731
        layers = []
        for i in range(cfg.n_layers):
            # odd layers mix with the toy state, even layers with attention: one model, two kinds of mixer
            mixer = PartSpec(cfg.mixer, {"hidden": cfg.hidden, "width": cfg.width, "decay": cfg.decay,
                                                 "prefix": "mix."}) if i % 2 else \
                PartSpec("gqa_attention", {"hidden": cfg.hidden, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16,
                                           "bias": False, "window": 0, "scale": None, "position": None,
                                           "prefix": "attn."})
            layers.append(LayerSpec("prenorm_residual", {
                "mixer_norm": norm("n1."), "mixer": mixer, "feed_forward_norm": norm("n2."),
                "feed_forward": PartSpec("swiglu", {"hidden": cfg.hidden, "intermediate": 2 * cfg.hidden,
                                                    "bias": False, "prefix": "ff."})}, f"l.{i}."))
        return ModelSpec(cfg.hidden, cfg.vocab,
                         PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.hidden, "prefix": "emb."}),
                         tuple(layers), tuple(ScheduleEntry(i) for i in range(cfg.n_layers)), norm("nf."),
                         PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.hidden, "tied": True,
                                                  "prefix": "head."}))

    register_architecture(Architecture(("ToyStateForCausalLM",), "test-only: attention and decaying-state mixers",
                                       ToyConfig, describe), replace=True)
    return ToyConfig


def _plain_toy(cfg, w, toks):
    from plain import llama_plain as P
    x = P.embed(w["emb.weight"], toks)
    T = len(toks)
    for i in range(cfg["layers"]):
        p = f"l.{i}."
        xn = P.rms_norm(x, w[p + "n1.weight"], cfg["eps"])
        if i % 2:
            s = np.zeros(cfg["width"])
            for r in range(T):
                s = cfg["decay"] * s + xn[r] @ w[p + "mix.in.weight"].T
                x[r] = x[r] + s @ w[p + "mix.out.weight"].T
        else:
            q = P.linear(xn, w[p + "attn.q_proj.weight"]).reshape(T, 2, 16)
            k = P.linear(xn, w[p + "attn.k_proj.weight"]).reshape(T, 1, 16)
            v = P.linear(xn, w[p + "attn.v_proj.weight"]).reshape(T, 1, 16)
            x = x + P.linear(P.causal_gqa_attention(q, k, v).reshape(T, 32), w[p + "attn.o_proj.weight"])
        xn = P.rms_norm(x, w[p + "n2.weight"], cfg["eps"])
        x = x + P.linear(P.silu(P.linear(xn, w[p + "ff.gate_proj.weight"])) * P.linear(xn, w[p + "ff.up_proj.weight"]),
                         w[p + "ff.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["nf.weight"], cfg["eps"]), w["emb.weight"])


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from helpers import load_plain
    from stratum_b200 import Stratum, StepEntry
    from stratum_b200.cache import StateSpec
    from stratum_b200.weights import write_random_model
    ToyConfig = _define_toy()
    raw = {"architectures": ["ToyStateForCausalLM"], "layers": 4, "hidden": 48, "width": 24, "decay": 0.9,
           "vocab": 120, "eps": 1e-5}
    cfg = ToyConfig.from_dict(raw)
    path = write_random_model(str(tmp_path / "toy"), cfg, seed=4, std=0.1, dtype="float32")     # random-weights mode
    with open(os.path.join(path, "config.json")) as f:
        assert json.load(f)["architectures"] == ["ToyStateForCausalLM"]
    llm = Stratum(path, dtype="float32", max_tokens=1024)                                        # chosen by config.json
    assert not llm.prompt_graphs.enabled        # a part that does not say `replays_prompts`: prompts launch by launch
    groups = llm.engine.cache.groups
    assert len(groups) == 2 and sum(isinstance(g.spec, StateSpec) for g in groups) == 1
    assert [g.state.shape for g in groups if g.state is not None] == [(2, llm.engine.cache.max_seqs + 1, 24)]
    c, w = load_plain(path)
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 120, size=n).tolist() for n in (40, 7, 70)]
    refs = [_plain_toy(c, w, s) for s in seqs]
    tol = lambda r: 3e-5 * np.max(np.abs(r))                                                      # noqa: E731
    for rnd in range(2):                       # twice: the second round reuses slots, whose state must be zeroed
        slots = [llm.acquire() for _ in seqs]
        cut = [30, 3, 64]
        out = llm.step([StepEntry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, cut)]).cpu().numpy()
        for i in range(3):
            assert np.max(np.abs(out[i] - refs[i][cut[i] - 1])) < tol(refs[i])
        live, k = [0, 1, 2], 0
        while live:
            out = llm.step([StepEntry(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                assert np.max(np.abs(out[row] - refs[i][cut[i] + k])) < tol(refs[i]), (rnd, i, k)
            k += 1
            for i in list(live):
                if cut[i] + k >= len(seqs[i]):
                    llm.release(slots[i]); live.remove(i)
    llm.engine.cache.check()
    # and through the generation loop (this mixer reads tensors on the host, which a graph capture refuses, so
    # the model steps launch by launch; the next test has the capturable form)
    plain_llm = Stratum(path, dtype="float32", max_tokens=1024, use_graphs=False)
    res = plain_llm.generate([seqs[1]], max_new_tokens=5, stop_ids=())
    seq = list(seqs[1])
    for tok in res[0].tokens:
        ref = _plain_toy(c, w, seq)[-1]
        assert ref[tok] >= ref.max() - 1e-4 * np.max(np.abs(ref))
        seq.append(tok)


def test_toy_state_under_replayed_graphs(tmp_path):
    """Generation with graphs on (the default) over a mixer with fixed-size state: the state must be updated
    exactly once per step, also in the step that captures a new graph, and a slot taken again starts from zero.
    Tokens and every step's logits against graphs off and against the plain restatement, in two rounds."""
    from helpers import load_plain
    from stratum_b200 import Stratum
    from stratum_b200.weights import write_random_model
    ToyConfig = _define_toy()
    raw = {"architectures": ["ToyStateForCausalLM"], "layers": 4, "hidden": 48, "width": 24, "decay": 0.9,
           "vocab": 120, "eps": 1e-5, "mixer": "toy_decay_state_on_device"}
    path = write_random_model(str(tmp_path / "toy"), ToyConfig.from_dict(raw), seed=6, std=0.1, dtype="float32")
    c, w = load_plain(path)
    graphed = Stratum(path, dtype="float32", max_tokens=2048)
    assert graphed.graphs is not None
    eager = Stratum(path, dtype="float32", max_tokens=2048, use_graphs=False)
    rng = np.random.default_rng(2)
    for rnd in range(2):
        lens, budgets = ((5, 17, 3), (9, 4, 12)) if rnd == 0 else ((8, 2, 30, 6), (6, 14, 3, 9))
        prompts = [rng.integers(0, 120, size=n).tolist() for n in lens]
        seen = []
        out = graphed.generate(prompts, max_new_tokens=list(budgets), stop_ids=(),
                               on_logits=lambda lg, ids: seen.append(lg.cpu().numpy().copy()))
        ref = eager.generate(prompts, max_new_tokens=list(budgets), stop_ids=())
        assert [r.tokens for r in out] == [r.tokens for r in ref]
        plain = [_plain_toy(c, w, p + r.tokens) for p, r in zip(prompts, out)]
        live = list(range(len(prompts)))
        for step, lg in enumerate(seen):
            for row, i in enumerate(live):
                want = plain[i][len(prompts[i]) - 1 + step]
                assert np.max(np.abs(lg[row] - want)) < 3e-5 * np.max(np.abs(want)), (rnd, step, i)
            live = [i for i in live if step + 1 < budgets[i]]
    assert graphed.graphs.captures >= 3
    graphed.engine.cache.check()
