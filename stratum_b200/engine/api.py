"""The Python entry point: open a model folder, step it, generate from it.

    from stratum_b200 import Stratum
    llm = Stratum("/path/to/model_dir", dtype="bfloat16", max_tokens=8192)
    out = llm.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)      # -> list of GenerationResult

The reference has no library API (everything is static in one translation unit,
CONTRIBUTING.md:52); the names follow its command line and environment switches.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..config.base import ModelConfig
from ..sampling import Pcg32, Sampler, SamplingParams
from .generate import Backend, GenerationResult, generate
from .graphs import DecodeGraphs, PromptGraphs
from .model import load_model, random_model_on_device
from .step import Engine, StepEntry

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


class _EngineBackend(Backend):
    def __init__(self, engine: Engine, sampler: Sampler, graphs=None, prompt_graphs=None):
        self.engine, self.sampler, self.graphs, self.prompt_graphs = engine, sampler, graphs, prompt_graphs
        self.n_pages, self.max_seqs = engine.cache.n_pages, engine.cache.max_seqs
        self.on_logits = None          # optional hook(logits [n, vocab] on the device, picked ids list)

    def acquire(self) -> int:
        return self.engine.acquire()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    # one step ahead of the host (replayed graphs only; with an on_logits hook every step is read before the next)
    @property
    def runs_ahead(self) -> bool:
        return self.graphs is not None and self.on_logits is None

    def launch_ahead(self, work, streams, params, after=None, rows_of=None):
        uniforms = None if params.greedy else [st.uniform() for st in streams]
        return self.graphs.launch([s for s, _ in work], [t for _, t in work], params.temperature, params.top_k,
                                  params.top_p, uniforms, trusted=True, advance_now=True, after=after,
                                  rows_of=rows_of)

    def collect(self, handle):
        picked, values, _ = self.graphs.collect(handle)
        return picked, values

    def step_and_pick(self, work, streams, params):
        if self.graphs is not None and all(len(toks) == 1 for _, toks in work):
            uniforms = None if params.greedy else [st.uniform() for st in streams]
            picked, values, captured = self.graphs.step([s for s, _ in work], [toks[0] for _, toks in work],
                                                        params.temperature, params.top_k, params.top_p, uniforms,
                                                        trusted=True)     # the loop feeds back ids picked here
            if self.on_logits is not None:
                self.on_logits(captured.logits[:len(work)], picked)
            return picked, values
        entries = [StepEntry(s, toks, [len(toks) - 1]) for s, toks in work]
        shape = self.prompt_graphs.shape_of(entries) if self.prompt_graphs is not None else None
        logits = self.prompt_graphs.step(entries, shape) if shape is not None else self.engine.step(entries)
        ids, values = self.sampler.pick(logits, params, streams, want_values=True)
        both = torch.stack([ids.to(torch.float64), values.to(torch.float64)]).cpu()     # one device-to-host copy
        picked = [int(v) for v in both[0].tolist()]
        if self.on_logits is not None:
            self.on_logits(logits, picked)
        return picked, both[1].tolist()


class Stratum:
    """A loaded model with its cache.  dtype: "bfloat16" (serving kernels) or "float32" (true 32-bit)."""

    def __init__(self, model_dir: Optional[str] = None, dtype: str = "bfloat16", max_tokens: int = 4096,
                 max_seqs: Optional[int] = None, device: str = "cuda", use_graphs: bool = True, *,
                 _model=None, _config=None):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype {dtype!r} not one of {sorted(_DTYPES)}")
        if not torch.cuda.is_available():
            raise RuntimeError("stratum_b200 needs a CUDA device (sm_100a); there is no CPU path")
        if _model is None:
            _model, _config = load_model(model_dir, _DTYPES[dtype], device)
        self.model, self.config = _model, _config
        self.dtype = dtype
        self.engine = Engine(self.model, max_tokens=max_tokens, max_seqs=max_seqs)
        self.sampler = Sampler(self.model.runtime.device)
        self.graphs = DecodeGraphs(self.engine) if use_graphs else None
        # short prompt steps are replayed too (STRATUM_PROMPT_GRAPHS=0: launch by launch, for measurements)
        self.prompt_graphs = (PromptGraphs(self.engine)
                              if use_graphs and os.environ.get("STRATUM_PROMPT_GRAPHS", "1") != "0" else None)
        self._backend = _EngineBackend(self.engine, self.sampler, self.graphs, self.prompt_graphs)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int = 0, dtype: str = "bfloat16", max_tokens: int = 4096,
                    max_seqs: Optional[int] = None, device: str = "cuda", std: float = 0.02,
                    use_graphs: bool = True) -> "Stratum":
        """Random weights made on the device from (config, seed); nothing is read or written."""
        model = random_model_on_device(config, seed, _DTYPES[dtype], device, std)
        return cls(None, dtype, max_tokens, max_seqs, device, use_graphs, _model=model, _config=config)

    # -- stepping by hand -----------------------------------------------------
    def acquire(self) -> int:
        return self.engine.acquire()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; float32 logits [wanted places, vocab] on the device.  (A short prompt step is
        replayed as a captured graph, like decode steps; the logits are then copied out of the graph's output.)"""
        shape = self.prompt_graphs.shape_of(entries) if self.prompt_graphs is not None else None
        if shape is not None:
            return self.prompt_graphs.step(entries, shape).clone()
        return self.engine.step(entries)

    def decode_step(self, slots: Sequence[int], tokens: Sequence[int],
                    sampling: SamplingParams = SamplingParams(), streams: Optional[Sequence[Pcg32]] = None,
                    with_logits: bool = False):
        """One token for each slot, picked on the device: (ids, logits of the ids) as host lists.  The step
        runs as a replayed CUDA graph (or launch by launch when graphs are off).  with_logits: a third value,
        the step's float32 logits [slots, vocab] on the device (valid until the next step)."""
        if self.graphs is None:
            kept = []
            self._backend.on_logits = (lambda lg, ids: kept.append(lg)) if with_logits else None
            try:
                ids, vals = self._backend.step_and_pick([(s, [t]) for s, t in zip(slots, tokens)], streams, sampling)
            finally:
                self._backend.on_logits = None
            return (ids, vals, kept[0]) if with_logits else (ids, vals)
        uniforms = None if sampling.greedy else [st.uniform() for st in streams]
        ids, vals, c = self.graphs.step(slots, tokens, sampling.temperature, sampling.top_k, sampling.top_p, uniforms)
        return (ids, vals, c.logits[:len(ids)]) if with_logits else (ids, vals)

    def launch_decode(self, slots: Sequence[int], tokens: Sequence[int],
                      sampling: SamplingParams = SamplingParams(), streams: Optional[Sequence[Pcg32]] = None):
        """Start one token for each slot and return a handle without waiting for the result; `collect(handle)`
        gives (ids, logits of the ids).  The sequences' lengths are advanced at once, so the next step may be
        launched before this one is collected (replayed graphs only).  Collect in the order of the launches, and
        keep at most two steps in flight."""
        if self.graphs is None:
            raise RuntimeError("launch_decode needs replayed graphs (use_graphs=True)")
        uniforms = None if sampling.greedy else [st.uniform() for st in streams]
        return self.graphs.launch(slots, tokens, sampling.temperature, sampling.top_k, sampling.top_p, uniforms,
                                  advance_now=True)

    def collect(self, handle):
        ids, vals, _ = self.graphs.collect(handle)
        return ids, vals

    # -- generation ---------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens=16, stop_ids: Optional[Sequence[int]] = None,
                 sampling: SamplingParams = SamplingParams(), max_batch: Optional[int] = None,
                 on_token: Optional[Callable] = None, want_values: bool = False,
                 on_logits: Optional[Callable] = None,
                 stream_ids: Optional[Sequence[int]] = None, run_ahead: bool = True) -> List[GenerationResult]:
        """stop_ids None: the configuration's eos ids; () : none.
        on_logits(logits on the device [live sequences, vocab], picked ids) is called after every step.
        stream_ids: the random stream each request draws from (default: its index in this call).
        run_ahead: decode steps are launched one ahead of the host's reading of the picked ids (replayed graphs
        only, and not with on_logits); the tokens are the same either way."""
        if stop_ids is None:
            stop_ids = tuple(getattr(self.config, "eos_token_ids", ()) or ())
        self._backend.on_logits = on_logits
        try:
            return generate(self._backend, prompts, max_new_tokens, stop_ids, sampling, max_batch, on_token,
                            want_values, stream_ids, run_ahead)
        finally:
            self._backend.on_logits = None
