"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early.

Requests are cut into batches that fit the cache; a batch's prompts run in one step, then one
token per live sequence per step.  A sequence ends on a stop id or at its token budget; it then
leaves the batch and its slot goes back at once, so later steps run only the live ones, and the
next batch reuses the slots.  The reference's loop is the single-sequence, fixed-count, greedy
case of this (stratum/native/stratum_arch_llama.inc.c:1605-1626, :2041-2061); its lock-step
multi-stream loop has no early end (:1493-1516).

The decisions (batching, who is live, why a sequence ended) are plain Python over a small
backend interface, so they are tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..cache.pages import pages_for
from ..sampling.params import SamplingParams
from ..sampling.pcg32 import Pcg32


class CapacityError(ValueError):
    """A request cannot fit the cache even alone."""


@dataclass
class GenerationResult:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)     # generated ids (a stop id, if hit, is the last)
    finish_reason: str = ""                               # "stop" | "length"
    logit_values: List[float] = field(default_factory=list)   # logit of each generated id (when asked for)


class Backend:
    """What the loop needs from an engine.  `step_and_pick` runs one step for (slot, tokens)
    pairs and returns the id picked from the logits at each pair's last token (and its logit)."""

    n_pages: int
    max_seqs: int

    def acquire(self) -> int: raise NotImplementedError
    def release(self, slot: int) -> None: raise NotImplementedError

    def step_and_pick(self, work: Sequence[Tuple[int, Sequence[int]]], streams: Sequence[Pcg32],
                      params: SamplingParams) -> Tuple[List[int], List[float]]:
        raise NotImplementedError


def plan_batches(prompt_lens: Sequence[int], max_new: Sequence[int], n_pages: int, max_seqs: int,
                 max_batch: Optional[int] = None) -> List[List[int]]:
    """Cut requests, in order, into batches whose worst-case page need fits the cache."""
    cap = min(max_seqs, max_batch) if max_batch else max_seqs
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, (n, m) in enumerate(zip(prompt_lens, max_new)):
        if n < 1:
            raise ValueError(f"request {i}: empty prompt")
        # the last generated token is never fed back, so a sequence holds at most n + m - 1 keys
        need = pages_for(n + max(m, 1) - 1)
        if need > n_pages:
            raise CapacityError(f"request {i}: {n} prompt + {m} new tokens exceeds KV capacity "
                                f"({n_pages * 64} tokens)")
        if cur and (len(cur) >= cap or used + need > n_pages):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens,
             stop_ids: Sequence[int] = (), params: SamplingParams = SamplingParams(),
             max_batch: Optional[int] = None,
             on_token: Optional[Callable[[int, int, int, int, float], None]] = None,
             want_values: bool = False, stream_ids: Optional[Sequence[int]] = None) -> List[GenerationResult]:
    """Generate for every prompt.  max_new_tokens: one int or one per request.
    on_token(request, index of the new token, token fed in, token picked, its logit).
    stream_ids: which random stream of the seed each request draws from (default: its index in this call).
    A request keeps its draws when it is given the same stream in another call, whatever else is in the
    batch (the reference seeds stream s with seed + s * 0x9E3779B97F4A7C15,
    stratum/native/stratum_arch_qwen35.inc.c:14010-14018)."""
    n_req = len(prompts)
    budgets = [int(max_new_tokens)] * n_req if isinstance(max_new_tokens, int) else [int(m) for m in max_new_tokens]
    if len(budgets) != n_req:
        raise ValueError("max_new_tokens: one value, or one per prompt")
    stop = set(int(s) for s in stop_ids)
    results = [GenerationResult(prompt_len=len(p)) for p in prompts]
    if stream_ids is None:
        stream_ids = range(n_req)
    elif len(stream_ids) != n_req:
        raise ValueError("stream_ids: one per prompt")
    streams = [Pcg32(params.seed, int(i)) for i in stream_ids]
    for batch in plan_batches([len(p) for p in prompts], budgets, backend.n_pages, backend.max_seqs, max_batch):
        live = [i for i in batch if budgets[i] > 0]
        for i in batch:
            if budgets[i] <= 0:
                results[i].finish_reason = "length"
        slots = {i: backend.acquire() for i in live}
        try:
            feed = {i: list(prompts[i]) for i in live}          # prompts first, then one token each
            while live:
                picked, values = backend.step_and_pick([(slots[i], feed[i]) for i in live],
                                                       [streams[i] for i in live], params)
                still = []
                for i, tok, val in zip(live, picked, values):
                    res = results[i]
                    if on_token is not None:
                        on_token(i, len(res.tokens), feed[i][-1], tok, val)
                    res.tokens.append(tok)
                    if want_values:
                        res.logit_values.append(val)
                    if tok in stop:
                        res.finish_reason = "stop"
                    elif len(res.tokens) >= budgets[i]:
                        res.finish_reason = "length"
                    if res.finish_reason:
                        backend.release(slots.pop(i))           # ends early: its slot is free at once
                    else:
                        feed[i] = [tok]
                        still.append(i)
                live = still
        finally:
            for s in slots.values():
                backend.release(s)
    return results
