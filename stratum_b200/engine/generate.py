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
    pairs and returns the id picked from the logits at each pair's last token (and its logit).

    A backend that can start a one-token step without waiting for its result says so with `runs_ahead` and
    gives `launch_ahead(work, streams, params, after=None, rows_of=None) -> handle`, where work is (slot, token)
    pairs and a token of None means "the id that the step `after` (launched before, not yet collected) picks
    in its row rows_of[i]", and `collect(handle) -> (picked ids, their logits)`.  The loop then keeps one step in
    flight while it reads the one before (the reference queues its decode steps on the GPU ahead of the host in
    the same way, stratum/native/stratum_arch_llama.inc.c:1992-2030)."""

    n_pages: int
    max_seqs: int
    runs_ahead = False

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
             want_values: bool = False, stream_ids: Optional[Sequence[int]] = None,
             run_ahead: bool = True) -> List[GenerationResult]:
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
        carried: List[int] = []          # slots of sequences that ended while a step launched ahead still carries them

        def take(i: int, fed: int, tok: int, val: float) -> bool:
            """Book one picked token; True if the request goes on."""
            res = results[i]
            if on_token is not None:
                on_token(i, len(res.tokens), fed, tok, val)
            res.tokens.append(tok)
            if want_values:
                res.logit_values.append(val)
            if tok in stop:
                res.finish_reason = "stop"
            elif len(res.tokens) >= budgets[i]:
                res.finish_reason = "length"
            return not res.finish_reason

        try:
            # the prompts, of unequal lengths, in one step
            picked, values = backend.step_and_pick([(slots[i], list(prompts[i])) for i in live],
                                                   [streams[i] for i in live], params) if live else ([], [])
            still = []
            for i, tok, val in zip(live, picked, values):
                if take(i, prompts[i][-1], tok, val):
                    still.append(i)
                else:
                    backend.release(slots.pop(i))               # ends early: its slot is free at once
            live = still
            if run_ahead and backend.runs_ahead:
                # one token per live sequence per step, the next step launched before this one's ids are read: it
                # takes them on the device.  Who hits a stop id is known a step late; such a sequence rides along
                # for one step more (its row is ignored, rows never mix) and its slot goes back after that step.
                flight = backend.launch_ahead([(slots[i], results[i].tokens[-1]) for i in live],
                                              [streams[i] for i in live], params) if live else None
                while flight is not None:
                    nxt = [i for i in live if not results[i].finish_reason
                           and len(results[i].tokens) + 1 < budgets[i]]                  # if no stop id comes
                    ahead = None
                    if nxt:
                        row = {i: r for r, i in enumerate(live)}
                        ahead = backend.launch_ahead([(slots[i], None) for i in nxt], [streams[i] for i in nxt],
                                                     params, after=flight, rows_of=[row[i] for i in nxt])
                    picked, values = backend.collect(flight)
                    while carried:                               # nothing in flight holds them any more
                        backend.release(carried.pop())
                    for i, tok, val in zip(live, picked, values):
                        if results[i].finish_reason:             # ended a step ago; this row was its ride along
                            continue
                        if not take(i, results[i].tokens[-1], tok, val):
                            if ahead is not None and i in nxt:
                                carried.append(slots.pop(i))
                            else:
                                backend.release(slots.pop(i))
                    flight, live = ahead, nxt
            else:
                while live:
                    picked, values = backend.step_and_pick([(slots[i], [results[i].tokens[-1]]) for i in live],
                                                           [streams[i] for i in live], params)
                    still = []
                    for i, tok, val in zip(live, picked, values):
                        if take(i, results[i].tokens[-1], tok, val):
                            still.append(i)
                        else:
                            backend.release(slots.pop(i))
                    live = still
        finally:
            for s in carried:
                backend.release(s)
            for s in slots.values():
                backend.release(s)
    return results
