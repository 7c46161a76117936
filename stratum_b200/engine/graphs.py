"""Decode steps as replayed CUDA graphs.

A decode step is some three hundred small launches; issued one by one from Python they cost more
host time than the GPU needs to run them.  So the whole step (embedding, every layer, final norm,
head, token pick) is captured once per shape into a CUDA graph and replayed: per step the host
fills one pinned buffer with the step's description (token ids, positions, page tables, sampling
numbers), copies it to the device in one go, replays, and reads the picked ids back, together with
the status word of the kernels' bounded waits.

Nothing runs twice.  Before a shape is captured the step is run once launch by launch (that compiles what
is missing and sizes the scratch buffers), but on padding rows only, which touch no sequence's keys, values
or state; the first real step of a shape is already a replay.  What a part must obey to be captured: its
forward launches on the current stream only, reads nothing back to the host, takes sizes from the
StepBatch's host numbers (never from device tensors), allocates only through torch or Runtime.scratch, and
leaves the cache of rows with sequence index -1 alone (their state row is the spare one, `max_seqs`).

A graph is specific to (rows, page-table width, how tokens are picked): rows is the batch padded up a little (padding
rows carry sequence index -1, which every kernel that touches the cache skips; rows never mix, so
padding changes no result), and the width is the next power of two of the pages the longest
sequence holds, which also fixes how the keys are split across warps.

A step is `launch` + `collect`.  A caller that launches the next step before it collects this one (the
generation loop does) lets that step take the picked ids on the device, through a small kernel in front of the
replay, so the GPU goes from one step to the next without waiting for the host: the reference queues its decode
steps on the GPU ahead of time for the same reason (stratum/native/stratum_arch_llama.inc.c:1992-2038).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS, pages_for
from .step import Engine, StepDescription, StepEntry, StepError


# How a graph picks its tokens: greedy, by a draw, or (many rows with top-k / top-p) by a draw with the sampling kernel
# that gives a row one block: with filters and more than SAMPLE_SPLIT_MAX_ROWS rows the kernel that cuts a row over
# 32 blocks queues thousands of blocks for the SMs and loses (110 against 83 us at 64 rows with top-k 50).
PICK_GREEDY, PICK_DRAW, PICK_FILTERED_MANY_ROWS = 0, 1, 2
SAMPLE_SPLIT_MAX_ROWS = 32


def pick_kind(rows: int, temperature: float, top_k: int, top_p: float) -> int:
    if not (temperature > 0.0):
        return PICK_GREEDY
    filtered = top_k > 0 or top_p < 1.0
    return PICK_FILTERED_MANY_ROWS if filtered and rows > SAMPLE_SPLIT_MAX_ROWS else PICK_DRAW


def padded_rows(n: int) -> int:
    """Rows a graph is captured for: exact up to 8, then the next multiple of 8."""
    return n if n <= 8 else ((n + 7) // 8) * 8


def width_bucket(n_pages: int) -> int:
    w = 1
    while w < n_pages:
        w *= 2
    return w


class _Captured:
    def __init__(self, engine: Engine, rows: int, width: int, pick: int):
        self.rows, self.width, self.pick = rows, width, pick
        self.greedy = pick == PICK_GREEDY
        B = rows
        self.desc = StepDescription(engine, B, B, B, width, pinned=True,
                                    extras=(("temperature", B), ("top_k", B), ("top_p", B), ("uniform", B),
                                            ("feed", B)))
        self.views = self.desc.views
        dev = engine.runtime.device
        # picked ids | their logits (float32 bits) | the kernels' status word: one copy back per step
        self.out = torch.zeros(2 * B + 1, dtype=torch.int32, device=dev)
        self.out_ids = self.out[:B]
        self.out_vals = self.out[B:2 * B].view(torch.float32)
        # two host buffers for the results, used in turn: a step may be launched before the one before it is read
        self.out_hosts = [torch.empty(2 * B + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.turn = 0
        self.uploaded = torch.cuda.Event()            # the description's copy to the device has been made
        self.upload_pending = False
        self.signature = None                         # (slots, cache epoch) the membership was last written for
        self.sampling = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels = 0
        self.scratch_epoch = -1
        self.logits: Optional[torch.Tensor] = None

    @property
    def total(self) -> int:
        return self.desc.total


class DecodeGraphs:
    """Runs one-token-per-sequence steps of an Engine through captured graphs."""

    def __init__(self, engine: Engine, max_graphs: int = 16):
        self.engine = engine
        self.max_graphs = max_graphs
        self.graphs: "OrderedDict[Tuple[int, int, bool], _Captured]" = OrderedDict()
        self.pool = None
        self.captures = 0
        self.h2d_bytes = self.d2h_bytes = 0           # of the last step

    # ------------------------------------------------------------------ building blocks
    def _forward_and_pick(self, c: _Captured) -> None:
        d = c.desc
        logits = self.engine.model.forward(d.batch(c.width * PAGE_TOKENS), self.engine.cache)
        f32 = lambda name: d.field(name).view(torch.float32)                     # noqa: E731
        if c.greedy:
            K.argmax(logits, c.out_ids, c.out_vals)
        else:
            K.sample(logits, f32("temperature"), d.field("top_k"), f32("top_p"), f32("uniform"), c.out_ids,
                     c.out_vals, one_block_per_row=c.pick == PICK_FILTERED_MANY_ROWS)
        c.out[2 * c.rows:].copy_(K.status_word())
        c.logits = logits

    def _capture(self, c: _Captured) -> None:
        """Warm up on padding rows only (no sequence's cache or state is touched), then capture."""
        d = c.desc
        d.write_membership([], [], None)
        d.write_tokens([], [])
        d.upload()
        self._forward_and_pick(c)
        torch.cuda.synchronize()
        K.check_status()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        g = torch.cuda.CUDAGraph()
        before = K.launch_count()
        with torch.cuda.graph(g, pool=self.pool):
            self._forward_and_pick(c)
        c.kernels = K.launch_count() - before
        K.count_launches(-c.kernels)                  # captured, not run
        c.graph = g
        c.scratch_epoch = K.scratch_epoch()
        c.signature = None
        self.captures += 1

    def _get(self, rows: int, width: int, pick: int) -> _Captured:
        key = (rows, width, pick)
        c = self.graphs.get(key)
        if c is not None and c.graph is not None and c.scratch_epoch != K.scratch_epoch():
            # a scratch buffer was regrown (and the old one freed) since this graph recorded its address
            del self.graphs[key]
            c = None
        if c is None:
            while len(self.graphs) >= self.max_graphs:
                self.graphs.popitem(last=False)
            c = _Captured(self.engine, rows, width, pick)
            self.graphs[key] = c
        else:
            self.graphs.move_to_end(key)
        return c

    # ------------------------------------------------------------------ one step
    def step(self, slots: Sequence[int], tokens: Sequence[int], temperature: float, top_k: int, top_p: float,
             uniforms: Optional[Sequence[float]], trusted: bool = False) -> Tuple[List[int], List[float], _Captured]:
        """One token for each slot; returns the picked ids and their logits (host lists).
        trusted: the tokens are ids this engine picked itself (no range check needed).
        On error nothing has changed: no sequence is longer than before."""
        return self.collect(self.launch(slots, tokens, temperature, top_k, top_p, uniforms, trusted))

    def launch(self, slots: Sequence[int], tokens: Sequence[Optional[int]], temperature: float, top_k: int,
               top_p: float, uniforms: Optional[Sequence[float]], trusted: bool = False,
               advance_now: bool = False, after: Optional["_InFlight"] = None,
               rows_of: Optional[Sequence[int]] = None) -> "_InFlight":
        """Start one token for each slot and return without waiting; `collect` gives the result.

        advance_now: the sequences' lengths are advanced here, at the launch, not at `collect`: a caller that
        launches the next step before it collects this one needs them so.  (A kernel that gives up a wait still
        raises at `collect`, but the lengths then stay advanced.)
        after / rows_of: the step launched just before this one (with advance_now), not yet collected, and for
        every slot its row there (-1: the token is given).  Such a slot's token is the id that step picks: it is
        fed back on the device, so the host launches this step before it has read the one before."""
        eng = self.engine
        cache = eng.cache
        B = len(slots)
        slots = list(slots)
        ahead = after is not None
        if ahead and not (advance_now and after.advanced):
            raise StepError("a step launched ahead of the one before needs both launched with advance_now")
        token_lists = [((0 if t is None else int(t)),) for t in tokens]
        eng.validate(slots, token_lists, None, trusted_tokens=trusted or ahead)
        ones = _ONES[:B] if B <= len(_ONES) else [1] * B
        cache.reserve(slots, ones)
        before = [cache.length(s) for s in slots]
        c = self._get(padded_rows(B), width_bucket(pages_for(max(before) + 1)),
                      pick_kind(padded_rows(B), temperature, top_k, top_p))
        if c.graph is None:
            self._capture(c)
        if c.upload_pending:                          # the pinned description is about to be rewritten
            c.uploaded.synchronize()
            c.upload_pending = False
        v = c.views
        # what a sequence holds changes every step; who is in the batch and which pages they own only now and then
        signature = (tuple(slots), cache.epoch)
        if signature != c.signature:
            c.signature = signature
            c.desc.write_membership(slots, ones, None)
        if c.sampling != (temperature, top_k, top_p):
            v["top_k"][:] = top_k
            v["temperature"].view(np.float32)[:] = temperature
            v["top_p"].view(np.float32)[:] = top_p
            c.sampling = (temperature, top_k, top_p)
        c.desc.write_tokens(token_lists, before)
        u = v["uniform"].view(np.float32)
        u[:] = 0.0
        if uniforms is not None:
            u[:B] = uniforms
        if ahead:
            v["feed"][:] = -1
            v["feed"][:B] = rows_of
        c.desc.upload()
        c.uploaded.record()
        c.upload_pending = True
        if ahead:
            K.feed_ids(c.desc.field("ids"), c.desc.field("feed"), after.captured.out_ids)
        c.graph.replay()
        K.count_launches(c.kernels)
        out_host = c.out_hosts[c.turn]
        c.turn ^= 1
        out_host.copy_(c.out, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        if advance_now:
            cache.advance(slots, ones)
        self.h2d_bytes, self.d2h_bytes = c.total * 4, (2 * c.rows + 1) * 4
        return _InFlight(c, slots, ones, out_host, done, advanced=advance_now)

    def collect(self, h: "_InFlight") -> Tuple[List[int], List[float], _Captured]:
        h.done.synchronize()
        c, B, R = h.captured, len(h.slots), h.captured.rows
        out = h.out_host.numpy()
        if out[2 * R] != 0:
            K.check_status()                          # raises, and clears the word
        if not h.advanced:
            self.engine.cache.advance(h.slots, h.ones)
        return out[:B].tolist(), out[R:R + B].view(np.float32).tolist(), c


class _InFlight:
    """A launched decode step whose result has not been read yet."""
    __slots__ = ("captured", "slots", "ones", "out_host", "done", "advanced")

    def __init__(self, captured, slots, ones, out_host, done, advanced):
        self.captured, self.slots, self.ones = captured, slots, ones
        self.out_host, self.done, self.advanced = out_host, done, advanced


_ONES = [1] * 1024


# ---------------------------------------------------------------------------------------------- prompt steps
def padded_tokens(n: int, limit: int) -> Optional[int]:
    """Tokens a prompt graph is captured for: multiples of 64 up to 512, of 128 above; None beyond `limit`."""
    p = ((n + 63) // 64) * 64 if n <= 512 else ((n + 127) // 128) * 128
    return p if p <= limit else None


def padded_seqs(n: int) -> int:
    w = 1
    while w < n:
        w *= 2
    return w


class _CapturedPrompt:
    def __init__(self):
        self.desc: Optional[StepDescription] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels = 0
        self.scratch_epoch = -1


class PromptGraphs:
    """Runs short prompt steps of an Engine (a batch's first step: prompts of unequal lengths) as replayed graphs.

    Issued launch by launch from Python a prompt step costs some ten microseconds of host time a launch, a dozen
    launches a layer; below a few hundred tokens (a few thousand for a small model) that is more than the GPU
    needs.  So a prompt step is captured once per shape (tokens padded up to a multiple of 64 or 128, sequences
    to a power of two, page tables to a power of two of pages) and replayed: the host writes the description
    (StepDescription.write_prompts) and replays.  Tokens beyond the step's have sequence index -1, sequences
    beyond the step's bring no token, and the query blocks of the attention are lists of a fixed length whose
    surplus entries are empty; rows never mix, so padding changes no result.  Only models whose parts all say
    `replays_prompts` are taken; a step of more than `max_tokens` tokens (there the GPU needs longer than the host:
    23.98 against 23.99 ms at 2,048 tokens on the Llama-8B shape), or one that wants more rows than it has
    sequences (trace replay asks for every position), runs launch by launch as before.

    Capturing a shape takes three passes (which query-block sizes are asked for; once launch by launch on
    padding only, so that every kernel has run and every scratch buffer exists; the capture), so a shape is
    captured when it is met for the second time (`capture_after` sightings run launch by launch first): a shape
    that never comes back costs nothing extra, one that does pays off from its third use on.
    """

    def __init__(self, engine: Engine, max_graphs: int = 12, max_tokens: int = 1024, capture_after: int = 1):
        self.engine = engine
        self.max_graphs, self.max_tokens, self.capture_after = max_graphs, max_tokens, capture_after
        self.sightings: Dict[Tuple[int, int, int], int] = {}
        self.graphs: "OrderedDict[Tuple[int, int, int], _CapturedPrompt]" = OrderedDict()
        self.pool = None
        self.captures = 0
        self.replays = 0
        self.enabled = engine.model.replays_prompts()

    def shape_of(self, entries: Sequence[StepEntry]) -> Optional[Tuple[int, int, int]]:
        """(padded tokens, padded sequences, page-table width) if this step is one that is replayed now, else
        None.  (Counts the sighting: call once per step.)"""
        key = self._shape(entries)
        if key is None or key in self.graphs:
            return key
        if len(self.sightings) > 4096:
            self.sightings.clear()
        n = self.sightings.get(key, 0)
        self.sightings[key] = n + 1
        return key if n >= self.capture_after else None

    def _shape(self, entries: Sequence[StepEntry]) -> Optional[Tuple[int, int, int]]:
        if not self.enabled or not entries:
            return None
        T = sum(len(e.tokens) for e in entries)
        S = padded_seqs(len(entries))
        if sum(len(e.want) for e in entries) > S or all(len(e.tokens) == 1 for e in entries):
            return None
        Tp = padded_tokens(T, self.max_tokens)
        if Tp is None:
            return None
        cache = self.engine.cache
        try:
            longest = max(cache.length(e.slot) + len(e.tokens) for e in entries)
        except Exception:
            return None                               # (a bad slot: the step function says so)
        return Tp, S, width_bucket(max(1, pages_for(longest)))

    def _all_padding(self, d: StepDescription) -> None:
        d.write_prompts([], [], [])
        d.write_tokens([], [])
        d.upload()

    def _capture(self, key: Tuple[int, int, int]) -> _CapturedPrompt:
        eng = self.engine
        Tp, S, width = key
        c = _CapturedPrompt()
        max_len = width * PAGE_TOKENS
        # 1. which query-block sizes the model asks for (with no tokens, nothing is launched for them)
        probe = StepDescription(eng, Tp, S, S, width)
        self._all_padding(probe)
        batch = probe.batch(max_len)
        batch.sizes_seen = set()
        eng.model.forward(batch, eng.cache)
        # 2. the description that stays; once launch by launch, on padding only
        c.desc = StepDescription(eng, Tp, S, S, width, pinned=True, qblock_sizes=sorted(batch.sizes_seen))
        self._all_padding(c.desc)
        eng.model.forward(c.desc.batch(max_len), eng.cache)
        torch.cuda.synchronize()
        K.check_status()
        # 3. the capture
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        g = torch.cuda.CUDAGraph()
        before = K.launch_count()
        with torch.cuda.graph(g, pool=self.pool):
            c.logits = eng.model.forward(c.desc.batch(max_len), eng.cache)
        c.kernels = K.launch_count() - before
        K.count_launches(-c.kernels)                  # captured, not run
        c.graph = g
        c.scratch_epoch = K.scratch_epoch()
        self.captures += 1
        return c

    def _get(self, key: Tuple[int, int, int]) -> _CapturedPrompt:
        c = self.graphs.get(key)
        if c is not None and c.scratch_epoch != K.scratch_epoch():
            del self.graphs[key]                      # a scratch buffer it recorded the address of was regrown
            c = None
        if c is None:
            while len(self.graphs) >= self.max_graphs:
                self.graphs.popitem(last=False)
            c = self._capture(key)
            if c.scratch_epoch != K.scratch_epoch():  # (the capture itself regrew one: its addresses are the new ones)
                c.scratch_epoch = K.scratch_epoch()
            self.graphs[key] = c
        else:
            self.graphs.move_to_end(key)
        return c

    def step(self, entries: Sequence[StepEntry], key: Optional[Tuple[int, int, int]] = None) -> torch.Tensor:
        """As Engine.step: float32 logits [wanted places, vocab] on the device (a view of the graph's own output,
        valid until this shape is stepped again).  On error nothing has changed."""
        eng = self.engine
        cache = eng.cache
        slots = [e.slot for e in entries]
        token_lists = [e.tokens for e in entries]
        wants = [e.want for e in entries]
        eng.validate(slots, token_lists, wants)
        key = key or self._shape(entries)
        if key is None:
            raise StepError("this step is not one that is replayed")
        n_new = [len(t) for t in token_lists]
        cache.reserve(slots, n_new)                   # raises CacheFull before anything is launched
        before = [cache.length(s) for s in slots]
        c = self._get(key)
        c.desc.write_prompts(slots, n_new, wants)
        c.desc.write_tokens(token_lists, before)
        c.desc.upload()
        c.graph.replay()
        K.count_launches(c.kernels)
        self.replays += 1
        eng.check_kernels()                           # synchronises; raises if a kernel gave up a wait
        cache.advance(slots, n_new)
        return c.logits[:sum(len(w) for w in wants)]
