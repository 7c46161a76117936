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

A graph is specific to (rows, page-table width, greedy or sampling): rows is the batch padded up a little (padding
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
from .step import Engine, StepDescription, StepError


def padded_rows(n: int) -> int:
    """Rows a graph is captured for: exact up to 8, then the next multiple of 8."""
    return n if n <= 8 else ((n + 7) // 8) * 8


def width_bucket(n_pages: int) -> int:
    w = 1
    while w < n_pages:
        w *= 2
    return w


class _Captured:
    def __init__(self, engine: Engine, rows: int, width: int, greedy: bool):
        self.rows, self.width, self.greedy = rows, width, greedy
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
                     c.out_vals)
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

    def _get(self, rows: int, width: int, greedy: bool) -> _Captured:
        key = (rows, width, greedy)
        c = self.graphs.get(key)
        if c is not None and c.graph is not None and c.scratch_epoch != K.scratch_epoch():
            # a scratch buffer was regrown (and the old one freed) since this graph recorded its address
            del self.graphs[key]
            c = None
        if c is None:
            while len(self.graphs) >= self.max_graphs:
                self.graphs.popitem(last=False)
            c = _Captured(self.engine, rows, width, greedy)
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
        c = self._get(padded_rows(B), width_bucket(pages_for(max(before) + 1)), not (temperature > 0.0))
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
