"""Decode steps as replayed CUDA graphs.

A decode step is some three hundred small launches; issued one by one from Python they cost more
host time than the GPU needs to run them.  So the whole step (embedding, every layer, final norm,
head, token pick) is captured once per shape into a CUDA graph and replayed: per step the host
fills one pinned buffer with the step's description (token ids, positions, page tables, sampling
numbers), copies it to the device in one go, replays, and reads the picked ids back.

A graph is specific to (rows, page-table width, greedy or sampling): rows is the batch padded up a little (padding
rows carry sequence index -1, which every kernel that touches the cache skips; rows never mix, so
padding changes no result), and the width is the next power of two of the pages the longest
sequence holds, which also fixes how the keys are split across warps.  The reference queues its
decode steps on the GPU ahead of time for the same reason
(stratum/native/stratum_arch_llama.inc.c:1994-2038).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS, pages_for
from ..cache.store import KVSpec
from .step import Engine, StepBatch, StepError


def padded_rows(n: int) -> int:
    """Rows a graph is captured for: exact up to 8, then the next multiple of 8."""
    return n if n <= 8 else ((n + 7) // 8) * 8


def width_bucket(n_pages: int) -> int:
    w = 1
    while w < n_pages:
        w *= 2
    return w


class _Captured:
    def __init__(self, rows: int, width: int, n_groups: int, device, greedy: bool):
        self.rows, self.width, self.greedy = rows, width, greedy
        B = rows
        # int32 words: ids | pos | seq | want | slot | start | len | tables | temperature | top_k | top_p | uniform
        self.off = {}
        o = 0
        for name, n in (("ids", B), ("pos", B), ("seq", B), ("want", B), ("slot", B), ("start", B + 1), ("len", B),
                        ("tables", n_groups * B * width), ("temperature", B), ("top_k", B), ("top_p", B),
                        ("uniform", B)):
            self.off[name] = (o, n)
            o += n
        self.total = o
        self.host = torch.empty(o, dtype=torch.int32).pin_memory()
        self.np = self.host.numpy()
        self.dev = torch.zeros(o, dtype=torch.int32, device=device)
        self.out_ids = torch.zeros(B, dtype=torch.int32, device=device)
        self.out_vals = torch.zeros(B, dtype=torch.float32, device=device)
        self.out_host = torch.empty(2 * B, dtype=torch.int32).pin_memory()
        self.views = {name: self.np[o:o + n] for name, (o, n) in self.off.items()}
        self.signature = None                         # (slots, pages per sequence) the host buffer was last filled for
        self.sampling = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels = 0
        self.logits: Optional[torch.Tensor] = None

    def view(self, name: str, dev: bool):
        o, n = self.off[name]
        return (self.dev if dev else self.np)[o:o + n]


class DecodeGraphs:
    """Runs one-token-per-sequence steps of an Engine through captured graphs."""

    def __init__(self, engine: Engine, max_graphs: int = 16):
        self.engine = engine
        self.max_graphs = max_graphs
        self.graphs: "OrderedDict[Tuple[int, int, bool], _Captured]" = OrderedDict()
        self.groups = [gi for gi, g in enumerate(engine.cache.groups) if isinstance(g.spec, KVSpec)]
        self.pool = None
        self.done = torch.cuda.Event()
        self.captures = 0
        self.h2d_bytes = self.d2h_bytes = 0           # of the last step

    # ------------------------------------------------------------------ building blocks
    def _batch(self, c: _Captured) -> StepBatch:
        B, W = c.rows, c.width
        tables = {}
        o, _ = c.off["tables"]
        for j, gi in enumerate(self.groups):
            tables[gi] = c.dev[o + j * B * W: o + (j + 1) * B * W].view(B, W)
        return StepBatch(n_tokens=B, n_seqs=B, token_ids=c.view("ids", True), token_pos=c.view("pos", True),
                         token_seq=c.view("seq", True), want_rows=c.view("want", True),
                         seq_slot=c.view("slot", True), seq_start=c.view("start", True), seq_len=c.view("len", True),
                         block_tables=tables, max_new=1, max_len=W * PAGE_TOKENS, all_single=True,
                         host={"n_new": [1] * B, "before": None})

    def _forward_and_pick(self, c: _Captured) -> None:
        logits = self.engine.model.forward(self._batch(c), self.engine.cache)
        if c.greedy:
            K.argmax(logits, c.out_ids, c.out_vals)
        else:
            K.sample(logits, c.view("temperature", True).view(torch.float32), c.view("top_k", True),
                     c.view("top_p", True).view(torch.float32), c.view("uniform", True).view(torch.float32),
                     c.out_ids, c.out_vals)
        c.logits = logits

    def _capture(self, c: _Captured) -> None:
        self._forward_and_pick(c)                     # once for real: compiles, sizes scratch, warms up
        torch.cuda.synchronize()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        g = torch.cuda.CUDAGraph()
        before = K.launch_count()
        with torch.cuda.graph(g, pool=self.pool):
            self._forward_and_pick(c)
        c.kernels = K.launch_count() - before
        K.count_launches(-c.kernels)                  # captured, not run
        c.graph = g
        self.captures += 1

    def _get(self, rows: int, width: int, greedy: bool) -> _Captured:
        key = (rows, width, greedy)
        c = self.graphs.get(key)
        if c is None:
            while len(self.graphs) >= self.max_graphs:
                self.graphs.popitem(last=False)
            c = _Captured(rows, width, len(self.groups), self.engine.runtime.device, greedy)
            self.graphs[key] = c
        else:
            self.graphs.move_to_end(key)
        return c

    # ------------------------------------------------------------------ one step
    def step(self, slots: Sequence[int], tokens: Sequence[int], temperature: float, top_k: int, top_p: float,
             uniforms: Optional[Sequence[float]], trusted: bool = False) -> Tuple[List[int], List[float], _Captured]:
        """One token for each slot; returns the picked ids and their logits (host lists).
        trusted: the tokens are ids this engine picked itself (no range check needed)."""
        eng = self.engine
        cache = eng.cache
        B = len(slots)
        if B == 0:
            raise StepError("a step needs at least one entry")
        if not trusted:
            if len(set(slots)) != B:
                raise StepError("a slot appears twice in one step")
            for s, t in zip(slots, tokens):
                if not cache.slots.is_live(s):
                    raise StepError(f"slot {s} is not held by a sequence")
                if not (0 <= int(t) < eng.vocab):
                    raise StepError(f"slot {s}: token id {t} outside the vocabulary [0, {eng.vocab})")
        cache.reserve(slots, _ONES[:B] if B <= len(_ONES) else [1] * B)
        before = [cache.length(s) for s in slots]
        c = self._get(padded_rows(B), width_bucket(pages_for(max(before) + 1)), not (temperature > 0.0))
        R, W = c.rows, c.width
        v = c.views
        # what a sequence holds changes every step; who is in the batch and which pages they own only now and then
        signature = (tuple(slots), tuple(len(r) for gi in self.groups for r in cache.page_table_rows(slots, gi)))
        if signature != c.signature:
            c.signature = signature
            v["ids"][:] = 0
            v["pos"][:] = 0
            v["seq"][:] = -1; v["seq"][:B] = np.arange(B, dtype=np.int32)
            v["want"][:] = np.arange(R, dtype=np.int32)
            v["slot"][:] = 0; v["slot"][:B] = slots
            v["start"][:] = np.arange(R + 1, dtype=np.int32)
            v["len"][:] = 0
            tb = v["tables"].reshape(len(self.groups), R, W)
            tb.fill(-1)
            for j, gi in enumerate(self.groups):
                for i, row in enumerate(cache.page_table_rows(slots, gi)):
                    tb[j, i, :len(row)] = row
            v["top_k"][:] = top_k
            v["temperature"].view(np.float32)[:] = temperature
            v["top_p"].view(np.float32)[:] = top_p
            v["uniform"].view(np.float32)[:] = 0.0
            c.sampling = (temperature, top_k, top_p)
        elif c.sampling != (temperature, top_k, top_p):
            v["top_k"][:] = top_k
            v["temperature"].view(np.float32)[:] = temperature
            v["top_p"].view(np.float32)[:] = top_p
            c.sampling = (temperature, top_k, top_p)
        v["ids"][:B] = tokens
        v["pos"][:B] = before
        v["len"][:B] = v["pos"][:B] + 1
        if uniforms is not None:
            v["uniform"].view(np.float32)[:B] = uniforms
        c.dev.copy_(c.host, non_blocking=True)
        if c.graph is None:
            self._capture(c)
        c.graph.replay()
        K.count_launches(c.kernels)
        c.out_host[:R].copy_(c.out_ids, non_blocking=True)
        c.out_host[R:].copy_(c.out_vals.view(torch.int32), non_blocking=True)
        self.done.record()
        self.done.synchronize()
        cache.advance(slots, _ONES[:B] if B <= len(_ONES) else [1] * B)
        self.h2d_bytes, self.d2h_bytes = c.total * 4, 2 * R * 4
        out = c.out_host.numpy()
        return out[:B].tolist(), out[R:R + B].view(np.float32).tolist(), c


_ONES = [1] * 1024
