"""The step function: run exactly the tokens given, as one batch, from the cache.

A step is a list of entries (slot, new tokens, wanted places).  A batch's first step
carries its prompts, of unequal lengths, in one go; later steps carry one token per live
sequence.  The tokens of all entries are packed into one row-major batch with, per token,
its sequence and its position (cached length + offset), so every kernel sees one flat batch
and padding does not exist.  The reference has the two halves separately: a chunk of one
sequence with `lm_mode` choosing where logits are made
(stratum/native/stratum_arch_llama.inc.c:785-1050) and lock-step streams with per-slot position
and length (:1070-1218); its capacity and vocabulary checks come before any work (:689-695,
stratum/native/stratum_engine.h:477-487), as here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.pages import PAGE_TOKENS, pages_for
from ..cache.store import KVSpec, SequenceCache
from .model import Model


class StepError(ValueError):
    """The step's entries are not acceptable (bad slot, token id, wanted place); nothing was run."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among `tokens` whose logits are asked for


@dataclass
class StepBatch:
    """Device-side description of one step, shared by every part."""
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor           # int32 [T]
    token_pos: torch.Tensor           # int32 [T] position of each token in its sequence
    token_seq: torch.Tensor           # int32 [T] index of its sequence within the step (-1 = padding)
    want_rows: torch.Tensor           # int32 [n_want] rows of the packed batch whose logits are wanted
    seq_slot: torch.Tensor            # int32 [B] cache slot of each sequence (rows of fixed-size state)
    seq_start: torch.Tensor           # int32 [B+1] first packed row of each sequence
    seq_len: torch.Tensor             # int32 [B] keys each sequence holds once this step's are appended
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # cache group -> int32 [B, pages]
    max_new: int = 1                  # longest run of new tokens of one sequence
    max_len: int = 1                  # longest sequence after this step
    all_single: bool = True           # every sequence brings exactly one token
    host: Optional[dict] = None       # the same numbers on the host, for parts that plan launches
    _qblocks: Dict[int, tuple] = field(default_factory=dict)

    def query_blocks(self, tokens_per_block: int):
        """Cut every sequence's new tokens into runs of at most `tokens_per_block`: int32 tensors
        (sequence, first packed row, tokens) on the device, made once per step and block size."""
        if tokens_per_block not in self._qblocks:
            seqs, rows, counts = [], [], []
            r = 0
            for i, n in enumerate(self.host["n_new"]):
                for b in range(0, n, tokens_per_block):
                    seqs.append(i); rows.append(r + b); counts.append(min(tokens_per_block, n - b))
                r += n
            dev = torch.from_numpy(np.asarray([seqs, rows, counts], dtype=np.int32)).to(self.token_ids.device)
            self._qblocks[tokens_per_block] = (dev[0], dev[1], dev[2])
        return self._qblocks[tokens_per_block]


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None):
        self.model = model
        self.runtime = model.runtime
        n_pages = pages_for(max_tokens)
        self.cache = SequenceCache(model.cache_specs(), max_tokens,
                                   max_seqs if max_seqs is not None else min(n_pages, 1024),
                                   self.runtime.dtype, self.runtime.device)
        self.vocab = model.vocab

    # ------------------------------------------------------------------ sequences
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.is_live(e.slot):
                raise StepError(f"slot {e.slot} is not held by a sequence")
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: a step entry needs at least one token")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab):
                    raise StepError(f"slot {e.slot}: token id {t} outside the vocabulary [0, {self.vocab})")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"slot {e.slot}: wanted place {w} outside its {len(e.tokens)} tokens")

    def build_batch(self, entries: Sequence[StepEntry]) -> StepBatch:
        """Pack the entries and copy their description to the device (one copy)."""
        B = len(entries)
        n_new = [len(e.tokens) for e in entries]
        T = sum(n_new)
        before = [self.cache.length(e.slot) for e in entries]
        n_want = sum(len(e.want) for e in entries)
        groups = [gi for gi, g in enumerate(self.cache.groups) if isinstance(g.spec, KVSpec)]
        max_len = max(b + n for b, n in zip(before, n_new))
        width = max(1, pages_for(max_len))
        # one int32 array: ids | pos | seq | want | slot | start | len | tables...
        total = 3 * T + n_want + B + (B + 1) + B + len(groups) * B * width
        buf = np.empty(total, dtype=np.int32)
        o = 0
        ids = buf[o:o + T]; o += T
        pos = buf[o:o + T]; o += T
        seq = buf[o:o + T]; o += T
        want = buf[o:o + n_want]; o += n_want
        slot = buf[o:o + B]; o += B
        start = buf[o:o + B + 1]; o += B + 1
        slen = buf[o:o + B]; o += B
        r = w = 0
        for i, e in enumerate(entries):
            n = n_new[i]
            ids[r:r + n] = np.asarray(e.tokens, dtype=np.int32)
            pos[r:r + n] = np.arange(before[i], before[i] + n, dtype=np.int32)
            seq[r:r + n] = i
            for p in e.want:
                want[w] = r + int(p); w += 1
            slot[i] = e.slot
            start[i] = r
            slen[i] = before[i] + n
            r += n
        start[B] = T
        tables = {}
        for gi in groups:
            tb = buf[o:o + B * width].reshape(B, width); o += B * width
            tb.fill(-1)
            for i, row in enumerate(self.cache.page_table_rows([e.slot for e in entries], gi)):
                tb[i, :len(row)] = row
            tables[gi] = tb
        dev = torch.from_numpy(buf).to(self.runtime.device)
        o = 0

        def take(n):
            nonlocal o
            t = dev[o:o + n]
            o += n
            return t

        d_ids, d_pos, d_seq = take(T), take(T), take(T)
        d_want, d_slot, d_start, d_len = take(n_want), take(B), take(B + 1), take(B)
        d_tables = {gi: take(B * width).view(B, width) for gi in groups}
        return StepBatch(n_tokens=T, n_seqs=B, token_ids=d_ids, token_pos=d_pos, token_seq=d_seq,
                         want_rows=d_want, seq_slot=d_slot, seq_start=d_start, seq_len=d_len,
                         block_tables=d_tables, max_new=max(n_new), max_len=max_len,
                         all_single=all(n == 1 for n in n_new),
                         host={"n_new": n_new, "before": before})

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; return float32 logits [wanted places, vocab] on the device,
        in the order of the entries and of each entry's `want`.  On error nothing has changed."""
        self._validate(entries)
        slots = [e.slot for e in entries]
        n_new = [len(e.tokens) for e in entries]
        self.cache.reserve(slots, n_new)          # raises CacheFull before anything is launched
        batch = self.build_batch(entries)
        logits = self.model.forward(batch, self.cache)
        self.cache.advance(slots, n_new)
        return logits
