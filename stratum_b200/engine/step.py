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
from .. import kernels as K
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
    fixed_qblocks: Optional[Dict[int, tuple]] = None   # a captured prompt step: its query blocks, padded lists
    sizes_seen: Optional[set] = None  # when set: the block sizes `query_blocks` was asked for are noted here
    _qblocks: Dict[int, tuple] = field(default_factory=dict)
    _rotation: Dict[object, torch.Tensor] = field(default_factory=dict)

    def rotation_table(self, rot) -> torch.Tensor:
        """(cos, sin) of every token's angles under a RotaryTable, float32 [tokens, pairs, 2] on the device: made
        by one small kernel the first time a layer of the step asks, and shared by all layers that rotate alike."""
        t = self._rotation.get(rot.key)
        if t is None:
            t = torch.empty((self.n_tokens, rot.inv_freq.numel(), 2), dtype=torch.float32, device=self.token_pos.device)
            K.rope_table(self.token_pos, rot.inv_freq, rot.magnitude, t)
            self._rotation[rot.key] = t
        return t

    def query_blocks(self, tokens_per_block: int):
        """Cut every sequence's new tokens into runs of at most `tokens_per_block`: int32 tensors
        (sequence, first packed row, tokens) on the device, made once per step and block size.  In a captured
        prompt step the lists have a fixed length; entries beyond the step's blocks have sequence -1 and no tokens."""
        if self.fixed_qblocks is not None:
            if tokens_per_block not in self.fixed_qblocks:
                raise StepError(f"this captured step was described without query blocks of {tokens_per_block} tokens")
            return self.fixed_qblocks[tokens_per_block]
        if self.sizes_seen is not None:
            self.sizes_seen.add(tokens_per_block)
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


class StepDescription:
    """A step's description as one int32 buffer on the host and its copy on the device.

    Both ways of running a step use this one builder: `Engine.step` makes a description of exactly the
    step's size, a captured decode graph keeps one of a fixed size (rows padded, page tables of a fixed width)
    and rewrites it before every replay.  A field that a new part needs is added here once.

    Fields, in order: ids | pos | seq | want | slot | start | len | one page table per key/value group | extras.
    Rows beyond the real tokens are padding: each is a sequence of its own with sequence index -1 (every kernel
    that touches the cache skips it), position 0, length 0, an empty page table, and the slot number `max_seqs`,
    which is a row of fixed-size state that belongs to no sequence.
    """

    def __init__(self, engine: "Engine", n_tokens: int, n_seqs: int, n_want: int, width: int,
                 extras: Sequence = (), pinned: bool = False, qblock_sizes: Sequence[int] = ()):
        self.engine = engine
        self.n_tokens, self.n_seqs, self.n_want, self.width = n_tokens, n_seqs, n_want, width
        self.groups = engine.kv_groups
        self.off: Dict[str, tuple] = {}
        # query blocks of each size a captured prompt step asks for: at most tokens / size + sequences of them
        self.qblock_sizes = tuple(sorted(qblock_sizes))
        self.qblock_max = {n: n_tokens // n + n_seqs for n in self.qblock_sizes}
        extras = tuple(extras) + tuple((f"qb{n}", 3 * self.qblock_max[n]) for n in self.qblock_sizes)
        o = 0
        for name, n in (("ids", n_tokens), ("pos", n_tokens), ("seq", n_tokens), ("want", n_want),
                        ("slot", n_seqs), ("start", n_seqs + 1), ("len", n_seqs),
                        ("tables", len(self.groups) * n_seqs * width)) + tuple(extras):
            self.off[name] = (o, n)
            o += n
        self.total = o
        self.host = torch.empty(o, dtype=torch.int32)
        if pinned:
            self.host = self.host.pin_memory()
        self.np = self.host.numpy()
        self.dev: Optional[torch.Tensor] = None
        self.views = {name: self.np[a:a + n] for name, (a, n) in self.off.items()}
        self.n_new: List[int] = []
        self.single = True
        self.before: Optional[List[int]] = None

    def write_membership(self, slots: Sequence[int], n_new: Sequence[int], wants: Optional[Sequence[Sequence[int]]]):
        """Who is in the step, with how many tokens each, whose logits are wanted and which pages they hold:
        what stays the same from one decode step to the next until a sequence leaves or a page is taken.
        wants None: every row's logits (the rows of a decode step)."""
        v = self.views
        B, T = len(slots), sum(n_new)
        pad = self.n_tokens - T
        if B + pad != self.n_seqs:
            raise StepError(f"step description for {self.n_seqs} sequences given {B} and {pad} padding rows")
        cache = self.engine.cache
        seq, start, slot = v["seq"], v["start"], v["slot"]
        if all(n == 1 for n in n_new):
            seq[:B] = np.arange(B, dtype=np.int32)
            start[:B + 1] = np.arange(B + 1, dtype=np.int32)
        else:
            r = 0
            for i, n in enumerate(n_new):
                seq[r:r + n] = i
                start[i] = r
                r += n
            start[B] = T
        seq[T:] = -1
        start[B:] = np.arange(T, T + pad + 1, dtype=np.int32)
        slot[:B] = slots
        slot[B:] = cache.max_seqs
        if wants is None:
            v["want"][:] = np.arange(self.n_want, dtype=np.int32)
        else:
            w = 0
            for i, ws in enumerate(wants):
                for p in ws:
                    v["want"][w] = start[i] + int(p)
                    w += 1
        if self.groups:
            tb = v["tables"].reshape(len(self.groups), self.n_seqs, self.width)
            tb.fill(-1)
            for j, gi in enumerate(self.groups):
                for i, row in enumerate(cache.page_table_rows(slots, gi)):
                    tb[j, i, :len(row)] = row
        self.n_new = list(n_new) + [1] * pad
        self.single = all(n == 1 for n in n_new)

    def write_prompts(self, slots: Sequence[int], n_new: Sequence[int], wants: Sequence[Sequence[int]]) -> None:
        """Like write_membership, for a description larger than the step in tokens, sequences and wanted rows,
        each by itself (a captured prompt step): tokens beyond the step's have sequence index -1 and belong to no
        sequence; sequences beyond the step's bring no token, hold nothing and have the spare state row; wanted
        rows beyond the step's point at row 0 (their logits are computed and not looked at)."""
        v = self.views
        B, T = len(slots), sum(n_new)
        n_want = sum(len(w) for w in wants)
        if B > self.n_seqs or T > self.n_tokens or n_want > self.n_want:
            raise StepError(f"step of {T} tokens, {B} sequences, {n_want} wanted rows in a description for "
                            f"{self.n_tokens}, {self.n_seqs}, {self.n_want}")
        cache = self.engine.cache
        seq, start, slot = v["seq"], v["start"], v["slot"]
        r = 0
        for i, n in enumerate(n_new):
            seq[r:r + n] = i
            start[i] = r
            r += n
        seq[T:] = -1
        start[B:] = T
        slot[:B] = slots
        slot[B:] = cache.max_seqs
        w = 0
        for i, ws in enumerate(wants):
            for p in ws:
                v["want"][w] = start[i] + int(p)
                w += 1
        v["want"][w:] = 0
        if self.groups:
            tb = v["tables"].reshape(len(self.groups), self.n_seqs, self.width)
            tb.fill(-1)
            for j, gi in enumerate(self.groups):
                for i, row in enumerate(cache.page_table_rows(slots, gi)):
                    tb[j, i, :len(row)] = row
        for size in self.qblock_sizes:
            m = self.qblock_max[size]
            qb = v[f"qb{size}"].reshape(3, m)
            k, r = 0, 0
            for i, n in enumerate(n_new):
                for b in range(0, n, size):
                    qb[0, k], qb[1, k], qb[2, k] = i, r + b, min(size, n - b)
                    k += 1
                r += n
            qb[0, k:] = -1
            qb[1, k:] = 0
            qb[2, k:] = 0
        self.n_new = list(n_new) + [0] * (self.n_seqs - B)
        self.single = False

    def write_tokens(self, token_lists: Sequence[Sequence[int]], before: Sequence[int]) -> None:
        """The tokens themselves, their positions, and each sequence's length once they are appended."""
        v = self.views
        B = len(before)
        ids, pos, slen = v["ids"], v["pos"], v["len"]
        T = 0
        if self.single:
            ids[:B] = [t[0] for t in token_lists]
            pos[:B] = before
            slen[:B] = pos[:B] + 1
            T = B
        else:
            for i, toks in enumerate(token_lists):
                n = len(toks)
                ids[T:T + n] = np.asarray(toks, dtype=np.int32)
                pos[T:T + n] = np.arange(before[i], before[i] + n, dtype=np.int32)
                slen[i] = before[i] + n
                T += n
        ids[T:] = 0
        pos[T:] = 0
        slen[B:] = 0
        self.before = list(before)

    def upload(self) -> None:
        dev = self.engine.runtime.device
        if self.dev is None:
            self.dev = torch.empty(self.total, dtype=torch.int32, device=dev)
        self.dev.copy_(self.host, non_blocking=True)

    def field(self, name: str) -> torch.Tensor:
        a, n = self.off[name]
        return self.dev[a:a + n]

    def batch(self, max_len: int) -> StepBatch:
        """The device copy's fields as a StepBatch (views; the buffer may be rewritten and uploaded again)."""
        R, W = self.n_seqs, self.width
        a, _ = self.off["tables"]
        tables = {gi: self.dev[a + j * R * W: a + (j + 1) * R * W].view(R, W) for j, gi in enumerate(self.groups)}
        fixed = None
        if self.qblock_sizes:
            fixed = {}
            for n in self.qblock_sizes:
                m, f = self.qblock_max[n], self.field(f"qb{n}")
                fixed[n] = (f[:m], f[m:2 * m], f[2 * m:3 * m])
        return StepBatch(n_tokens=self.n_tokens, n_seqs=R, token_ids=self.field("ids"), token_pos=self.field("pos"),
                         token_seq=self.field("seq"), want_rows=self.field("want"), seq_slot=self.field("slot"),
                         seq_start=self.field("start"), seq_len=self.field("len"), block_tables=tables,
                         max_new=max(self.n_new, default=0), max_len=max_len, all_single=self.single,
                         host={"n_new": list(self.n_new), "before": self.before}, fixed_qblocks=fixed)


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None):
        self.model = model
        self.runtime = model.runtime
        n_pages = pages_for(max_tokens)
        self.cache = SequenceCache(model.cache_specs(), max_tokens,
                                   max_seqs if max_seqs is not None else min(n_pages, 1024),
                                   self.runtime.dtype, self.runtime.device)
        self.kv_groups = [gi for gi, g in enumerate(self.cache.groups) if isinstance(g.spec, KVSpec)]
        self.vocab = model.vocab

    # ------------------------------------------------------------------ sequences
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ the step
    def validate(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
                 wants: Optional[Sequence[Sequence[int]]] = None, trusted_tokens: bool = False) -> None:
        """Refuse a step before anything runs.  trusted_tokens: the ids were picked by this engine itself."""
        if not slots:
            raise StepError("a step needs at least one entry")
        if len(set(slots)) != len(slots):
            dup = next(s for i, s in enumerate(slots) if s in slots[:i])
            raise StepError(f"slot {dup} appears twice in one step")
        for i, (s, toks) in enumerate(zip(slots, token_lists)):
            if not self.cache.slots.is_live(s):
                raise StepError(f"slot {s} is not held by a sequence")
            if len(toks) == 0:
                raise StepError(f"slot {s}: a step entry needs at least one token")
            if not trusted_tokens:
                for t in toks:
                    if not (0 <= int(t) < self.vocab):
                        raise StepError(f"slot {s}: token id {t} outside the vocabulary [0, {self.vocab})")
            if wants is not None:
                for w in wants[i]:
                    if not (0 <= int(w) < len(toks)):
                        raise StepError(f"slot {s}: wanted place {w} outside its {len(toks)} tokens")

    def build_batch(self, entries: Sequence[StepEntry]) -> StepBatch:
        """Pack the entries and copy their description to the device (one copy)."""
        slots = [e.slot for e in entries]
        n_new = [len(e.tokens) for e in entries]
        before = [self.cache.length(s) for s in slots]
        max_len = max(b + n for b, n in zip(before, n_new))
        d = StepDescription(self, sum(n_new), len(entries), sum(len(e.want) for e in entries),
                            max(1, pages_for(max_len)))
        d.write_membership(slots, n_new, [e.want for e in entries])
        d.write_tokens([e.tokens for e in entries], before)
        d.upload()
        return d.batch(max_len)

    def check_kernels(self) -> None:
        """Raise if a kernel gave up a bounded wait since the last check (synchronises)."""
        K.check_status()

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; return float32 logits [wanted places, vocab] on the device,
        in the order of the entries and of each entry's `want`.  On error nothing has changed:
        a refused step launches nothing, and a step in which a kernel gave up a wait leaves
        every sequence at the length it had."""
        slots = [e.slot for e in entries]
        self.validate(slots, [e.tokens for e in entries], [e.want for e in entries])
        n_new = [len(e.tokens) for e in entries]
        self.cache.reserve(slots, n_new)          # raises CacheFull before anything is launched
        batch = self.build_batch(entries)
        logits = self.model.forward(batch, self.cache)
        self.check_kernels()
        self.cache.advance(slots, n_new)
        return logits
