"""The cache: per-sequence slots, paged keys and values per layer group, fixed-size state.

Layers whose mixers ask for the same kind of storage form a group; each group
has storage and page bookkeeping of its own (a group that keeps every key, a
group that keeps a window of them, a group of fixed-size recurrent state).  The
reference classifies its layers the same way and sizes key/value rows or
convolution/recurrent state per class (stratum/native/stratum_arch.h:53-67,
:82-105); its Llama handler has one class, all keys
(stratum/native/stratum_arch_llama.inc.c:636-682).

Key/value storage of a group: K and V of shape
[layers in group, pages, kv heads, PAGE_TOKENS, head size], so the rows of one
(page, head) are contiguous.  State storage: [layers in group, slots, *shape].
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .pages import (PAGE_TOKENS, CacheFull, CacheMisuse, PagePool, SequencePages, SlotTable,
                    pages_for)


@dataclass(frozen=True)
class KVSpec:
    """Keys and values per token: `window` = 0 keeps all of them, W > 0 the last W.  `key_order` names the order
    in which a mixer keeps the dimensions of a key (mixers that share a cache must agree on it, so it is part of
    what makes two specs equal)."""
    n_kv_heads: int
    head_dim: int
    window: int = 0
    key_order: str = "as_projected"


@dataclass(frozen=True)
class StateSpec:
    """A fixed-size block per sequence, zeroed when a slot is taken.  dtype: "float32" or "compute"."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


CacheSpec = Union[KVSpec, StateSpec]


@dataclass
class LayerCache:
    """What one stop of the schedule sees of the cache during a step."""
    spec: Optional[CacheSpec]
    writes: bool                                  # False when reading another layer's cache
    k: Optional[torch.Tensor] = None              # [pages, kv heads, PAGE_TOKENS, head size]
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None    # int32 [sequences in step, pages per sequence]
    state: Optional[torch.Tensor] = None          # [slots, *shape]; rows indexed by StepBatch.seq_slot


class _Group:
    def __init__(self, spec: CacheSpec):
        self.spec = spec
        self.layers: List[int] = []
        self.pool: Optional[PagePool] = None
        self.k = self.v = self.state = None


class SequenceCache:
    """Slots, pages and storage for one model.

    layer_specs: for each stop of the schedule that owns a cache, its spec (None for stops without).
    max_tokens: tokens that live sequences may hold together, each sequence's count rounded
                up to a multiple of PAGE_TOKENS.
    max_seqs:   sequences that may be live at once.
    """

    def __init__(self, layer_specs: Sequence[Optional[CacheSpec]], max_tokens: int, max_seqs: int,
                 dtype: torch.dtype, device, allocate: bool = True):
        if max_tokens < 1 or max_seqs < 1:
            raise ValueError("cache needs max_tokens >= 1 and max_seqs >= 1")
        self.n_pages = pages_for(max_tokens)
        self.max_seqs = min(max_seqs, self.n_pages)
        self.dtype, self.device = dtype, device
        self.slots = SlotTable(self.max_seqs)
        self.groups: List[_Group] = []
        self.layer_group: Dict[int, Tuple[int, int]] = {}       # layer -> (group, index in group)
        by_spec: Dict[CacheSpec, int] = {}
        for li, spec in enumerate(layer_specs):
            if spec is None:
                continue
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                self.groups.append(_Group(spec))
            g = self.groups[by_spec[spec]]
            self.layer_group[li] = (by_spec[spec], len(g.layers))
            g.layers.append(li)
        for g in self.groups:
            if isinstance(g.spec, KVSpec):
                g.pool = PagePool(self.n_pages)
        self._seq: Dict[int, List[Optional[SequencePages]]] = {}
        self._len: Dict[int, int] = {}
        self.epoch = 0          # grows whenever a slot or a page changes hands: page tables copied earlier are stale
        if allocate:
            self._allocate()

    # ------------------------------------------------------------------ storage
    def _allocate(self) -> None:
        for g in self.groups:
            n = len(g.layers)
            if isinstance(g.spec, KVSpec):
                shape = (n, self.n_pages, g.spec.n_kv_heads, PAGE_TOKENS, g.spec.head_dim)
                g.k = torch.zeros(shape, dtype=self.dtype, device=self.device)
                g.v = torch.zeros(shape, dtype=self.dtype, device=self.device)
            else:
                dt = torch.float32 if g.spec.dtype == "float32" else self.dtype
                # one row more than there are slots: row `max_seqs` belongs to no sequence; the padding rows of a
                # step point there, so a mixer may update "their" state without harm to anyone's
                g.state = torch.zeros((n, self.max_seqs + 1) + tuple(g.spec.shape), dtype=dt, device=self.device)

    def storage_bytes(self) -> int:
        total = 0
        for g in self.groups:
            for t in (g.k, g.v, g.state):
                if t is not None:
                    total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ sequences
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self._seq[slot] = [SequencePages(g.pool, g.spec.window) if isinstance(g.spec, KVSpec) else None
                           for g in self.groups]
        for g in self.groups:
            if g.state is not None:
                g.state[:, slot].zero_()
        self._len[slot] = 0
        self.epoch += 1
        return slot

    def length(self, slot: int) -> int:
        self._need(slot)
        return self._len[slot]

    def _need(self, slot: int) -> None:
        if not self.slots.is_live(slot):
            raise CacheMisuse(f"slot {slot} is not held by a sequence")

    def reserve(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """Take the pages a step needs, for every sequence or for none."""
        if len(set(slots)) != len(slots):
            raise CacheMisuse("a slot appears twice in one step")
        for s in slots:
            self._need(s)
        for gi, g in enumerate(self.groups):
            if g.pool is None:
                continue
            need = sum(self._seq[s][gi].pages_needed(n) for s, n in zip(slots, n_new))
            if need > g.pool.free_pages:
                held = self.n_pages - g.pool.free_pages
                raise CacheFull(f"step needs {need} more pages of {PAGE_TOKENS} tokens; {held} of "
                                f"{self.n_pages} are held (capacity {self.n_pages * PAGE_TOKENS} tokens)")
        for gi, g in enumerate(self.groups):
            if g.pool is None:
                continue
            for s, n in zip(slots, n_new):
                sp = self._seq[s][gi]
                if sp.pages_needed(n):
                    sp.reserve(n)
                    self.epoch += 1

    def advance(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        for s, n in zip(slots, n_new):
            self._need(s)
            for sp in self._seq[s]:
                if sp is not None and sp.advance(n):
                    self.epoch += 1
            self._len[s] += n

    def release(self, slot: int) -> None:
        self._need(slot)
        for sp in self._seq.pop(slot):
            if sp is not None:
                sp.release()
        del self._len[slot]
        self.slots.release(slot)
        self.epoch += 1

    def release_all(self) -> None:
        for s in self.slots.live():
            self.release(s)

    def tokens_held(self) -> int:
        """Tokens' worth of pages held in the fullest group."""
        held = [self.n_pages - g.pool.free_pages for g in self.groups if g.pool is not None]
        return (max(held) if held else 0) * PAGE_TOKENS

    def check(self) -> None:
        """Bookkeeping invariants: nothing lost, held twice or freed twice."""
        self.slots.check()
        for gi, g in enumerate(self.groups):
            if g.pool is None:
                continue
            g.pool.check()
            seen = set()
            for s, per_group in self._seq.items():
                for p in per_group[gi].table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheMisuse(f"page {p} is held by two sequences")
                    seen.add(p)
            if len(seen) != self.n_pages - g.pool.free_pages:
                raise CacheMisuse("pages held by sequences and pages missing from the pool differ")
        if set(self._seq) != set(self.slots.live()):
            raise CacheMisuse("live slots and sequences with pages differ")

    # ------------------------------------------------------------------ views for a step
    def page_table_rows(self, slots: Sequence[int], group: int) -> List[List[int]]:
        return [self._seq[s][group].table for s in slots]

    def layer_view(self, layer: int, writes: bool, block_tables: Dict[int, torch.Tensor]) -> LayerCache:
        if layer not in self.layer_group:
            return LayerCache(spec=None, writes=False)
        gi, idx = self.layer_group[layer]
        g = self.groups[gi]
        if isinstance(g.spec, KVSpec):
            return LayerCache(spec=g.spec, writes=writes, k=g.k[idx], v=g.v[idx],
                              block_table=block_tables.get(gi))
        return LayerCache(spec=g.spec, writes=writes, state=g.state[idx])
