"""Trace replay: feed given token ids through the step function and keep the logits.

Nothing is sampled here and nothing is computed here: steps are lists of (request, next tokens, wanted
places) that `play_step` hands to `Engine.step`, the step function generation uses.  Three ways of cutting
the same requests into steps are planned by `plan_steps`, so that their logits can be compared:

  mode 1  each request alone and whole: one step, every position's logits;
  mode 2  each request alone: all but its last tokens in one step, then its last `tail` tokens one by one;
  mode 3  batches of requests of unequal lengths: the first parts of all of a batch's requests in one step,
          then one token per live request per step; requests have unequal numbers of single-token steps, so
          the shorter ones end earlier; one batch after another, as many requests per batch as the cache
          holds, so that slots and pages given back are used again.

Every mode asks for the logits of every position of every request, so the records of two runs pair up by
(request, position).  Records go to a file of the form

    magic "SB2LOG01" | u32 vocab | repeat { u32 request | u32 position | f32[vocab] }        (little-endian)

which is the reference's logits dump with a request and a position per record instead of a token
(stratum/native/stratum_engine.h:489-525: "SLOG0001" | u32 n_vocab | repeat { u32 token; f32[n_vocab] }).
`compare_records` gives what the reference's compare tool prints for two such files: KL(base || other),
max |difference| and whether the best ids agree, per record and in summary
(stratum/native/tools_logit_compare.c:59-139); the reference checks its lock-step streams against the
serial path in the same spirit (stratum/native/stratum_arch_llama.inc.c:1505-1514).
"""
from __future__ import annotations

import json
import struct
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

MAGIC = b"SB2LOG01"
DEFAULT_TAIL = 32


# ---------------------------------------------------------------------------------------------- planning
def read_requests(path: str) -> List[Tuple[str, List[int]]]:
    """One JSON object per line: {"id": "a", "tokens": [5, 17, 3]}."""
    out = []
    with open(path) as f:
        for n, line in enumerate(f):
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            toks = [int(t) for t in rec["tokens"]]
            if not toks:
                raise ValueError(f"{path}:{n + 1}: request {rec.get('id')!r} has no tokens")
            out.append((str(rec["id"]), toks))
    if len({i for i, _ in out}) != len(out):
        raise ValueError(f"{path}: request ids are not unique")
    return out


def tail_of(index: int, length: int, tail: int, unequal: bool) -> int:
    """How many of a request's last tokens go one by one.  unequal: a different count for neighbouring
    requests (between 1 and `tail`), so that the requests of a batch end at different steps."""
    want = 1 + (7 * index + 3) % tail if unequal else tail
    return max(0, min(want, length - 1))


def plan_steps(requests: Sequence[Tuple[str, Sequence[int]]], mode: int, max_tokens: int,
               tail: int = DEFAULT_TAIL) -> List[dict]:
    """The steps of one mode, in the form the replay program reads: {"step", "entries": [{"id", "tokens",
    "want"}], "end"}.  Every position of every request is wanted exactly once.  max_tokens: what live
    requests may hold together, each rounded up to a page; mode 3 sizes its batches by it."""
    from .cache.pages import PAGE_TOKENS, pages_for        # (imported here: comparing records needs no torch)
    if mode not in (1, 2, 3):
        raise ValueError("mode must be 1 (whole), 2 (last tokens one by one) or 3 (unequal batches)")
    if tail < 1:
        raise ValueError("tail must be at least 1")
    n_pages = pages_for(max_tokens)
    for rid, toks in requests:
        if pages_for(len(toks)) > n_pages:
            raise ValueError(f"request {rid!r}: {len(toks)} tokens do not fit {n_pages * PAGE_TOKENS}")
    steps: List[dict] = []

    def add(entries, end):
        steps.append({"step": len(steps), "entries": entries, "end": end})

    if mode == 1:
        for rid, toks in requests:
            add([{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}], [rid])
        return steps
    if mode == 2:
        for i, (rid, toks) in enumerate(requests):
            k = tail_of(i, len(toks), tail, unequal=False)
            head = len(toks) - k
            add([{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}], [rid] if k == 0 else [])
            for j in range(head, len(toks)):
                add([{"id": rid, "tokens": [toks[j]], "want": [0]}], [rid] if j == len(toks) - 1 else [])
        return steps
    # mode 3: as many requests per batch, in order, as the pages hold
    batches: List[List[int]] = []
    cur, used = [], 0
    for i, (_, toks) in enumerate(requests):
        need = pages_for(len(toks))
        if cur and used + need > n_pages:
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    for batch in batches:
        tails = {i: tail_of(i, len(requests[i][1]), tail, unequal=True) for i in batch}
        heads = {i: len(requests[i][1]) - tails[i] for i in batch}
        add([{"id": requests[i][0], "tokens": list(requests[i][1][:heads[i]]), "want": list(range(heads[i]))}
             for i in batch], [requests[i][0] for i in batch if tails[i] == 0])
        live = [i for i in batch if tails[i] > 0]
        k = 0
        while live:
            ending = [i for i in live if k == tails[i] - 1]
            add([{"id": requests[i][0], "tokens": [requests[i][1][heads[i] + k]], "want": [0]} for i in live],
                [requests[i][0] for i in ending])
            live = [i for i in live if i not in ending]
            k += 1
    return steps


# ---------------------------------------------------------------------------------------------- playing
class Player:
    """Plays steps on an Engine: requests get slots at their first step and give them back when a step's
    `end` names them.  `sink(request id, position, float32 logits row)` receives every wanted row."""

    def __init__(self, engine, sink: Optional[Callable[[str, int, np.ndarray], None]] = None):
        self.engine = engine
        self.sink = sink
        self.slots: Dict[str, int] = {}

    def play_step(self, rec: dict) -> Optional[np.ndarray]:
        """Run one step; returns the wanted logits [wanted, vocab] as float32 on the host (None if none)."""
        from .engine.step import StepEntry
        entries, who = [], []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in self.slots:
                self.slots[rid] = self.engine.acquire()
            slot = self.slots[rid]
            entries.append(StepEntry(slot, e["tokens"], e.get("want", [])))
            who.append((rid, self.engine.length(slot), e.get("want", [])))
        out = None
        if entries:
            logits = self.engine.step(entries)
            if logits.shape[0] > 0:
                out = logits.cpu().numpy().astype("<f4", copy=False)
                if self.sink is not None:
                    row = 0
                    for rid, before, want in who:
                        for w in want:
                            self.sink(rid, before + int(w), out[row])
                            row += 1
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.engine.release(self.slots.pop(rid))
        return out


# ---------------------------------------------------------------------------------------------- records
class RecordWriter:
    def __init__(self, path: str, vocab: int):
        self.vocab = vocab
        self.f = open(path, "wb")
        self.f.write(MAGIC + struct.pack("<I", vocab))

    def write(self, request: int, position: int, logits: np.ndarray) -> None:
        row = np.ascontiguousarray(logits, dtype="<f4")
        if row.shape != (self.vocab,):
            raise ValueError(f"record of {row.shape} values in a file of vocabulary {self.vocab}")
        self.f.write(struct.pack("<II", request, position))
        self.f.write(row.tobytes())

    def close(self) -> None:
        self.f.close()


def read_records(path: str) -> Tuple[int, Dict[Tuple[int, int], np.ndarray]]:
    """(vocab, {(request, position): float32 logits}); a malformed file is an error, never a guess."""
    with open(path, "rb") as f:
        blob = f.read()
    if len(blob) < 12 or blob[:8] != MAGIC:
        raise ValueError(f"{path}: not a logits record file (bad magic)")
    (vocab,) = struct.unpack("<I", blob[8:12])
    if vocab == 0 or vocab > (1 << 26):
        raise ValueError(f"{path}: bad vocabulary size {vocab}")
    size = 8 + 4 * vocab
    body = len(blob) - 12
    if body % size:
        raise ValueError(f"{path}: truncated record ({body} bytes are no multiple of {size})")
    out: Dict[Tuple[int, int], np.ndarray] = {}
    for i in range(body // size):
        o = 12 + i * size
        req, pos = struct.unpack("<II", blob[o:o + 8])
        if (req, pos) in out:
            raise ValueError(f"{path}: request {req} position {pos} recorded twice")
        out[req, pos] = np.frombuffer(blob, dtype="<f4", count=vocab, offset=o + 8)
    return vocab, out


# ---------------------------------------------------------------------------------------------- comparing
def _log_softmax(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float64)
    m = x.max()
    return x - (m + np.log(np.exp(x - m).sum()))


def compare_records(base: Dict[Tuple[int, int], np.ndarray], other: Dict[Tuple[int, int], np.ndarray]):
    """Per (request, position) present in both: (KL(base || other), max |difference|, best ids agree, same bits);
    and a summary dict.  Keys present in only one of the two are counted in the summary."""
    rows = []
    keys = sorted(set(base) & set(other))
    for key in keys:
        b, o = base[key], other[key]
        lb, lo = _log_softmax(b), _log_softmax(o)
        p = np.exp(lb)
        kl = float(np.sum(np.where(p > 1e-300, p * (lb - lo), 0.0)))
        maxd = float(np.max(np.abs(b.astype(np.float64) - o.astype(np.float64))))
        rows.append((key, kl, maxd, int(np.argmax(b)) == int(np.argmax(o)), bool(np.array_equal(b, o))))
    n = len(rows)
    summary = {"records": n, "only_in_base": len(set(base) - set(other)), "only_in_other": len(set(other) - set(base)),
               "mean_kl": float(np.mean([r[1] for r in rows])) if n else 0.0,
               "max_kl": max((r[1] for r in rows), default=0.0),
               "max_abs_diff": max((r[2] for r in rows), default=0.0),
               "top1_agree": sum(r[3] for r in rows), "identical": sum(r[4] for r in rows),
               "max_abs_logit": max((float(np.max(np.abs(base[k]))) for k in keys), default=0.0)}
    return rows, summary
