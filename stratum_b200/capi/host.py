"""What the C interface forwards to: one function per exported symbol of stratum.h.

Arrays arrive as addresses of the caller's memory and are read and written in place; everything else is the
Python entry point's (`Stratum`): the same model, step function, cache and kernels.  Errors are raised; the C
layer turns them into a status code and a message.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List

import numpy as np

_open: Dict[int, object] = {}
_next = [1]


def _ints(address: int, n: int) -> List[int]:
    if n == 0:
        return []
    if not address:
        raise ValueError("a needed array is null")
    return np.ctypeslib.as_array(ctypes.cast(address, ctypes.POINTER(ctypes.c_int32)), shape=(n,)).tolist()


def _get(handle: int):
    try:
        return _open[handle]
    except KeyError:
        raise ValueError(f"context {handle} is not open") from None


def open_model(model_dir: str, dtype: str, max_tokens: int, max_seqs: int) -> int:
    from ..engine.api import Stratum
    llm = Stratum(model_dir, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs or None)
    handle = _next[0]
    _next[0] += 1
    _open[handle] = llm
    return handle


def close_model(handle: int) -> int:
    _open.pop(handle, None)
    return 0


def vocab(handle: int) -> int:
    return int(_get(handle).engine.vocab)


def slot_acquire(handle: int) -> int:
    return int(_get(handle).acquire())


def slot_release(handle: int, slot: int) -> int:
    _get(handle).release(slot)
    return 0


def slot_length(handle: int, slot: int) -> int:
    return int(_get(handle).engine.length(slot))


def step(handle: int, n_seq: int, slots: int, n_tok: int, tokens: int, n_want: int, want: int, logits: int) -> int:
    """Returns the number of logits rows written."""
    from ..engine.step import StepEntry
    llm = _get(handle)
    slot_list, counts, wants = _ints(slots, n_seq), _ints(n_tok, n_seq), _ints(n_want, n_seq)
    if any(c < 0 for c in counts) or any(w < 0 for w in wants):
        raise ValueError("a count is negative")
    toks, places = _ints(tokens, sum(counts)), _ints(want, sum(wants))
    entries, t, w = [], 0, 0
    for s, c, k in zip(slot_list, counts, wants):
        entries.append(StepEntry(s, toks[t:t + c], places[w:w + k]))
        t, w = t + c, w + k
    rows = sum(wants)
    if rows and not logits:
        raise ValueError("logits are wanted but the logits array is null")
    out = llm.step(entries)
    if rows:
        V = out.shape[1]
        dst = np.ctypeslib.as_array(ctypes.cast(logits, ctypes.POINTER(ctypes.c_float)), shape=(rows, V))
        dst[...] = out.cpu().numpy()
    return rows


def generate(handle: int, n_prompts: int, prompt_len: int, prompt_tokens: int, max_new: int, stop_ids: int,
             n_stop: int, temperature: float, top_k: int, top_p: float, seed: int, out_tokens: int,
             out_count: int) -> int:
    from ..sampling.params import SamplingParams
    llm = _get(handle)
    lens = _ints(prompt_len, n_prompts)
    if any(n < 1 for n in lens):
        raise ValueError("every prompt needs at least one token")
    flat = _ints(prompt_tokens, sum(lens))
    prompts, t = [], 0
    for n in lens:
        prompts.append(flat[t:t + n])
        t += n
    results = llm.generate(prompts, max_new_tokens=max_new, stop_ids=tuple(_ints(stop_ids, n_stop)),
                           sampling=SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed))
    counts = np.ctypeslib.as_array(ctypes.cast(out_count, ctypes.POINTER(ctypes.c_int32)), shape=(n_prompts,))
    if max_new > 0:
        ids = np.ctypeslib.as_array(ctypes.cast(out_tokens, ctypes.POINTER(ctypes.c_int32)), shape=(n_prompts, max_new))
        for i, r in enumerate(results):
            ids[i, :len(r.tokens)] = r.tokens
    counts[:] = [len(r.tokens) for r in results]
    return 0
