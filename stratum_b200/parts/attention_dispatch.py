"""Which attention kernel serves a given step."""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS


def run(att, qkv: torch.Tensor, cache, step, out: torch.Tensor) -> None:
    K.attention_simple(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                       att.n_heads, att.n_kv_heads, att.head_dim, PAGE_TOKENS, att.window, att.scale)
