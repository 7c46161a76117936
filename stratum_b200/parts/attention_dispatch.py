"""Which attention kernel serves a given step.

float32, and head sizes the tensor-core kernel refuses (above 128, or no multiple of 16): the CUDA-core
kernel with the fixed key order.  bfloat16 decode steps: the TMA-fed kernel that spreads all pages evenly over
the SMs (head size 64 or 128, up to 8 heads per kv head), else the kernel whose keys are cut into splits per
sequence, which needs scratch for the partial results.  bfloat16 prompts: the tcgen05 kernel, else the tile kernel.
"""
from __future__ import annotations

import os

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS

# work items (warps) wanted in flight on decode steps: 148 SMs times the warps an SM holds of the decode kernel
TARGET_WARPS = int(os.environ.get("STRATUM_ATTENTION_WARPS", 148 * 8))


MAX_SPLITS = 256                # what the merge kernel takes


def plan_splits(n_items: int, max_len: int):
    """(n_splits, keys per split) for decode steps: enough splits to fill the GPU, whole pages per split."""
    pages = max(1, (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
    want = max(1, min(pages, MAX_SPLITS, (TARGET_WARPS + n_items - 1) // n_items))
    chunk = ((pages + want - 1) // want) * PAGE_TOKENS
    return (max_len + chunk - 1) // chunk, chunk


WHOLE_PAGES_MIN = 1184          # pages of all sequences and kv heads: eight to an SM of 148


def _stream_form() -> str:
    """STRATUM_ATTENTION_STREAM_FORM=0: never whole pages per warp (for measurements)."""
    return os.environ.get("STRATUM_ATTENTION_STREAM_FORM", "")


def run(att, qkv: torch.Tensor, cache, step, out: torch.Tensor) -> None:
    hd = att.head_dim
    if qkv.dtype != torch.bfloat16 or hd % 16 != 0 or hd > 128 or qkv.stride(0) % 8 != 0:
        K.attention_simple(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                           att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS, att.window, att.scale)
        return
    gs = att.n_heads // att.n_kv_heads
    rows_per_token = min(gs, 16)
    head_groups = (gs + 15) // 16
    if (step.all_single and hd in (64, 128) and gs <= 8 and step.n_tokens <= 1024
            and os.environ.get("STRATUM_ATTENTION_STREAM", "1") != "0"):
        # decode steps: the pages of all sequences spread evenly over the SMs, streamed by TMA.  With more than
        # two sequences the kernels after it get a head start while the last pages stream in (3 % of a step on
        # the Llama-8B shape at 8 sequences); with one or two it costs more than it gives (measured)
        # heads of 64: whole pages per warp where an SM gets more than a few pages (by the step's longest sequence;
        # measured: 93 against 119 us at 64 sequences of 4,096 tokens, 11.2 against 9.9 us at one)
        pages = step.n_tokens * att.n_kv_heads * ((step.max_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
        K.attention_stream(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                           att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS, att.window, att.scale,
                           late_trigger=step.n_tokens > 2,
                           whole_pages=hd == 64 and pages >= WHOLE_PAGES_MIN and _stream_form() != "0")
    elif step.all_single:
        n_splits, chunk = plan_splits(step.n_tokens * att.n_kv_heads * head_groups, step.max_len)
        part_o = part_ml = None
        if n_splits > 1:
            n = step.n_tokens * att.n_heads * n_splits
            part_o = att.runtime.scratch("attention_part_o", n * hd, torch.float32)
            part_ml = att.runtime.scratch("attention_part_ml", n * 2, torch.float32)
        K.attention_mma(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, None, 1, out,
                        part_o, part_ml, att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS, att.window, att.scale,
                        n_splits, chunk)
    elif hd in (64, 128) and 128 % gs == 0 and os.environ.get("STRATUM_ATTENTION_TC", "1") != "0":
        # prompts: the tcgen05 kernel; a CTA owns 256 query rows (2 x 128 / gs tokens) whose two halves share every
        # key and value tile (STRATUM_ATTENTION_HALVES=1: 128 rows per CTA, two CTAs per SM; measurements)
        halves = int(os.environ.get("STRATUM_ATTENTION_HALVES", "2"))
        K.attention_tc(qkv, cache.k, cache.v, step.token_pos, cache.block_table,
                       step.query_blocks(halves * (128 // gs)), out, att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS,
                       att.window, att.scale, halves)
    else:
        per_warp = 16 // rows_per_token
        K.attention_tile(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table,
                         step.query_blocks(4 * per_warp), per_warp, out, att.n_heads, att.n_kv_heads, hd,
                         PAGE_TOKENS, att.window, att.scale)
