"""Grouped-query attention over the paged cache.

q = Wq xn, k = Wk xn, v = Wv xn (+ biases); optionally normalise every head of q and of k
(stratum/native/stratum_arch_llama.inc.c:403-420, :866-884: tensors found by name, skipped when
absent); rotate q and k; append k and v to the cache at the
token's position; score_t = (q_h . K_t[kv(h)]) * scale for the keys the token may see; softmax;
o_h = sum_t p_t V_t[kv(h)]; residual += Wo o.  kv(h) = h / (n_heads / n_kv_heads).
(stratum/native/stratum_arch_llama.inc.c:398-524.)  The three projections run as one matrix
product over a weight made by stacking their rows (the reference fuses them at dispatch time,
stratum/native/stratum_linear.h:1086-1121).

Where the position encoding rotates pairs (k, k + n_pairs), the rows of Wq and Wk (and their biases, and the
gains of the per-head norms) are reordered once, when the weights are bound, so that a pair's two dimensions
are neighbours (2k, 2k+1): q . k is the same sum in another order, the rotation touches neighbours only, and a
matrix product's epilogue can rotate what one thread (or two neighbouring lanes) holds.  The reference's
converter does the same to its Llama files, which is why its handler rotates neighbours
(stratum/native/stratum_arch_llama.inc.c:82-87).  Keys therefore lie in the cache in that order.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS
from ..cache.store import KVSpec, LayerCache
from .base import Mixer, NormedRows
from .linear import ADD_TO_F32, QKV_ROPE, STORE, Linear
from .registry import find_part, register_part
from .spec import PartSpec, TensorSpec


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, bias, window (0 = all keys), scale (None =
    1/sqrt(head_dim)), position (PartSpec of a position encoding, or None), q_norm / k_norm (PartSpec of a
    norm of size head_dim applied to every query / key head between projection and rotation, or None), prefix."""
    takes_normed_rows = True
    hands_on = True

    @property
    def replays_prompts(self) -> bool:
        """(as far as the parts inside it do: the position encoding and the norms of the heads)"""
        inner = [p for p in (self.position, self.q_norm, self.k_norm) if p is not None]
        return all(getattr(p, "replays_prompts", False) for p in inner)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.bias = bool(spec.get("bias", False))
        self.window = int(spec.get("window", 0) or 0)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv_heads} kv heads")
        if self.head_dim % 2:
            raise ValueError(f"attention: head_dim {self.head_dim} must be even")
        pos: Optional[PartSpec] = spec.get("position")
        self.position = find_part("position", pos.kind)(pos, runtime) if pos is not None else None
        self.q_norm = self._head_norm(spec.get("q_norm"), runtime)
        self.k_norm = self._head_norm(spec.get("k_norm"), runtime)
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def _head_norm(self, ps: Optional[PartSpec], runtime):
        if ps is None:
            return None
        norm = find_part("norm", ps.kind)(ps, runtime)
        norm.prefix = self.prefix + norm.prefix           # its tensors live under this mixer's names
        return norm

    def tensors(self) -> Dict[str, TensorSpec]:
        p, H, D = self.prefix, self.hidden, self.head_dim
        t = {p + "q_proj.weight": TensorSpec((self.n_heads * D, H)),
             p + "k_proj.weight": TensorSpec((self.n_kv_heads * D, H)),
             p + "v_proj.weight": TensorSpec((self.n_kv_heads * D, H)),
             p + "o_proj.weight": TensorSpec((H, self.n_heads * D))}
        if self.bias:
            t.update({p + "q_proj.bias": TensorSpec((self.n_heads * D,), role="vector"),
                      p + "k_proj.bias": TensorSpec((self.n_kv_heads * D,), role="vector"),
                      p + "v_proj.bias": TensorSpec((self.n_kv_heads * D,), role="vector"),
                      p + "o_proj.bias": TensorSpec((H,), role="vector")})
        for norm in (self.q_norm, self.k_norm):
            if norm is not None:
                t.update(norm.tensors())
        return t

    def _pair_order(self) -> Optional[torch.Tensor]:
        """For every dimension of a head, the projected dimension that takes its place (None: as projected)."""
        layout = self.position.pair_layout() if self.position is not None else None
        if layout is None or layout[1]:
            return None
        n_pairs = layout[0]
        order = list(range(self.head_dim))
        for k in range(n_pairs):
            order[2 * k], order[2 * k + 1] = k, k + n_pairs
        return torch.tensor(order, dtype=torch.long)

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        p, D = self.prefix, self.head_dim
        order = self._pair_order()

        def heads(t: torch.Tensor, n: int) -> torch.Tensor:
            """Rows (or entries) of n heads, each head's dimensions in the cache's order."""
            if order is None:
                return t
            idx = (torch.arange(n).unsqueeze(1) * D + order.unsqueeze(0)).reshape(-1).to(t.device)
            return t.index_select(0, idx)

        w = torch.cat([heads(weights[p + "q_proj.weight"], self.n_heads),
                       heads(weights[p + "k_proj.weight"], self.n_kv_heads),
                       weights[p + "v_proj.weight"]], dim=0).contiguous()
        b = None
        if self.bias:
            b = torch.cat([heads(weights[p + "q_proj.bias"], self.n_heads),
                           heads(weights[p + "k_proj.bias"], self.n_kv_heads),
                           weights[p + "v_proj.bias"]]).contiguous()
        self.qkv = Linear(self.runtime, w, b)
        self.o = Linear(self.runtime, weights[p + "o_proj.weight"], weights.get(p + "o_proj.bias"))
        for norm in (self.q_norm, self.k_norm):
            if norm is not None:
                names = list(norm.tensors())
                norm.bind({n: heads(weights[n], 1).contiguous() if weights[n].shape == (D,) else weights[n]
                           for n in names if n in weights})

    def cache_spec(self) -> KVSpec:
        reordered = self._pair_order() is not None
        return KVSpec(self.n_kv_heads, self.head_dim, self.window,
                      f"pairs_adjacent_{self.position.pair_layout()[0]}" if reordered else "as_projected")

    def _fused_projection(self, xn, step) -> bool:
        """Whether rotation and cache write ride on the projection's epilogue: the tensor-core product takes the
        call anyway, a chunk of its epilogue lies inside one head, and nothing stands between projection and
        rotation.  Used for decode steps, where it takes one launch off every layer at the same step time; for
        prompts the epilogue's trips to the rotation table cost more than the separate kernel's pass over q and k
        (measured on the Llama-8B layer sizes: 107 us against 80 + 16 us at 2,048 tokens).
        STRATUM_FUSE_ROPE=0 turns it off, =2 turns it on for prompts too (measurements)."""
        from . import gemm_dispatch
        mode = os.environ.get("STRATUM_FUSE_ROPE", "1")
        if mode == "0" or (mode != "2" and not step.all_single):
            return False
        x = xn.x if isinstance(xn, NormedRows) else xn
        return (self.head_dim % 32 == 0 and self.q_norm is None and self.k_norm is None
                and gemm_dispatch.takes_tensor_cores(x, self.qkv.weight, extras=isinstance(xn, NormedRows)))

    def forward(self, xn, residual: torch.Tensor, step, cache: LayerCache, emit=None) -> None:
        rot = self.position.rotary() if self.position is not None else None
        if self._fused_projection(xn, step):
            extra = K.GemmExtra().qkv_rope(None if rot is None else step.rotation_table(rot), step.token_pos,
                                           step.token_seq, cache.block_table, cache.k, cache.v, self.n_heads,
                                           self.n_kv_heads, self.head_dim, PAGE_TOKENS, cache.writes)
            qkv = self.qkv(xn, mode=QKV_ROPE, extra=extra)        # only the query columns are written
        else:
            qkv = self.qkv(xn, mode=STORE)
            if self.q_norm is not None:
                self.q_norm.forward_heads(qkv, 0, self.n_heads, self.head_dim)
            if self.k_norm is not None:
                self.k_norm.forward_heads(qkv, self.n_heads * self.head_dim, self.n_kv_heads, self.head_dim)
            K.rope_store(qkv, step.token_pos, step.token_seq, cache.block_table,
                         None if rot is None else rot.inv_freq, rot is not None,       # pairs are neighbours: see bind
                         1.0 if rot is None else rot.magnitude, cache.k, cache.v,
                         self.n_heads, self.n_kv_heads, self.head_dim, PAGE_TOKENS, cache.writes)
        out = self.runtime.empty(qkv.shape[0], self.n_heads * self.head_dim)
        from . import attention_dispatch
        attention_dispatch.run(self, qkv, cache, step, out)
        self.o(out, out=residual, mode=ADD_TO_F32, emit=emit)
