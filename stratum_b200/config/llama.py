"""LlamaConfig: the Llama dense decoder's sizes and constants, read from config.json.

Field-by-field counterpart of what the reference pulls from file metadata for
its Llama handler (stratum/native/stratum_arch.h:306-349: block_count,
embedding_length, feed_forward_length, head_count, head_count_kv (default =
head_count), key_length (default = embedding/heads), rope.dimension_count
(default = head size), layer_norm_rms_epsilon (default 1e-5), rope.freq_base
(default 10000)), with the keys a Llama config.json uses.  Rope scaling types
none / linear / yarn follow stratum/native/stratum_rope.h:23-25; llama3 scaling,
attention/MLP biases and stop ids are not in the reference and follow the
published Llama configuration format.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig

_ROPE_KINDS = ("default", "none", "linear", "llama3", "yarn")
_DTYPES = ("float32", "bfloat16", "float16")


@dataclass(frozen=True)
class RopeScaling:
    """How the rotation frequencies are rescaled for long contexts."""
    kind: str = "none"                      # none | linear | llama3 | yarn
    factor: float = 1.0
    low_freq_factor: float = 1.0            # llama3
    high_freq_factor: float = 4.0           # llama3
    original_max_position: int = 0          # llama3, yarn
    beta_fast: float = 32.0                 # yarn (stratum/native/stratum_rope.h:47-48)
    beta_slow: float = 1.0                  # yarn
    attention_factor: float = -1.0          # yarn: >0 fixes the magnitude scale, <0 derives it

    @classmethod
    def from_reader(cls, r: Optional[KeyReader]) -> "RopeScaling":
        if r is None:
            return cls()
        kind = r.raw.get("rope_type", r.raw.get("type", "default"))
        if kind not in _ROPE_KINDS:
            r.problems.append(f"rope_type={kind!r} not one of {list(_ROPE_KINDS)}")
            return cls()
        if kind in ("default", "none"):
            return cls()
        factor = r.number("factor", lo=1.0)
        if kind == "linear":
            return cls(kind="linear", factor=factor or 1.0)
        if kind == "llama3":
            low = r.number("low_freq_factor", lo=0.0)
            high = r.number("high_freq_factor", lo=0.0)
            orig = r.integer("original_max_position_embeddings")
            if low is not None and high is not None:
                r.require(high > low, "high_freq_factor must exceed low_freq_factor")
            return cls(kind="llama3", factor=factor or 1.0, low_freq_factor=low or 1.0,
                       high_freq_factor=high or 4.0, original_max_position=orig or 0)
        # yarn
        orig = r.integer("original_max_position_embeddings")
        return cls(kind="yarn", factor=factor or 1.0, original_max_position=orig or 0,
                   beta_fast=r.number("beta_fast", 32.0, lo=1e-6),
                   beta_slow=r.number("beta_slow", 1.0, lo=1e-6),
                   attention_factor=r.number("attention_factor", -1.0))

    def to_dict(self) -> Optional[Dict[str, Any]]:
        if self.kind == "none":
            return None
        d: Dict[str, Any] = {"rope_type": self.kind, "factor": self.factor}
        if self.kind == "llama3":
            d.update(low_freq_factor=self.low_freq_factor, high_freq_factor=self.high_freq_factor,
                     original_max_position_embeddings=self.original_max_position)
        if self.kind == "yarn":
            d.update(original_max_position_embeddings=self.original_max_position,
                     beta_fast=self.beta_fast, beta_slow=self.beta_slow)
            if self.attention_factor > 0:
                d["attention_factor"] = self.attention_factor
        return d


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    n_layers: int
    hidden: int
    intermediate: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_dim: int = 0                        # 0 = head_dim
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    rope_interleaved: bool = False           # pairs (2k,2k+1) instead of (k,k+D/2)
    max_position: int = 4096
    tie_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"            # dtype a written folder stores its weights in

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LlamaConfig":
        r = KeyReader(raw)
        n_layers = r.integer("num_hidden_layers", hi=4096)
        hidden = r.integer("hidden_size", hi=1 << 20)
        inter = r.integer("intermediate_size", hi=1 << 24)
        n_heads = r.integer("num_attention_heads", hi=1 << 14)
        n_kv = r.integer("num_key_value_heads", default=n_heads, hi=1 << 14)
        head_dim = r.integer("head_dim", default=None, hi=1 << 14)
        vocab = r.integer("vocab_size", hi=1 << 26)
        eps = r.number("rms_norm_eps", 1e-5, lo=0.0, hi=1.0)
        theta = r.number("rope_theta", 10000.0, lo=1.0 + 1e-9)
        rope_dim = r.integer("rope_dim", default=0, lo=0, hi=1 << 14)
        sub = r.child("rope_scaling")
        scaling = RopeScaling.from_reader(sub)
        if sub is not None:
            r.adopt(sub)
        inter_leaved = r.boolean("rope_interleaved", False)
        max_pos = r.integer("max_position_embeddings", 4096, hi=1 << 24)
        tie = r.boolean("tie_word_embeddings", False)
        abias = r.boolean("attention_bias", False)
        mbias = r.boolean("mlp_bias", False)
        act = r.string("hidden_act", "silu", choices=("silu",))
        dtype = r.string("torch_dtype", "bfloat16", choices=_DTYPES)
        bos = r.raw.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int) or bos < 0):
            r.problems.append(f"'bos_token_id' must be a token id, got {bos!r}")
            bos = None
        eos = r.id_list("eos_token_id", vocab)

        if head_dim is None and hidden and n_heads:
            r.require(hidden % n_heads == 0,
                      f"hidden_size={hidden} is not a multiple of num_attention_heads={n_heads} "
                      "and no head_dim is given")
            head_dim = hidden // n_heads
        if n_heads and n_kv:
            r.require(n_heads % n_kv == 0,
                      f"num_attention_heads={n_heads} is not a multiple of num_key_value_heads={n_kv}")
        if head_dim:
            r.require(head_dim % 2 == 0, f"head_dim={head_dim} must be even")
            if rope_dim:
                r.require(rope_dim % 2 == 0 and rope_dim <= head_dim,
                          f"rope_dim={rope_dim} must be even and at most head_dim={head_dim}")
        if scaling.kind in ("llama3", "yarn"):
            r.require(scaling.original_max_position > 0,
                      "rope_scaling.original_max_position_embeddings must be positive")
        r.finish()
        return cls(n_layers=n_layers, hidden=hidden, intermediate=inter, n_heads=n_heads,
                   n_kv_heads=n_kv, head_dim=head_dim, vocab=vocab, rms_eps=eps, rope_theta=theta,
                   rope_dim=rope_dim or head_dim, rope_scaling=scaling, rope_interleaved=inter_leaved,
                   max_position=max_pos, tie_embeddings=tie, attention_bias=abias, mlp_bias=mbias,
                   hidden_act=act, bos_token_id=bos, eos_token_ids=eos, torch_dtype=dtype)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.n_layers,
            "hidden_size": self.hidden,
            "intermediate_size": self.intermediate,
            "num_attention_heads": self.n_heads,
            "num_key_value_heads": self.n_kv_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab,
            "rms_norm_eps": self.rms_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict(),
            "max_position_embeddings": self.max_position,
            "tie_word_embeddings": self.tie_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_dim and self.rope_dim != self.head_dim:
            d["rope_dim"] = self.rope_dim
        if self.rope_interleaved:
            d["rope_interleaved"] = True
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 \
                else self.eos_token_ids[0]
        return d
