"""The Llama dense decoder as data: LlamaConfig -> ModelSpec.

Every layer: RMSNorm -> grouped-query attention with rotary positions -> residual;
RMSNorm -> SwiGLU feed-forward -> residual; then a final RMSNorm and the output head
(stratum/native/stratum_arch_llama.inc.c:369-562, :713-723).  Tensor names are the
safetensors ones (`model.layers.N.self_attn.q_proj.weight`, ...), the naming family the
reference's archived safetensors loader binds (stratum/native/stratum_p35.c:305-317).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def describe_llama(cfg: LlamaConfig) -> ModelSpec:
    sc = cfg.rope_scaling
    scaling = None if sc.kind == "none" else {
        "kind": sc.kind, "factor": sc.factor, "low_freq_factor": sc.low_freq_factor,
        "high_freq_factor": sc.high_freq_factor, "original_max_position": sc.original_max_position,
        "beta_fast": sc.beta_fast, "beta_slow": sc.beta_slow, "attention_factor": sc.attention_factor}
    rope = PartSpec("rope", {"rope_dim": cfg.rope_dim or cfg.head_dim, "theta": cfg.rope_theta,
                             "interleaved": cfg.rope_interleaved, "scaling": scaling})
    layers = []
    for i in range(cfg.n_layers):
        layers.append(LayerSpec(
            arrangement="prenorm_residual",
            parts={
                "mixer_norm": PartSpec("rmsnorm", {"size": cfg.hidden, "eps": cfg.rms_eps,
                                                   "prefix": "input_layernorm."}),
                "mixer": PartSpec("gqa_attention", {
                    "hidden": cfg.hidden, "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads,
                    "head_dim": cfg.head_dim, "bias": cfg.attention_bias, "window": 0, "scale": None,
                    "position": rope, "q_norm": None, "k_norm": None, "prefix": "self_attn."}),
                "feed_forward_norm": PartSpec("rmsnorm", {"size": cfg.hidden, "eps": cfg.rms_eps,
                                                          "prefix": "post_attention_layernorm."}),
                "feed_forward": PartSpec("swiglu", {"hidden": cfg.hidden, "intermediate": cfg.intermediate,
                                                    "bias": cfg.mlp_bias, "prefix": "mlp."})},
            prefix=f"model.layers.{i}."))
    return ModelSpec(
        hidden=cfg.hidden, vocab=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.hidden,
                                               "prefix": "model.embed_tokens."}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.n_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden, "eps": cfg.rms_eps, "prefix": "model.norm."}),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.hidden,
                                      "tied": cfg.tie_embeddings, "prefix": "lm_head."}))


LLAMA = register_architecture(Architecture(
    names=("LlamaForCausalLM", "llama"),
    description="Llama dense decoder: GQA attention, rotary positions, SwiGLU, RMSNorm",
    config_class=LlamaConfig,
    describe_model=describe_llama,
    # the rotation frequencies some exporters store as a buffer per layer; they follow from the configuration
    ignored_tensor_suffixes=("rotary_emb.inv_freq",)), replace=True)
