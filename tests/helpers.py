"""Tiny configurations, model folders and comparisons shared by the tests."""
import json
import os

import numpy as np
import torch

from plain import llama_plain as P

# Tiny Llama configurations that differ in every size and option.
TINY_A = {   # grouped heads, untied, no bias, plain rope
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "intermediate_size": 176,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 128,
    "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False, "hidden_act": "silu",
}
TINY_B = {   # one kv head, tied head, biases, llama3 rope scaling
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "intermediate_size": 256,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 320,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0, "max_position_embeddings": 256,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "tie_word_embeddings": True, "attention_bias": True, "mlp_bias": True, "hidden_act": "silu",
}
TINY_C = {   # heads*head_dim != hidden, as many kv heads as heads, interleaved pairs, partial rotation
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 1, "hidden_size": 80, "intermediate_size": 112,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "vocab_size": 200,
    "rms_norm_eps": 1e-4, "rope_theta": 1000.0, "rope_dim": 32, "rope_interleaved": True,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0}, "max_position_embeddings": 512,
    "tie_word_embeddings": False, "attention_bias": True, "mlp_bias": False, "hidden_act": "silu",
}
TINY_D = {   # head size 64 in groups of two: the TMA / tcgen05 attention and matrix kernels at model level
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 136, "intermediate_size": 200,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 331,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False, "hidden_act": "silu",
}
TINY_E = {   # head size 128, eight heads on one kv head, llama3 scaling
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 1, "hidden_size": 192, "intermediate_size": 328,
    "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 128, "vocab_size": 517,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0, "max_position_embeddings": 1024,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 256},
    "tie_word_embeddings": True, "attention_bias": False, "mlp_bias": True, "hidden_act": "silu",
}
TINY_F = {   # a width, an inner size and a vocabulary that no vector load divides: the fallback kernels
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 102, "intermediate_size": 150,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "vocab_size": 203,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "attention_bias": False, "mlp_bias": False, "hidden_act": "silu",
}
TINY_G = {   # heads of 80 in groups of three, yarn scaling whose ramp covers pairs 0 to 9 of 40
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 144, "intermediate_size": 232,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 80, "vocab_size": 411,
    "rms_norm_eps": 3e-6, "rope_theta": 50000.0, "max_position_embeddings": 1024,
    "rope_scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32,
                     "beta_fast": 4.0, "beta_slow": 0.5},
    "tie_word_embeddings": False, "attention_bias": True, "mlp_bias": False, "hidden_act": "silu",
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F, "G": TINY_G}


def make_model_dir(path, cfg_dict, seed, dtype="float32", std=0.02, edit=None):
    """Write a random model folder; `edit(tensors)` may change tensors before they are stored."""
    from stratum_b200.config import find_architecture
    from stratum_b200.engine.model import expected_tensors
    from stratum_b200.weights.random_init import random_tensors, _TORCH_DTYPES
    from stratum_b200.weights.safetensors_io import write_safetensors
    arch = find_architecture(cfg_dict)
    cfg = arch.config_class.from_dict(cfg_dict)
    tensors = random_tensors(expected_tensors(cfg), seed, std, _TORCH_DTYPES[dtype])
    if edit is not None:
        edit(tensors)
    os.makedirs(path, exist_ok=True)
    raw = cfg.to_dict()
    raw["torch_dtype"] = dtype
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def load_plain(path):
    """config dict and float64-ready numpy weights of a model folder, read independently of the loader."""
    import struct
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[8 + hlen + b: 8 + hlen + e]
        if info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif info["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(info["dtype"])
        w[name] = a.reshape(info["shape"])
    if cfg.get("rope_scaling") is None:
        cfg.pop("rope_scaling", None)
    return cfg, w


def plain_logits(cfg, w, tokens):
    return P.forward_logits(cfg, w, tokens)


def rand_tokens(rng, n, vocab):
    return rng.integers(0, vocab, size=n).tolist()


# Tolerances, as a fraction of the largest reference logit of the comparison.  float32: rounding of
# float32 sums and of float32 rotation angles against the float64 oracle.  bfloat16: activations are
# rounded to 8 bits of mantissa (2^-9 relative) a handful of times per layer.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def assert_close(got, ref, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    scale = np.max(np.abs(ref))
    err = np.max(np.abs(got - ref))
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    assert err <= TOL[dtype] * scale, f"{what}: max error {err:.3e} > {TOL[dtype]:.0e} x {scale:.3e}"
