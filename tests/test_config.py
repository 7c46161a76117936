"""Typed configuration and the architecture registry (no GPU)."""
import copy
import json

import pytest

from helpers import TINY_A, TINY_B, TINY_C
from stratum_b200.config import (Architecture, ConfigError, LlamaConfig, find_architecture,
                                 read_config_json, register_architecture, registered_architectures)
import stratum_b200.architectures  # noqa: F401


def test_reads_every_key_and_defaults():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.n_layers, c.hidden, c.intermediate, c.n_heads, c.n_kv_heads, c.head_dim, c.vocab) == \
        (3, 96, 256, 3, 1, 32, 320)
    assert c.rms_eps == 1e-6 and c.rope_theta == 500000.0 and c.tie_embeddings and c.attention_bias and c.mlp_bias
    assert c.rope_scaling.kind == "llama3" and c.rope_scaling.factor == 8.0
    assert c.rope_scaling.original_max_position == 64 and c.rope_scaling.high_freq_factor == 4.0
    d = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32, "intermediate_size": 48,
         "num_attention_heads": 4, "vocab_size": 100}
    c = LlamaConfig.from_dict(d)
    assert c.n_kv_heads == 4 and c.head_dim == 8 and c.rope_dim == 8
    assert c.rms_eps == 1e-5 and c.rope_theta == 10000.0 and not c.tie_embeddings
    assert c.eos_token_ids == ()


def test_round_trip_through_own_keys():
    for raw in (TINY_A, TINY_B, TINY_C):
        c = LlamaConfig.from_dict(raw)
        assert LlamaConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_eos_id_or_list():
    d = dict(TINY_A, eos_token_id=7)
    assert LlamaConfig.from_dict(d).eos_token_ids == (7,)
    d = dict(TINY_A, eos_token_id=[7, 9])
    assert LlamaConfig.from_dict(d).eos_token_ids == (7, 9)
    with pytest.raises(ConfigError, match="eos_token_id"):
        LlamaConfig.from_dict(dict(TINY_A, eos_token_id=99999))


@pytest.mark.parametrize("change, word", [
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"hidden_size": 0}, "hidden_size"),
    ({"num_attention_heads": 3, "num_key_value_heads": 2}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rope_scaling": {"rope_type": "spiral"}}, "rope_type"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"intermediate_size": 2**40}, "intermediate_size"),
])
def test_bad_values_are_refused(change, word):
    d = copy.deepcopy(TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(d)


def test_all_problems_in_one_error():
    d = dict(TINY_A, hidden_size=-1, vocab_size=0)
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert "hidden_size" in str(e.value) and "vocab_size" in str(e.value)


def test_registry_by_name_and_unknown():
    assert find_architecture(TINY_A).config_class is LlamaConfig
    assert find_architecture({"model_type": "llama"}).config_class is LlamaConfig
    with pytest.raises(ConfigError, match="registered: .*LlamaForCausalLM"):
        find_architecture({"architectures": ["MambaForCausalLM"]})
    with pytest.raises(ConfigError):
        find_architecture({})
    with pytest.raises(KeyError):
        register_architecture(Architecture(("llama",), "dup", LlamaConfig, lambda c: None))
    assert any("llama" in a.names for a in registered_architectures())


def test_config_json_errors(tmp_path):
    with pytest.raises(ConfigError, match="no such file"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("[1,2]")
    with pytest.raises(ConfigError, match="JSON object"):
        read_config_json(str(tmp_path))


def test_model_description_is_data():
    """Layers are chosen by the configuration; the schedule is a list."""
    from stratum_b200.config.registry import find_architecture
    cfg = LlamaConfig.from_dict(TINY_B)
    spec = find_architecture(TINY_B).describe_model(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].parts["mixer"]
    assert m.kind == "gqa_attention" and m["n_kv_heads"] == 1 and m["head_dim"] == 32 and m["bias"] is True
    assert m["position"].kind == "rope" and m["position"]["scaling"]["kind"] == "llama3"
    ff = spec.layers[0].parts["feed_forward"]
    assert ff.kind == "swiglu" and ff["intermediate"] == 256
    assert sorted(spec.layers[0].parts) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm"]
    assert spec.head["tied"] is True
