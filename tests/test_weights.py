"""safetensors container, binding by name, error reports, random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from helpers import TINY_A, TINY_B, load_plain, make_model_dir
from stratum_b200.config import LlamaConfig
from stratum_b200.engine.model import expected_tensors
from stratum_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights,
                                  write_random_model, write_safetensors)


def test_container_round_trip(tmp_path):
    ts = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(4),
          "d": torch.randn(2, 2).half()}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, ts)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == sorted(ts)
    for k, v in ts.items():
        assert torch.equal(f.tensor(k), v)
    f.close()


def _raw_file(path, header: dict, data: bytes, hlen=None):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob) if hlen is None else hlen) + blob + data)


@pytest.mark.parametrize("header, data, hlen, word", [
    ({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, None, "outside the file"),
    ({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8, None, "needs 12"),
    ({"t": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, None, "unsupported dtype"),
    ({"t": {"dtype": "F32", "shape": [2]}}, b"\0" * 8, None, "lacks"),
    ({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, 10**12, "does not fit"),
    ({"t": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, b"\0" * 8, None, "malformed shape"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, None, "overlap"),
])
def test_hostile_containers_are_refused(tmp_path, header, data, hlen, word):
    p = str(tmp_path / "bad.safetensors")
    _raw_file(p, header, data, hlen)
    with pytest.raises(SafetensorsError, match=word):
        SafetensorsFile(p)


def test_duplicate_names_and_garbage(tmp_path):
    p = str(tmp_path / "dup.safetensors")
    blob = b'{"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="duplicate"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)


def test_random_folder_loads_by_name(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_B)
    d = write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype="bfloat16")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    exp = expected_tensors(cfg)
    assert "lm_head.weight" in exp and exp["lm_head.weight"].optional          # tied: may be absent
    w = load_weights(d, exp, torch.bfloat16, "cpu")
    assert "lm_head.weight" not in w
    assert w["model.embed_tokens.weight"].dtype == torch.bfloat16              # matrices stay bfloat16
    assert w["model.norm.weight"].dtype == torch.float32                       # gains are held in float32
    assert torch.all(w["model.norm.weight"] == 1.0)
    assert w["model.layers.2.mlp.down_proj.bias"].shape == (96,)
    std = w["model.layers.0.mlp.up_proj.weight"].float().std().item()
    assert 0.018 < std < 0.022
    # same seed, same values; another seed, other values; a tensor does not depend on the others
    d2 = write_random_model(str(tmp_path / "m2"), cfg, seed=1, dtype="bfloat16")
    w2 = load_weights(d2, exp, torch.bfloat16, "cpu")
    assert all(torch.equal(w[k], w2[k]) for k in w)
    cfg_a = LlamaConfig.from_dict(dict(TINY_B, num_hidden_layers=1))
    d3 = write_random_model(str(tmp_path / "m3"), cfg_a, seed=1, dtype="bfloat16")
    w3 = load_weights(d3, expected_tensors(cfg_a), torch.bfloat16, "cpu")
    assert torch.equal(w3["model.layers.0.self_attn.q_proj.weight"], w["model.layers.0.self_attn.q_proj.weight"])
    d4 = write_random_model(str(tmp_path / "m4"), cfg, seed=2, dtype="bfloat16")
    w4 = load_weights(d4, exp, torch.bfloat16, "cpu")
    assert not torch.equal(w4["model.embed_tokens.weight"], w["model.embed_tokens.weight"])


def test_float32_file_stays_float32_and_widening_is_exact(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_A)
    d = write_random_model(str(tmp_path / "m"), cfg, seed=3, dtype="float32")
    w = load_weights(d, expected_tensors(cfg), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w.values())
    db = write_random_model(str(tmp_path / "mb"), cfg, seed=3, dtype="bfloat16")
    wb = load_weights(db, expected_tensors(cfg), torch.float32, "cpu")      # bfloat16 file on the 32-bit path
    _, plain = load_plain(db)
    for k, t in wb.items():
        assert t.dtype == torch.float32
        assert np.array_equal(t.numpy().astype(np.float64), plain[k])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
        t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
        t["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    d = make_model_dir(str(tmp_path / "m"), TINY_A, seed=0, edit=edit)
    cfg = LlamaConfig.from_dict(TINY_A)
    with pytest.raises(WeightError) as e:
        load_weights(d, expected_tensors(cfg), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(err.wrong) == 2
    msg = str(err)
    assert "missing (2)" in msg and "unexpected (1)" in msg and "[64, 32]" in msg and "[64, 64]" in msg
    # an architecture may name buffers that published files carry and the model does not use: those pass,
    # everything else about the file is still reported
    from stratum_b200.config import find_architecture
    ignore = find_architecture(TINY_A).ignored_tensor_suffixes
    assert "rotary_emb.inv_freq" in ignore
    with pytest.raises(WeightError) as e:
        load_weights(d, expected_tensors(cfg), torch.float32, "cpu", ignore)
    assert e.value.unexpected == [] and len(e.value.missing) == 2 and len(e.value.wrong) == 2


def test_buffers_on_the_ignore_list_do_not_stop_a_load(tmp_path):
    def edit(t):
        for i in range(2):
            t[f"model.layers.{i}.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    d = make_model_dir(str(tmp_path / "m"), TINY_A, seed=0, edit=edit)
    from stratum_b200.engine.model import config_from_dir
    cfg, arch = config_from_dir(d)
    w = load_weights(d, expected_tensors(cfg), torch.float32, "cpu", arch.ignored_tensor_suffixes)
    assert not any(n.endswith("inv_freq") for n in w)
    with pytest.raises(WeightError, match="unexpected \\(2\\)"):
        load_weights(d, expected_tensors(cfg), torch.float32, "cpu")


def test_untied_model_needs_its_head(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, seed=0, edit=lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(d, expected_tensors(LlamaConfig.from_dict(TINY_A)), torch.float32, "cpu")


def test_missing_files(tmp_path):
    with pytest.raises(SafetensorsError, match="neither"):
        load_weights(str(tmp_path), {}, torch.float32, "cpu")
