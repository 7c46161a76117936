#!/usr/bin/env python3
"""Pin the plain oracle (tests/plain/llama_plain.py) on the reference's own tools.

Runs, on the CPU and with no network:
  1. the reference's deterministic tiny-model generator
     (stratum/tools/make_tiny_model.py, arch llama, F16, its default 4 layers) -> a GGUF;
  2. the reference's PyTorch restatement of its Llama engine
     (stratum/tools/hidden_oracle.py) over that GGUF for a fixed prompt plus
     greedy continuation;
and writes tests/golden/tiny_llama_reference.npz holding
  - the weights under safetensors-style names (float16, as the GGUF stores them),
  - the config as JSON text (rope_interleaved=true: the GGUF "llama" layout),
  - per run: prompt, greedy ids, and the residual stream after the last layer for
    every position the oracle processed.
tests/test_plain_reference.py compares the plain oracle with these files.

Usage:  python tests/golden/make_golden.py --reference /path/to/reference/checkout
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

RUNS = [
    # (prompt ids, greedy tokens to continue with)
    (list(range(1, 9)), 4),      # the prompt the reference's CI pins (.github/workflows/ci.yml:134-141)
    ([1, 2, 3, 4], 8),           # stratum/tools/campaign_tiny_test.py:33
]

LEAF = {
    "attn_norm.weight": "input_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight",
    "attn_k.weight": "self_attn.k_proj.weight",
    "attn_v.weight": "self_attn.v_proj.weight",
    "attn_output.weight": "self_attn.o_proj.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight",
    "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
}


def load_module(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("STRATUM_REFERENCE"),
                    help="checkout of shiaho777/stratum (or set STRATUM_REFERENCE)")
    ap.add_argument("--layers", type=int, default=4)
    args = ap.parse_args()
    if not args.reference:
        ap.error("give --reference DIR (a checkout of shiaho777/stratum) or set STRATUM_REFERENCE")
    tools = os.path.join(args.reference, "stratum", "tools")
    tmp = tempfile.mkdtemp(prefix="golden_")
    gguf = os.path.join(tmp, "tiny.gguf")
    env = dict(os.environ, STRATUM_TINY_N_LAYERS=str(args.layers))
    subprocess.run([sys.executable, os.path.join(tools, "make_tiny_model.py"), "--arch", "llama",
                    "--out", gguf], check=True, env=env)
    oracle = load_module(os.path.join(tools, "hidden_oracle.py"), "ref_hidden_oracle")
    meta, T = oracle.read_gguf(gguf)
    p = "llama."
    L = meta[p + "block_count"]
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": L,
        "hidden_size": meta[p + "embedding_length"],
        "intermediate_size": meta[p + "feed_forward_length"],
        "num_attention_heads": meta[p + "attention.head_count"],
        "num_key_value_heads": meta[p + "attention.head_count_kv"],
        "head_dim": meta[p + "attention.key_length"],
        "rms_norm_eps": float(meta.get(p + "attention.layer_norm_rms_epsilon", 1e-5)),
        "rope_theta": float(meta.get(p + "rope.freq_base", 10000.0)),
        "rope_interleaved": True,
        "tie_word_embeddings": False,
        "hidden_act": "silu",
        "max_position_embeddings": 128,
    }
    weights = {
        "model.embed_tokens.weight": T("token_embd.weight"),
        "model.norm.weight": T("output_norm.weight"),
        "lm_head.weight": T("output.weight"),
    }
    for li in range(L):
        for g, h in LEAF.items():
            weights[f"model.layers.{li}.{h}"] = T(f"blk.{li}.{g}")
    cfg["vocab_size"] = int(weights["model.embed_tokens.weight"].shape[0])

    out = {"config_json": np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8)}
    for name, t in weights.items():
        a = t.numpy()
        # matrices are F16 in the GGUF; norm gains are F32
        out["w:" + name] = a.astype(np.float16) if a.ndim == 2 else a.astype(np.float32)
        assert np.array_equal(out["w:" + name].astype(np.float32), a), name

    eps = cfg["rms_norm_eps"]
    for ri, (prompt, n_gen) in enumerate(RUNS):
        step = oracle.make_forward(meta, T, L - 1)
        K = [None] * L
        V = [None] * L
        kv_len, x, hidden, ids = 0, None, [], []
        for tok in prompt:
            x, caps, kv_len, K, V, _ = step(tok, kv_len, K, V)
            hidden.extend(caps)
        for _ in range(n_gen):
            xn = oracle.rmsnorm_local(x, T("output_norm.weight"), eps)
            nxt = int(torch.argmax(xn @ T("output.weight").T))
            ids.append(nxt)
            x, caps, kv_len, K, V, _ = step(nxt, kv_len, K, V)
            hidden.extend(caps)
        out[f"run{ri}:prompt"] = np.asarray(prompt, dtype=np.int32)
        out[f"run{ri}:greedy"] = np.asarray(ids, dtype=np.int32)
        out[f"run{ri}:hidden_last"] = torch.stack(hidden).numpy().astype(np.float32)
        print(f"run {ri}: prompt {prompt} -> greedy {ids}")
    dst = os.path.join(HERE, "tiny_llama_reference.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
