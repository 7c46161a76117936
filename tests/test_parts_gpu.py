"""Each part of a layer alone, built from its PartSpec, against the plain functions."""
import math

import numpy as np
import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOLS = {"float32": 3e-5, "bfloat16": 2e-2}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def as64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rel_err(got, ref):
    return float(np.max(np.abs(got - ref)) / (np.max(np.abs(ref)) + 1e-30))


def _runtime(dtype):
    from stratum_b200.parts import Runtime
    return Runtime(DT[dtype], "cuda")


def _weights(part, rng, dtype, std=0.05):
    """Random tensors for everything the part declares, placed as the loader would place them."""
    out = {}
    for name, ts in part.tensors().items():
        a = rng.standard_normal(ts.shape) * std + (1.0 if ts.init == "ones" else 0.0)
        out[name] = dev(a, torch.float32 if ts.role == "vector" else DT[dtype])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from stratum_b200.parts import PartSpec, find_part
    rng = np.random.default_rng(0)
    part = find_part("norm", "rmsnorm")(PartSpec("rmsnorm", {"size": 200, "eps": 1e-3, "prefix": "n."}), _runtime(dtype))
    assert list(part.tensors()) == ["n.weight"]
    w = _weights(part, rng, dtype)
    part.bind(w)
    x = dev(rng.standard_normal((9, 200)) * 2)
    ref = P.rms_norm(as64(x), as64(w["n.weight"]), 1e-3)
    assert rel_err(as64(part.forward(x)), ref) < TOLS[dtype]
    rows = dev([8, 0], torch.int32)
    assert rel_err(as64(part.forward(x, rows)), ref[[8, 0]]) < TOLS[dtype]


def test_rope_tables_match_the_plain_rules():
    from stratum_b200.parts.rope import inverse_frequencies
    for rope_dim, theta, scaling, plain_scaling in [
        (64, 10000.0, None, None),
        (32, 500000.0, {"kind": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                        "original_max_position": 64},
         {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}),
        (128, 500000.0, {"kind": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position": 8192},
         {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}),
        (48, 1000.0, {"kind": "linear", "factor": 4.0}, {"rope_type": "linear", "factor": 4.0}),
    ]:
        inv, mag = inverse_frequencies(rope_dim, theta, scaling)
        ref = P.rope_inv_freq(rope_dim, theta, plain_scaling)
        assert mag == 1.0 and inv.dtype == np.float32
        assert np.max(np.abs(inv.astype(np.float64) - ref) / ref) < 3e-7
    # llama3 leaves short wavelengths alone and divides long ones by the factor
    inv, _ = inverse_frequencies(128, 500000.0, {"kind": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                 "high_freq_factor": 4.0, "original_max_position": 8192})
    base, _ = inverse_frequencies(128, 500000.0, None)
    assert inv[0] == base[0] and abs(inv[-1] * 8.0 / base[-1] - 1.0) < 1e-6
    # yarn: a magnitude factor 0.1 ln(factor) + 1 (stratum/native/stratum_rope.h:108-112), frequencies between
    # the unscaled and the interpolated ones
    inv, mag = inverse_frequencies(64, 10000.0, {"kind": "yarn", "factor": 4.0, "original_max_position": 2048})
    base, _ = inverse_frequencies(64, 10000.0, None)
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert np.all(inv <= base * (1 + 1e-6)) and np.all(inv >= base / 4.0 * (1 - 1e-6))
    assert inv[0] == base[0] and abs(inv[-1] * 4.0 / base[-1] - 1.0) < 1e-6


def _plain_swiglu(x64, w, prefix):
    return P.swiglu_mlp(x64, {k: as64(v) for k, v in w.items()}, prefix)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [3, 70])
@pytest.mark.parametrize("bias", [False, True])
def test_swiglu_part(dtype, rows, bias):
    from stratum_b200.parts import PartSpec, find_part
    rng = np.random.default_rng(rows)
    part = find_part("feed_forward", "swiglu")(
        PartSpec("swiglu", {"hidden": 96, "intermediate": 176, "bias": bias, "prefix": "mlp."}), _runtime(dtype))
    w = _weights(part, rng, dtype)
    part.bind(w)
    xn = dev(rng.standard_normal((rows, 96)), DT[dtype])
    res = dev(rng.standard_normal((rows, 96)))
    before = as64(res)
    part.forward(xn, res, None)
    ref = before + _plain_swiglu(as64(xn), w, "mlp.")
    assert rel_err(as64(res), ref) < TOLS[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from stratum_b200.parts import PartSpec, find_part
    rng = np.random.default_rng(5)
    rt = _runtime(dtype)
    emb = find_part("embedding", "token_embedding")(PartSpec("token_embedding", {"vocab": 300, "hidden": 72,
                                                                                 "prefix": "e."}), rt)
    table = dev(rng.standard_normal((300, 72)), DT[dtype])
    emb.bind({"e.weight": table})
    ids = dev([299, 0, 5, 5], torch.int32)
    assert torch.equal(emb.forward(ids), table[[299, 0, 5, 5]].float())
    xn = dev(rng.standard_normal((4, 72)), DT[dtype])
    tied = find_part("head", "linear_head")(PartSpec("linear_head", {"vocab": 300, "hidden": 72, "tied": True,
                                                                     "prefix": "h."}), rt)
    assert tied.tensors()["h.weight"].optional
    tied.bind_with_embedding({}, emb.table())                    # the file has no head: the table serves
    assert rel_err(as64(tied.forward(xn)), as64(xn) @ as64(table).T) < TOLS[dtype]
    own = dev(rng.standard_normal((300, 72)), DT[dtype])
    tied.bind_with_embedding({"h.weight": own}, emb.table())     # the file has one: it wins
    assert rel_err(as64(tied.forward(xn)), as64(xn) @ as64(own).T) < TOLS[dtype]
    untied = find_part("head", "linear_head")(PartSpec("linear_head", {"vocab": 300, "hidden": 72, "tied": False,
                                                                       "prefix": "h."}), rt)
    assert not untied.tensors()["h.weight"].optional


def _attention_setup(dtype, n_heads, n_kv, hd, hidden, window, position, bias, lens_before, n_new, rng):
    """An attention part with a cache of its own, and a step over sequences that already hold keys."""
    from stratum_b200.cache import KVSpec, SequenceCache
    from stratum_b200.engine.step import StepBatch
    from stratum_b200.parts import PartSpec, find_part
    rt = _runtime(dtype)
    part = find_part("mixer", "gqa_attention")(
        PartSpec("gqa_attention", {"hidden": hidden, "n_heads": n_heads, "n_kv_heads": n_kv, "head_dim": hd,
                                   "bias": bias, "window": window, "scale": None, "position": position,
                                   "prefix": "a."}), rt)
    assert part.cache_spec() == KVSpec(n_kv, hd, window, part.cache_spec().key_order)
    w = _weights(part, rng, dtype, std=0.15)
    part.bind(w)
    cache = SequenceCache([part.cache_spec()], 64 * 40, 8, DT[dtype], "cuda")
    slots = [cache.acquire() for _ in lens_before]
    xs = [rng.standard_normal((a + b, hidden)) for a, b in zip(lens_before, n_new)]
    xs = [as64(dev(x, DT[dtype])) for x in xs]

    def run(counts, offsets):
        """One step feeding counts[i] rows of sequence i starting at offsets[i]; returns the residual."""
        cache.reserve(slots, counts)
        T = sum(counts)
        pos, seq, rows = [], [], []
        for i, (n, o) in enumerate(zip(counts, offsets)):
            pos += list(range(o, o + n)); seq += [i] * n; rows.append(xs[i][o:o + n])
        width = max(len(r) for r in cache.page_table_rows(slots, 0))
        table = np.full((len(slots), width), -1, dtype=np.int32)
        for i, r in enumerate(cache.page_table_rows(slots, 0)):
            table[i, :len(r)] = r
        batch = StepBatch(n_tokens=T, n_seqs=len(slots), token_ids=dev([0] * T, torch.int32),
                          token_pos=dev(pos, torch.int32), token_seq=dev(seq, torch.int32),
                          want_rows=dev([], torch.int32), seq_slot=dev(slots, torch.int32),
                          seq_start=dev(np.cumsum([0] + counts), torch.int32),
                          seq_len=dev([o + n for n, o in zip(counts, offsets)], torch.int32),
                          block_tables={0: dev(table, torch.int32)}, max_new=max(counts),
                          max_len=max(o + n for n, o in zip(counts, offsets)),
                          all_single=all(n == 1 for n in counts), host={"n_new": counts, "before": offsets})
        xn = dev(np.concatenate(rows), DT[dtype])
        res = torch.zeros(T, hidden, dtype=torch.float32, device="cuda")
        part.forward(xn, res, batch, cache.layer_view(0, True, batch.block_tables))
        cache.advance(slots, counts)
        return as64(res)

    return part, w, xs, run


def _plain_attention(xs, w, n_heads, n_kv, hd, window, rope, bias):
    W = {k: as64(v) for k, v in w.items()}
    outs = []
    for x in xs:
        T = x.shape[0]
        q = P.linear(x, W["a.q_proj.weight"], W.get("a.q_proj.bias")).reshape(T, n_heads, hd)
        k = P.linear(x, W["a.k_proj.weight"], W.get("a.k_proj.bias")).reshape(T, n_kv, hd)
        v = P.linear(x, W["a.v_proj.weight"], W.get("a.v_proj.bias")).reshape(T, n_kv, hd)
        if rope is not None:
            inv = P.rope_inv_freq(rope["rope_dim"], rope["theta"])
            q = P.apply_rope(q, np.arange(T), inv, rope["interleaved"])
            k = P.apply_rope(k, np.arange(T), inv, rope["interleaved"])
        o = P.causal_gqa_attention(q, k, v, window).reshape(T, n_heads * hd)
        outs.append(P.linear(o, W["a.o_proj.weight"], W.get("a.o_proj.bias")))
    return outs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["grouped-rope", "window-norope", "mha-interleaved-bias"])
def test_attention_part_prompts_then_single_tokens(dtype, case):
    from stratum_b200.parts import PartSpec
    rng = np.random.default_rng(len(case))
    if case == "grouped-rope":
        n_heads, n_kv, hd, hidden, window, bias = 8, 2, 64, 80, 0, False
        rope = {"rope_dim": 64, "theta": 10000.0, "interleaved": False}
    elif case == "window-norope":
        n_heads, n_kv, hd, hidden, window, bias, rope = 4, 1, 32, 48, 70, False, None
    else:
        n_heads, n_kv, hd, hidden, window, bias = 3, 3, 48, 64, 0, True
        rope = {"rope_dim": 32, "theta": 1000.0, "interleaved": True}
    position = None if rope is None else PartSpec("rope", dict(rope, scaling=None))
    lens, tail = [150, 64, 9], 5
    part, w, xs, run = _attention_setup(dtype, n_heads, n_kv, hd, hidden, window, position, bias, lens, [tail] * 3, rng)
    ref = _plain_attention(xs, w, n_heads, n_kv, hd, window, rope, bias)
    got = run(lens, [0, 0, 0])                                   # the prompts in one step
    assert rel_err(got, np.concatenate([r[:n] for r, n in zip(ref, lens)])) < TOLS[dtype]
    for j in range(tail):                                        # then one token each, from the cache
        got = run([1, 1, 1], [n + j for n in lens])
        assert rel_err(got, np.stack([r[n + j] for r, n in zip(ref, lens)])) < TOLS[dtype]


def test_blocks_run_in_the_order_the_schedule_gives():
    """A schedule may name a layer twice and let a stop read another layer's cache."""
    from helpers import TINY_A, load_plain
    from stratum_b200.config import LlamaConfig, find_architecture
    from stratum_b200.engine import Engine, StepEntry, model_from_tensors
    from stratum_b200.engine.model import Model, expected_tensors
    from stratum_b200.parts import Runtime, ScheduleEntry
    from stratum_b200.weights.random_init import random_tensors
    import dataclasses
    cfg = LlamaConfig.from_dict(TINY_A)
    spec = find_architecture(TINY_A).describe_model(cfg)
    tensors = random_tensors(expected_tensors(cfg), 3, 0.05, torch.float32)
    toks = [5, 9, 200, 17, 3, 88, 1]

    def logits(schedule):
        s = dataclasses.replace(spec, schedule=tuple(schedule))
        model = Model(s, Runtime(torch.float32, "cuda"))
        from stratum_b200.weights.loader import place
        model.bind({n: place(tensors[n], ts, torch.float32, "cuda") for n, ts in model.tensors().items() if n in tensors})
        eng = Engine(model, max_tokens=256)
        slot = eng.acquire()
        whole = eng.step([StepEntry(slot, toks, list(range(len(toks))))]).cpu().numpy()
        eng.release(slot)
        slot = eng.acquire()                                     # and token by token: the cache must serve the same
        one = np.concatenate([eng.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks])
        assert np.max(np.abs(one - whole)) <= 2e-5 * np.max(np.abs(whole))
        return whole

    plain = logits([ScheduleEntry(0), ScheduleEntry(1)])
    w64 = {k: v.numpy().astype(np.float64) for k, v in tensors.items()}
    assert rel_err(plain, P.forward_logits(TINY_A, w64, toks)) < 3e-5
    twice = logits([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1)])
    shared = logits([ScheduleEntry(0), ScheduleEntry(1, cache_of=0)])
    assert rel_err(twice, plain) > 1e-3 and rel_err(shared, plain) > 1e-3
    # layer 1 reading layer 0's keys and values: restate that with the plain parts
    c = P.normalized_config(TINY_A)
    inv = P.rope_inv_freq(c["head_dim"], c["rope_theta"])
    pos = np.arange(len(toks))
    x = P.embed(w64["model.embed_tokens.weight"], toks)
    x = P.decoder_layer(x, pos, w64, 0, c, inv)
    p0, p1 = "model.layers.0.", "model.layers.1."
    x0 = P.embed(w64["model.embed_tokens.weight"], toks)
    xn0 = P.rms_norm(x0, w64[p0 + "input_layernorm.weight"], c["rms_norm_eps"])
    T, Nq, Nk, Hd = len(toks), c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    k0 = P.apply_rope(P.linear(xn0, w64[p0 + "self_attn.k_proj.weight"]).reshape(T, Nk, Hd), pos, inv, False)
    v0 = P.linear(xn0, w64[p0 + "self_attn.v_proj.weight"]).reshape(T, Nk, Hd)
    xn = P.rms_norm(x, w64[p1 + "input_layernorm.weight"], c["rms_norm_eps"])
    q1 = P.apply_rope(P.linear(xn, w64[p1 + "self_attn.q_proj.weight"]).reshape(T, Nq, Hd), pos, inv, False)
    o = P.causal_gqa_attention(q1, k0, v0).reshape(T, Nq * Hd)
    x = x + P.linear(o, w64[p1 + "self_attn.o_proj.weight"])
    x = x + P.swiglu_mlp(P.rms_norm(x, w64[p1 + "post_attention_layernorm.weight"], c["rms_norm_eps"]), w64, p1 + "mlp.")
    ref = P.linear(P.rms_norm(x, w64["model.norm.weight"], c["rms_norm_eps"]), w64["lm_head.weight"])
    assert rel_err(shared, ref) < 3e-5
