#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape on one B200, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers L]
    python bench.py --impl reference        # the reference arm (see below)

Prints ONE JSON line.  `value` is decoded tokens per second at the given batch, with every
sequence's cache filled to the given context at the end of the timed steps (so the timed steps
read the longest keys of the run); a "step" is one decode step of the whole batch, timed on the
device with CUDA events over exactly K steps after W warm-up steps (given token ids; every step is launched
while the one before runs, as generation does, and its picked ids and the kernels' status word are read).  `e2e` is the same through
the Python entry point (`Stratum.generate`): host token ids in, host token ids out, every step's
inputs copied from pinned host memory and its picked ids read back.  `prefill` times one prompt
of 2,048 tokens; `roofline` relates the decode step to the bytes it must read (every weight it
uses once, and the cached keys and values of the live requests); `points` adds batch 1 and 64.
Weights (15 GB) exceed the 126 MB L2 by two orders of magnitude, so no flush is needed
between timed steps.  Peaks come from MEASURED_PEAKS.json beside this file when it exists.

Only one GPU is used; `--gpus N` with N > 1 prints a line saying so and exits with 2.
The reference (shiaho777/stratum) is C11 with NEON/Accelerate/Metal for Apple Silicon, has no
Python package metadata and no CUDA path, so it cannot be installed or run here: `--impl
reference` prints {"impl": "reference", "unavailable": ...} and exits 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_31_8B = {   # the Llama-3.1-8B shape named by the baseline's third configuration
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "intermediate_size": 14336,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False, "hidden_act": "silu",
    "torch_dtype": "bfloat16",
}
# The baseline's other two shapes, for the short --decode-only / --prefill-only lines (the JSON line of the
# contract is always the Llama-3.1-8B shape).
OTHER_SHAPES = {
    "llama2-7b": dict(LLAMA_31_8B, num_key_value_heads=32, intermediate_size=11008, vocab_size=32000,
                      rope_theta=10000.0, rope_scaling=None, max_position_embeddings=4096),
    "llama3.2-1b": dict(LLAMA_31_8B, num_hidden_layers=16, hidden_size=2048, intermediate_size=8192, head_dim=64,
                        tie_word_embeddings=True,
                        rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PREFILL_TOKENS = 2048


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "source": "measured"}
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_bytes(cfg, n_layers, batch, context):
    """Bytes one decode step has to read: each weight it uses once, and the live requests' keys and values."""
    H, F, D = cfg.hidden, cfg.intermediate, cfg.head_dim
    per_layer = (cfg.n_heads + 2 * cfg.n_kv_heads) * D * H + H * cfg.n_heads * D + 3 * H * F
    weights = 2 * (n_layers * per_layer + cfg.vocab * H)
    kv = 2 * batch * context * 2 * cfg.n_kv_heads * D * n_layers
    return weights + kv


def prefill_flops(cfg, n_layers, tokens):
    H, F, D = cfg.hidden, cfg.intermediate, cfg.head_dim
    per_layer = (cfg.n_heads + 2 * cfg.n_kv_heads) * D * H + H * cfg.n_heads * D + 3 * H * F
    linear = 2 * tokens * n_layers * per_layer + 2 * cfg.vocab * H          # the head runs on one row
    attention = n_layers * 2 * 2 * cfg.n_heads * D * (tokens * (tokens + 1) // 2)
    return linear + attention


def fill_to(llm, slots, n_tokens, vocab, rng, chunk=2048):
    """Bring every slot's cache to n_tokens with random ids, in steps of at most `chunk` tokens each."""
    from stratum_b200 import StepEntry
    done = 0
    while done < n_tokens:
        n = min(chunk, n_tokens - done)
        llm.step([StepEntry(s, rng.integers(0, vocab, size=n).tolist(), []) for s in slots])
        done += n


def time_decode(llm, batch, context, steps, warmup, vocab, rng):
    """(ms per step, launches per step) for `steps` decode steps ending at `context` tokens per sequence."""
    import torch
    from stratum_b200 import StepEntry, kernels
    warmup = warmup + SETTLE_STEPS           # (see E2E_EXTRA_WARMUP: the steps right after the prompts run slower)
    slots = [llm.acquire() for _ in range(batch)]
    try:
        fill_to(llm, slots, context - steps - warmup, vocab, rng)
        toks = rng.integers(0, vocab, size=(steps + warmup, batch)).tolist()
        for i in range(warmup):
            llm.decode_step(slots, toks[i])
        torch.cuda.synchronize()
        l0 = kernels.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        # the steps follow one another on the device as they do in generation: each is launched while the one
        # before runs, and read (picked ids, status word) while the next runs
        flying = None
        for i in range(warmup, warmup + steps):
            h = llm.launch_decode(slots, toks[i])
            if flying is not None:
                llm.collect(flying)
            flying = h
        llm.collect(flying)
        e1.record()
        torch.cuda.synchronize()
        kernels.check_status()               # a kernel that gave up a wait makes the number worthless: raise
        return e0.elapsed_time(e1) / steps, (kernels.launch_count() - l0) / steps
    finally:
        for s in slots:
            llm.release(s)


def time_prefill(llm, tokens, vocab, rng, repeats=3):
    import torch
    from stratum_b200 import StepEntry
    best = None
    for _ in range(repeats + 1):            # the first run warms up
        slot = llm.acquire()
        ids = rng.integers(0, vocab, size=tokens).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.step([StepEntry(slot, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        llm.release(slot)
        ms = e0.elapsed_time(e1)
        best = ms if best is None else min(best, ms)
    return best


# Decode steps that follow a long prompt directly run slower for a few tens of milliseconds (the step time comes
# down in stages, 6.0 -> 5.2 -> 4.4 ms at batch 8, while the GPU's power management settles after the dense
# prompt), so the end-to-end run decodes this many more untimed tokens than --warmup before its timed ones.
E2E_EXTRA_WARMUP = 24
SETTLE_STEPS = 24          # the same for the device-timed decode steps: untimed steps after the cache is filled


def time_e2e(llm, batch, context, steps, warmup, vocab, rng):
    """Decode tokens per second through Stratum.generate: host ids in, host ids out."""
    import torch
    warmup = warmup + E2E_EXTRA_WARMUP
    prompts = [rng.integers(0, vocab, size=context - steps - warmup).tolist() for _ in range(batch)]
    marks = {}

    def on_token(req, index, fed, picked, logit):
        if index == warmup and req == batch - 1:
            marks["t0"] = time.perf_counter()

    torch.cuda.synchronize()
    llm.generate(prompts, max_new_tokens=warmup + steps + 1, stop_ids=(), on_token=on_token)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    return batch * steps / (t1 - marks["t0"])


def run_workload(llm, cfg, n_layers, workload, shape, peaks, rng):
    """The baseline's other two workloads, end to end through Stratum.generate (host ids in and out): 8 prompts
    of uniform random lengths in [64, 2048] + 256 new tokens each, or 64 prompts of 512 + 512 new tokens each.
    `decode_frac`: bytes the decode steps had to read (every weight once per step, the live requests' keys and
    values) / decode time / the HBM peak."""
    import torch
    from stratum_b200 import kernels
    vocab = cfg.vocab
    if workload == "unequal8":
        lens = [int(x) for x in rng.integers(64, 2049, size=8)]
        new = 256
    else:
        lens = [512] * 64
        new = 512
    prompts = [rng.integers(0, vocab, size=n).tolist() for n in lens]
    marks = {}

    def on_token(req, index, fed, picked, logit):
        if index == 0 and req == len(lens) - 1:
            marks["first"] = time.perf_counter()

    # compile, load and warm up what this very workload uses (which kernels a step takes depends on its rows: a
    # kernel's first launch loads its code, and a shape's first decode step captures its graph)
    llm.generate(prompts, max_new_tokens=4, stop_ids=())
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = llm.generate(prompts, max_new_tokens=new, stop_ids=(), on_token=on_token)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    kernels.check_status()
    n_out = sum(len(r.tokens) for r in out)
    decode_s = t1 - marks["first"]
    # decode step k (k = 1 .. new-1) reads the weights once and, per request, the keys and values of len + k tokens
    total = sum(decode_bytes(cfg, n_layers, 0, 0) + sum(decode_bytes(cfg, n_layers, 1, n + k) -
                                                        decode_bytes(cfg, n_layers, 0, 0) for n in lens)
                for k in range(1, new))
    return {"workload": workload, "shape": shape, "prompt_tokens": sum(lens), "new_tokens": n_out,
            "prompt_s": round(marks["first"] - t0, 4),
            "prompt_tok_per_s": round(sum(lens) / (marks["first"] - t0), 1),
            "decode_s": round(decode_s, 4),
            "decode_tok_per_s": round((n_out - len(lens)) / decode_s, 1),
            "decode_frac": round(total / decode_s / 1e9 / peaks["hbm_gbs"], 4)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--decode-only", action="store_true",
                    help="time the decode steps only and print a short line (for profiler runs)")
    ap.add_argument("--workload", default=None, choices=["unequal8", "batch64"],
                    help="the baseline's other workloads through Stratum.generate: 8 unequal prompts of 64..2048 "
                         "tokens + 256 new tokens (Llama-2-7B), or 64 prompts of 512 + 512 new tokens (Llama-3.2-1B)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="prompt length of --prefill-only (the JSON line of the contract always uses 2,048)")
    ap.add_argument("--shape", default="llama3.1-8b", choices=["llama3.1-8b"] + sorted(OTHER_SHAPES),
                    help="layer sizes for the short lines of --decode-only / --prefill-only")
    ap.add_argument("--prefill-only", action="store_true",
                    help="time the 2,048-token prompt only and print a short line (for profiler runs)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "shiaho777/stratum is C11 + NEON/Accelerate/Metal for Apple Silicon with no Python "
                          "package metadata and no CUDA path: it cannot be installed or run on this machine"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    from stratum_b200 import Stratum, kernels
    from stratum_b200.config import LlamaConfig

    raw = dict(LLAMA_31_8B if args.shape == "llama3.1-8b" else OTHER_SHAPES[args.shape])
    if raw.get("rope_scaling") is None:
        raw.pop("rope_scaling", None)
    if args.shape != "llama3.1-8b" and not (args.decode_only or args.prefill_only or args.workload):
        print("bench.py: --shape other than llama3.1-8b goes with --decode-only, --prefill-only or --workload")
        return 2
    n_layers_full = raw["num_hidden_layers"]
    n_layers = args.layers or n_layers_full
    raw["num_hidden_layers"] = n_layers
    cfg = LlamaConfig.from_dict(raw)
    peaks = load_peaks()
    rng = np.random.default_rng(0)
    biggest = max(args.batch, 1 if (args.no_points or args.decode_only or args.prefill_only) else 64)
    if args.workload:
        biggest = 64 if args.workload == "batch64" else 8
        args.context = 1024 if args.workload == "batch64" else 2304
    llm = Stratum.from_random(cfg, seed=0, dtype="bfloat16",
                              max_tokens=max(biggest * (args.context + 64), args.prefill_tokens + 64),
                              max_seqs=biggest)
    vocab = cfg.vocab

    if args.workload:
        print(json.dumps(run_workload(llm, cfg, n_layers, args.workload, args.shape, peaks, rng)))
        return 0
    if args.prefill_only:
        n_tok = args.prefill_tokens
        ms = time_prefill(llm, n_tok, vocab, rng, repeats=2)
        print(json.dumps({"prefill_only": True, "tokens": n_tok, "layers": n_layers, "ms": round(ms, 3),
                          "tflops": round(prefill_flops(cfg, n_layers, n_tok) / ms / 1e9, 1)}))
        return 0
    with ClockSampler() as clocks:
        ms_step, launches = time_decode(llm, args.batch, args.context, args.steps, args.warmup, vocab, rng)
    value = args.batch * 1000.0 / ms_step
    clock_summary = clocks.summary()
    if args.decode_only:
        print(json.dumps({"decode_only": True, "batch": args.batch, "context": args.context, "layers": n_layers,
                          "ms_per_step": round(ms_step, 4), "tokens_per_s": round(value, 1),
                          "launches_per_step": launches}))
        return 0

    e2e_value = time_e2e(llm, args.batch, args.context, args.steps, args.warmup, vocab, rng)
    # bytes copied per decode step: host to device the step's description (ids, positions, page tables,
    # sampling numbers) from pinned memory, device to host the picked ids and their logits
    h2d_bytes, d2h_bytes = llm.graphs.h2d_bytes, llm.graphs.d2h_bytes
    prefill_ms = time_prefill(llm, PREFILL_TOKENS, vocab, rng)
    pf_flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            ms_b, _ = time_decode(llm, b, args.context, max(8, args.steps // 2), 3, vocab, rng)
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)

        # the baseline's fourth and fifth configurations, each on a model of its own shape, through generate
        del llm
        torch.cuda.empty_cache()
        for key, shape, workload, seqs, ctx in (("llama2_7b_unequal8", "llama2-7b", "unequal8", 8, 2304),
                                                ("llama3_2_1b_batch64", "llama3.2-1b", "batch64", 64, 1024)):
            raw_o = {k: v for k, v in OTHER_SHAPES[shape].items() if v is not None}
            if args.layers:
                raw_o["num_hidden_layers"] = min(args.layers, raw_o["num_hidden_layers"])
            cfg_o = LlamaConfig.from_dict(raw_o)
            other = Stratum.from_random(cfg_o, seed=0, dtype="bfloat16", max_tokens=seqs * (ctx + 64), max_seqs=seqs)
            w = run_workload(other, cfg_o, cfg_o.n_layers, workload, shape, peaks, rng)
            points[key + "_decode"] = w["decode_tok_per_s"]
            points[key + "_decode_frac"] = w["decode_frac"]
            points[key + "_prompt"] = w["prompt_tok_per_s"]
            del other
            torch.cuda.empty_cache()

    step_bytes = decode_bytes(cfg, n_layers, args.batch, args.context)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s @ batch 8 (Llama-3.1-8B bf16, context 4096)" if args.batch == 8 and
                  args.context == 4096 else f"decode tok/s @ batch {args.batch} (Llama-3.1-8B bf16, context {args.context})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights N(0,0.02), uniform random token ids",
        "config": {
            "model": "Llama-3.1-8B shape", "layers": n_layers, "layers_full": n_layers_full,
            "hidden": cfg.hidden, "heads": cfg.n_heads, "kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate, "vocab": cfg.vocab, "global_batch": args.batch,
            "seq_len": args.context, "rope_theta": cfg.rope_theta, "rope_scaling": "llama3 f8 lo1 hi4 orig8192",
            "rms_eps": cfg.rms_eps, "tied": cfg.tie_embeddings, "cache_dtype": "bf16",
            "parallelism": "single GPU", "l2": "weights (GBs) far exceed the 126 MB L2; no flush needed",
            "peaks": peaks["source"], "settle_steps": SETTLE_STEPS},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": d2h_bytes, "warmup": args.warmup + E2E_EXTRA_WARMUP},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(pf_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
