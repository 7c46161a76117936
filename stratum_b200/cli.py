"""Command line in the reference's manner:

    ./stratum <model_dir> [N_GENERATE=4] [PROMPT_TOKEN_ID ... | @file]

as `./stratum <model.gguf> [N_GENERATE] [PROMPT_TOKEN_ID...]` there (stratum/native/stratum.c:50-68,
stratum/native/stratum_arch_llama.inc.c:1407-1439): N_GENERATE decode steps after the prompt (default 4),
prompt token ids as arguments or `@path` to a file of whitespace-separated ids, default prompt `1 12968`.
The token picked after the prompt is reported as "after prefill", then one line per step on stderr,
  step %2d  in=%d  stratum_argmax=%d  logit=%g
the line the reference's own scripts parse (:1620, :2053); generated ids go to stdout (the reference
prints text from the vocabulary stored in its model file; a model folder here holds no vocabulary).

Switches carry the reference's environment-variable names as well: --temp / STRATUM_TEMP,
--top-k / STRATUM_TOP_K, --top-p / STRATUM_TOP_P, --seed / STRATUM_SEED
(stratum/native/stratum_arch_qwen35.inc.c:17118-17125), --max-kv / STRATUM_MAX_KV
(stratum/native/stratum_rope.h:55-64), --multiseq / STRATUM_MULTISEQ (B copies of the prompt in
one batch, stratum/native/stratum_arch_llama.inc.c:1458-1524), --timing / STRATUM_TIMING (:2062-2070),
--logits-dump / STRATUM_LOGITS_DUMP (stratum/native/stratum_engine.h:489-525), --ppl / STRATUM_PPL
(stratum/native/stratum_arch_llama.inc.c:1535-1557), --profile / STRATUM_TYPETIME (device time per kind of
kernel, launch by launch, as the reference totals its matrix products per weight type, :2081-2091).
Without a counterpart there: --batch-file FILE, one prompt
per line, run as one batch of unequal lengths (every request's ids come out on a line of their own).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import struct
import sys
import time
from typing import List

KV_CAP_MIN, KV_CAP_MAX, KV_CAP_DEFAULT = 32, 1 << 20, 4096     # stratum/native/stratum_rope.h:27-29


def _usage_with_architectures() -> str:
    from . import architectures  # noqa: F401
    from .config.registry import registered_architectures
    lines = ["stratum - Llama-family generation on one B200", "",
             "usage: stratum <model_dir> [N_GENERATE] [PROMPT_TOKEN_ID... | @file] [options]", "",
             "Reads the folder's config.json, picks the registered handler for its architecture.", "",
             f"Registered architectures ({len(registered_architectures())}):"]
    for a in registered_architectures():
        lines.append(f"  {','.join(a.names):<28} {a.description}")
    return "\n".join(lines)


def resolve_kv_cap(context_length: int, requested: int) -> int:
    """Capacity in tokens: the request, else the model's context length, else 4096; clamped to [32, 2^20]
    (stratum/native/stratum_rope.h:55-64)."""
    mk = context_length if context_length > 0 else KV_CAP_DEFAULT
    if requested and requested > 0:
        mk = requested
    return max(KV_CAP_MIN, min(KV_CAP_MAX, mk))


def read_prompt(args_ids: List[str], capacity: int) -> List[int]:
    if not args_ids:
        return [1, 12968]
    if args_ids[0].startswith("@"):
        path = args_ids[0][1:]
        try:
            with open(path) as f:
                ids = [int(t) for t in f.read().split()]
        except OSError as e:
            raise SystemExit(f"  prompt file {path}: {e.strerror}")
        except ValueError as e:
            raise SystemExit(f"  prompt file {path}: {e}")
    else:
        try:
            ids = [int(t) for t in args_ids]
        except ValueError as e:
            raise SystemExit(f"  prompt: {e}")
    if len(ids) > capacity:
        print(f"  prompt truncated at KV capacity {capacity}", file=sys.stderr)
        ids = ids[:capacity]
    return ids


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(_usage_with_architectures(), file=sys.stderr)
        print("\noptions: --dtype bfloat16|float32  --fp32  --temp T  --top-k K  --top-p P  --seed S  --stop ID\n"
              "         --max-kv N  --multiseq B  --timing  --profile  --logits-dump PATH  --ppl  --batch-file FILE\n"
              "         --random-weights SEED --config FILE   (write <model_dir> with random weights first)",
              file=sys.stderr)
        return 1
    env = os.environ
    ap = argparse.ArgumentParser(prog="stratum", add_help=False)
    ap.add_argument("model_dir")
    ap.add_argument("rest", nargs="*")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--temp", type=float, default=float(env.get("STRATUM_TEMP", 0.0)))
    ap.add_argument("--top-k", type=int, default=int(env.get("STRATUM_TOP_K", 0)))
    ap.add_argument("--top-p", type=float, default=float(env.get("STRATUM_TOP_P", 1.0)))
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--stop", type=int, action="append", default=[])
    ap.add_argument("--max-kv", type=int, default=int(env.get("STRATUM_MAX_KV", 0) or 0))
    ap.add_argument("--multiseq", type=int, default=int(env.get("STRATUM_MULTISEQ", 0) or 0))
    ap.add_argument("--timing", action="store_true", default="STRATUM_TIMING" in env)
    ap.add_argument("--profile", action="store_true", default="STRATUM_TYPETIME" in env)
    ap.add_argument("--logits-dump", default=env.get("STRATUM_LOGITS_DUMP", ""))
    ap.add_argument("--ppl", action="store_true", default="STRATUM_PPL" in env)
    ap.add_argument("--batch-file", default=None,
                    help="one prompt per line (token ids); the prompts run as one batch of unequal lengths")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED")
    ap.add_argument("--config", default=None, help="config.json to build random weights for")
    args = ap.parse_args(argv)

    from .config.base import ConfigError, read_config_json
    from .config.registry import find_architecture
    from .sampling import DEFAULT_SEED, SamplingParams
    from .weights import SafetensorsError, WeightError

    dtype = "float32" if args.fp32 else args.dtype
    try:
        if args.random_weights is not None:
            if not args.config:
                raise SystemExit("  --random-weights needs --config FILE")
            with open(args.config) as f:
                raw = json.load(f)
            cfg = find_architecture(raw).config_class.from_dict(raw)
            from .weights import write_random_model
            write_random_model(args.model_dir, cfg, args.random_weights)
            print(f"  wrote random weights (seed {args.random_weights}) to {args.model_dir}", file=sys.stderr)
        raw = read_config_json(args.model_dir)
        arch = find_architecture(raw)
        cfg = arch.config_class.from_dict(raw)
    except (ConfigError, OSError, json.JSONDecodeError) as e:
        print(f"  {e}", file=sys.stderr)
        return 1
    print(f"  architecture: {'/'.join(arch.names)}\n{cfg.describe()}", file=sys.stderr)

    try:
        n_gen = int(args.rest[0]) if args.rest else 4
    except ValueError:
        print(f"  N_GENERATE must be an integer, got {args.rest[0]!r}", file=sys.stderr)
        return 1
    capacity = resolve_kv_cap(int(getattr(cfg, "max_position", 0) or 0), args.max_kv)
    prompt = read_prompt(args.rest[1:], capacity) if not args.batch_file else []
    vocab = cfg.vocab
    for t in prompt:
        if not (0 <= t < vocab):
            print(f"  prompt token id {t} outside the vocabulary [0, {vocab})", file=sys.stderr)
            return 1
    if len(prompt) + n_gen > capacity:
        print(f"  prompt {len(prompt)} + {n_gen} generated exceeds KV capacity {capacity}", file=sys.stderr)
        return 1

    prompts = None
    if args.batch_file:
        try:
            with open(args.batch_file) as f:
                prompts = [[int(t) for t in line.split()] for line in f if line.strip()]
        except (OSError, ValueError) as e:
            print(f"  batch file {args.batch_file}: {e}", file=sys.stderr)
            return 1
        if not prompts:
            print(f"  batch file {args.batch_file}: no prompts", file=sys.stderr)
            return 1
        for q in prompts:
            if any(not (0 <= t < vocab) for t in q):
                print(f"  batch file: a token id lies outside the vocabulary [0, {vocab})", file=sys.stderr)
                return 1
            if len(q) + n_gen > capacity:
                print(f"  batch file: prompt {len(q)} + {n_gen} generated exceeds KV capacity {capacity}", file=sys.stderr)
                return 1

    from .engine.api import Stratum
    B = len(prompts) if prompts else max(1, args.multiseq)
    try:
        llm = Stratum(args.model_dir, dtype=dtype, max_tokens=B * (((capacity + 63) // 64) * 64), max_seqs=B,
                      use_graphs=not args.profile)      # a profile brackets every launch: no replayed graphs
    except (WeightError, SafetensorsError, RuntimeError) as e:
        print(f"  {e}", file=sys.stderr)
        return 1
    print(f"  KV capacity {capacity} tokens x {B} sequence(s), cache {llm.engine.cache.storage_bytes() / 2**20:.1f} MiB,"
          f" dtype {dtype}", file=sys.stderr)

    if args.ppl:
        return _perplexity(llm, prompt)

    params = SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p,
                            seed=args.seed if args.seed is not None else int(env.get("STRATUM_SEED", DEFAULT_SEED)))
    if not params.greedy:
        print(f"  sampler: temp={params.temperature:.3f} top_p={params.top_p:.3f} top_k={params.top_k} "
              f"seed={params.seed}", file=sys.stderr)
    dump = _LogitsDump(args.logits_dump, vocab) if args.logits_dump else None
    times = {}

    def on_token(req, index, fed, picked, logit):
        if index == 0:
            times.setdefault("prefill_end", time.perf_counter())
            if req == 0:
                print(f"  after prefill, stratum_argmax = {picked}  (logit={logit:g})", file=sys.stderr)
        elif req == 0:
            print(f"  step {index - 1:2d}  in={fed}  stratum_argmax={picked}  logit={logit:g}", file=sys.stderr)
        if req == 0:
            print(picked, end=" ", flush=True)

    import torch
    from . import kernels
    if args.profile:
        kernels.profile_start()
    t0 = time.perf_counter()
    on_logits = None
    if dump is not None:
        # sequence 0 stays first among the live ones until it ends
        on_logits = lambda logits, picked: dump.record(picked[0], logits[0].cpu().numpy())   # noqa: E731
    if prompts:
        results = llm.generate(prompts, max_new_tokens=n_gen + 1, stop_ids=args.stop, sampling=params)
        torch.cuda.synchronize()
        for i, r in enumerate(results):
            print(f"  request {i}: prompt {len(prompts[i])} tok, {len(r.tokens)} generated, ended by {r.finish_reason}",
                  file=sys.stderr)
            print(" ".join(map(str, r.tokens)), flush=True)
        if args.profile:
            _print_profile(kernels.profile_report())
        return 0
    results = llm.generate([prompt] * B, max_new_tokens=n_gen + 1, stop_ids=args.stop, sampling=params,
                           on_token=on_token, want_values=True, on_logits=on_logits)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    print(flush=True)
    if B > 1 and params.greedy:
        same = all(r.tokens == results[0].tokens for r in results)
        print(f"  multiseq: {B} streams, {'all equal' if same else 'MISMATCH between streams'}", file=sys.stderr)
        if not same:
            return 1
    if dump is not None:
        dump.close()
    if args.profile:
        _print_profile(kernels.profile_report())
    if args.timing:
        pf = times.get("prefill_end", t1) - t0
        gn = t1 - times.get("prefill_end", t1)
        n_dec = max(1, len(results[0].tokens) - 1)
        print(f"\n  [timing] prefill {len(prompt)} tok: {pf:.3f}s ({1000 * pf / len(prompt):.1f} ms/tok)  |  "
              f"gen {n_dec} tok: {gn:.3f}s ({1000 * gn / n_dec:.1f} ms/tok, {B * n_dec / gn:.1f} tok/s)",
              file=sys.stderr)
    return 0


def _print_profile(rows) -> None:
    print("  [profile] device time per kernel launcher (launch by launch, CUDA events):", file=sys.stderr)
    for name, calls, secs in rows:
        print(f"    {name:<18} {secs:.4f}s over {calls} calls ({1000.0 * secs / calls:.3f} ms/call)", file=sys.stderr)


class _LogitsDump:
    """"SLOG0001" | u32 n_vocab | repeat { u32 token; f32[n_vocab] } (stratum/native/stratum_engine.h:489-525)."""

    def __init__(self, path: str, vocab: int):
        self.f = open(path, "wb")
        self.f.write(b"SLOG0001" + struct.pack("<I", vocab))

    def record(self, token: int, logits) -> None:
        self.f.write(struct.pack("<I", token))
        self.f.write(logits.astype("<f4").tobytes())

    def close(self) -> None:
        self.f.close()


def _perplexity(llm, prompt: List[int]) -> int:
    """Teacher-forced negative log-likelihood of the prompt from the engine's own logits."""
    from .engine.step import StepEntry
    slot = llm.acquire()
    logits = llm.step([StepEntry(slot, prompt, list(range(len(prompt) - 1)))]).cpu().numpy().astype("float64")
    llm.release(slot)
    nll, n = 0.0, 0
    for t in range(len(prompt) - 1):
        row = logits[t]
        mx = row.max()
        lse = mx + math.log(float((2.718281828459045 ** (row - mx)).sum()))
        nll += lse - row[prompt[t + 1]]
        n += 1
    ppl = math.exp(nll / max(n, 1))
    print(f"\n  [PPL] {n} scored tokens, mean NLL {nll / max(n, 1):.4f}, perplexity {ppl:.4f}", file=sys.stderr)
    print(f"PPL {ppl:.6f} {n}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
