"""The command line, in the manner of the reference's ``smolmoe <model> [--prompt ...]``
(src/main.c:72-126,128-224): the same option names and meanings where the reference has
them. This library starts at token ids, so ``--prompt`` takes ids ("5 17 3" or "5,17,3")
and ``--prompt-file`` a file with one prompt of ids per line; ``--batch`` is the number of
sequences that start together, and ``--step-tokens`` the most tokens one step brings (what
the reference calls ``--batch``: the portion of its one sequence's prompt per pass).

    python -m smolmoe_c99_b200 MODEL_DIR --prompt "1 2 3" --tokens 16
    python -m smolmoe_c99_b200 --random CONFIG.json --seed 3 --save DIR      # writes a model folder
"""
from __future__ import annotations

import argparse
import json
import math
import re
import struct
import sys
import time
from typing import List, Optional, Sequence

from .. import __version__

FNV_OFFSET, FNV_PRIME = 0xCBF29CE484222325, 0x100000001B3


def parse_ids(text: str) -> List[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"smolmoe: a prompt is a list of token ids, got {text!r}")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="smolmoe_c99_b200", description="Qwen2 generation on one NVIDIA B200 from token ids.")
    p.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    p.add_argument("--model", dest="model_opt", help="the same, as an option")
    g = p.add_argument_group("input")
    g.add_argument("--prompt", action="append", default=[], help="token ids, e.g. \"5 17 3\"; may be repeated")
    g.add_argument("--prompt-file", help="one prompt of token ids per line")
    g.add_argument("--stop-ids", default=None, help="token ids that end a sequence (default: the configuration's eos)")
    g = p.add_argument_group("generation")
    g.add_argument("--tokens", type=int, default=64, help="max new tokens (default 64)")
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (default), positive = sample")
    g.add_argument("--top-k", type=int, default=40, help="sample among the N most likely tokens (default 40, 0 = all)")
    g.add_argument("--top-p", type=float, default=0.95, help="nucleus sampling mass in (0,1] (default 0.95)")
    g.add_argument("--seed", type=int, default=1, help="nonzero sampling seed (default 1)")
    g = p.add_argument_group("resources")
    g.add_argument("--context", type=int, default=None, help="cache positions per sequence (default min(config, 2048))")
    g.add_argument("--batch", type=int, default=8, help="sequences that start together (default 8)")
    g.add_argument("--step-tokens", type=int, default=None,
                   help="most tokens one step brings; longer prompts go through in portions (default: no limit)")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16 kernels, or the whole model in true 32-bit")
    g.add_argument("--kernels", choices=["fast", "plain"], default="fast",
                   help="plain: every product and attention on the plain kernels, for comparison")
    g = p.add_argument_group("diagnostics")
    g.add_argument("--stats", help="JSON statistics (always printed to stderr)")
    g.add_argument("--trace", help="exact hexadecimal logits of every processed token of every prompt")
    g.add_argument("--hash-logits", action="store_true", help="FNV-1a64 of every raw logit, reported in the stats")
    g.add_argument("--token-ids", help="prompt and generated token ids, one per line; a blank line between requests")
    g.add_argument("--perplexity", action="store_true", help="score the prompts (teacher-forced NLL); no generation")
    g.add_argument("--profile", action="store_true", help="device time per phase of the forward pass, in the stats")
    g = p.add_argument_group("random weights")
    g.add_argument("--random", metavar="CONFIG.json", help="make random weights for this configuration instead of reading a model")
    g.add_argument("--save", metavar="DIR", help="with --random: write the model folder here and exit")
    p.add_argument("--version", action="version", version=f"smolmoe_c99_b200 {__version__}")
    return p


def fnv1a_logits(h: int, row) -> int:
    """FNV-1a64 over the raw bits of the logits, byte by byte (src/main.c:311-319)."""
    for b in row.numpy().astype("<f4").tobytes():
        h = ((h ^ b) * FNV_PRIME) & 0xFFFFFFFFFFFFFFFF
    return h


def token_nll(row, target: int) -> float:
    """-log softmax(logits)[target] in double (src/main.c:321-329)."""
    r = row.double()
    high = float(r.max())
    return high + math.log(float((r - high).exp().sum())) - float(r[target])


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    model_dir = args.model_opt or args.model
    if args.random:
        from ..config import config_from_json
        from ..weights.random_init import write_random_model
        with open(args.random, "r", encoding="utf-8") as f:
            config = config_from_json(json.load(f))
        if args.save:
            write_random_model(config, args.save, args.seed)
            print(args.save)
            return 0
    elif not model_dir:
        raise SystemExit("smolmoe: a model folder (or --random CONFIG.json) is needed")
    prompts = [parse_ids(t) for t in args.prompt]
    if args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as f:
            prompts += [parse_ids(line) for line in f if line.strip()]
    if not prompts or any(not p for p in prompts):
        raise SystemExit("smolmoe: --prompt or --prompt-file with token ids is needed")
    if not args.seed or args.batch <= 0:
        raise SystemExit("smolmoe: seed and batch must be nonzero")   # src/main.c:221
    if args.tokens < 0 or (args.step_tokens is not None and args.step_tokens <= 0):
        raise SystemExit("smolmoe: tokens must not be negative and step-tokens must be positive")
    if args.context is not None and args.context <= 0:
        raise SystemExit("smolmoe: context must be positive")
    if not (args.temperature == 0 or 1e-6 <= args.temperature <= 100) or not 0 < args.top_p <= 1 or args.top_k < 0:
        raise SystemExit("smolmoe: temperature is 0 or in [1e-6, 100], top-p in (0, 1], top-k not negative")   # src/main.c:160-170

    import torch
    from .entry import Model

    started = time.perf_counter()
    try:
        if args.random:
            model = Model.from_random(config, args.seed, args.dtype, args.context, args.batch,
                                      step_tokens=args.step_tokens, kernels=args.kernels)
        else:
            model = Model.from_folder(model_dir, args.dtype, args.context, args.batch,
                                      step_tokens=args.step_tokens, kernels=args.kernels)
    except (ValueError, RuntimeError, OSError) as e:
        raise SystemExit(f"smolmoe: {e}")
    loaded = time.perf_counter()
    engine = model.engine
    if args.profile:
        engine.start_profile()
    stats = {"version": __version__, "backend": f"cuda sm_100a {args.kernels}", "dtype": args.dtype, "batch": args.batch,
             "kv_bytes": engine.cache.bytes_per_token() * engine.cache.max_tokens,
             "weight_bytes": engine.weight_bytes(), "load_seconds": loaded - started}
    logits_hash = FNV_OFFSET
    trace = open(args.trace, "w", encoding="utf-8") if args.trace else None
    try:
        if args.perplexity or trace or args.hash_logits:
            # every prompt position through the step function: the prompts in batches of --batch sequences that
            # start together, in portions of --step-tokens (src/main.c:553-568); rows are recorded prompt by prompt
            from .generate import prompt_portions
            nll, nll_tokens = 0.0, 0
            try:
                for first in range(0, len(prompts), args.batch):
                    group = prompts[first:first + args.batch]
                    slots = [engine.open_sequence() for _ in group]
                    rows = [[] for _ in group]
                    for portion in prompt_portions([len(p) for p in group], args.step_tokens):
                        lg = engine.step([slots[i] for i, _, _ in portion], [group[i][b:e] for i, b, e in portion],
                                         [list(range(e - b)) for _, b, e in portion]).cpu()
                        at = 0
                        for i, b, e in portion:
                            rows[i].append(lg[at:at + e - b])
                            at += e - b
                    for slot in slots:
                        engine.close_sequence(slot)
                    for prompt, parts in zip(group, rows):
                        logits = torch.cat(parts, dim=0)
                        for pos in range(len(prompt)):
                            if trace:
                                trace.write(str(pos) + "".join(" " + float(v).hex() for v in logits[pos].tolist()) + "\n")
                            if args.hash_logits:
                                logits_hash = fnv1a_logits(logits_hash, logits[pos])
                            if args.perplexity and pos + 1 < len(prompt):
                                nll += token_nll(logits[pos], prompt[pos + 1])
                                nll_tokens += 1
            except ValueError as e:
                raise SystemExit(f"smolmoe: {e}")
            if args.perplexity:
                mean = nll / nll_tokens if nll_tokens else 0.0
                stats.update(perplexity_tokens=nll_tokens, nll=mean, perplexity=math.exp(mean))
        completions = []
        if not args.perplexity:
            stop_ids = parse_ids(args.stop_ids) if args.stop_ids is not None else None
            try:
                completions = model.generate(prompts, tokens=args.tokens, temperature=args.temperature, top_k=args.top_k,
                                             top_p=args.top_p, seed=args.seed, stop_ids=stop_ids, batch=args.batch,
                                             return_completions=True)
            except ValueError as e:
                raise SystemExit(f"smolmoe: {e}")
            for c in completions:
                print(" ".join(str(t) for t in c.tokens))
            stats.update(model.last_stats.as_dict())
    finally:
        if trace:
            trace.close()
    if args.token_ids:
        with open(args.token_ids, "w", encoding="utf-8") as f:
            for i, prompt in enumerate(prompts):
                ids = list(prompt) + (completions[i].tokens if completions else [])
                f.write("\n".join(str(t) for t in ids) + "\n\n")
    stats["logits_hash"] = f"{logits_hash if args.hash_logits else 0:016x}"
    if args.profile:
        stats["profile"] = {k: round(v, 6) for k, v in engine.stop_profile().items()}
    line = json.dumps(stats)
    print(line, file=sys.stderr)
    if args.stats:
        with open(args.stats, "w", encoding="utf-8") as f:
            f.write(line + "\n")
    return 0
