#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen2.5-0.5B-shaped model with random weights on
one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--dtype bfloat16|float32] [--impl reference]

A step is one decode step of the whole batch (default: 8 sequences that each hold a
2,048-token prompt, context 4,096). ``value`` is decoded tokens a second timed on the device
with CUDA events around K graph replays plus the greedy choice that feeds the next step;
``e2e`` is the same through ``Model.generate`` with token ids on the host going in and
coming out. Each decode step reads every weight (~1 GB) and the live cache, more than the
126 MB of L2, so no flush is needed between steps.

``--impl reference`` times ktfth/smolmoe-c99 itself: the unmodified tree under ``baseline/_ref`` is built with its
own Makefile and its command line runs a random checkpoint of the same shape (its format: Q8 weights) on the CPU,
one sequence at a time, which is all it can do.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s at batch 8 (Qwen2.5-0.5B shape, bf16, 2048-token prompts, context 4096)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def base_config():
    with open(os.path.join(ROOT, "BASELINE.json"), "r", encoding="utf-8") as f:
        text = json.load(f)["configs"][2]
    # the sizes BASELINE.json's configs[2] states in words
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu",
           "num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
           "head_dim": 64, "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0,
           "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 32768}
    for key, word in (("num_hidden_layers", "24 layers"), ("hidden_size", "hidden 896"), ("vocab_size", "vocab 151936"),
                      ("intermediate_size", "intermediate 4864")):
        assert word in text, f"BASELINE.json configs[2] no longer says {word!r}"
    return cfg


# BASELINE.json's configs[3] and configs[4], as they state them
OTHER_SHAPES = {
    "1.5b": {"num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128,
             "intermediate_size": 8960, "vocab_size": 151936, "tie_word_embeddings": True},
    "7b": {"num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
           "intermediate_size": 18944, "vocab_size": 152064, "tie_word_embeddings": False},
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            raw = json.load(f)
        out = dict(FALLBACK_PEAKS)
        out.update({k: float(v) for k, v in raw.items() if k in out and isinstance(v, (int, float))})
        return out, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: one nvidia-smi
    process that prints a line every 100 ms, started before the region and stopped after it."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.3)   # the first line is out before the timed region begins
        except OSError:
            self.proc = None

    def summary(self):
        samples = []
        if self.proc is not None:
            self.proc.terminate()   # the exact process started above
            try:
                out, _ = self.proc.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                out, _ = self.proc.communicate()
            samples = [[c.strip() for c in line.split(",")] for line in out.strip().splitlines() if line.count(",") >= 5]
        mhz = sorted(int(s[0]) for s in samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(samples[0][1]) if samples and samples[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(samples)}


def prefill_flops(cfg, T):
    D, H, A, K, HD, L, V = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                            cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"], cfg["vocab_size"])
    per_layer = (A + 2 * K) * HD * D + D * A * HD + 3 * H * D
    linear = 2.0 * T * per_layer * L
    attention = 4.0 * HD * A * L * T * (T + 1) / 2
    return linear + attention + 2.0 * V * D


def decode_tokens_per_second(engine, slots, steps, warmup):
    """K decode steps of the whole batch on the device: each step's greedy choice feeds the next."""
    import torch
    ops = engine.runtime.ops
    tokens = torch.zeros(len(slots), dtype=torch.int32, device=engine.device)
    for _ in range(warmup):
        tokens = ops.argmax(engine.step(slots, tokens))
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        tokens = ops.argmax(engine.step(slots, tokens))
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    return len(slots) * 1000.0 / ms, ms


# ---- the reference arm -------------------------------------------------------------------------------------------
REF_RECORD = "<40sIIIIQQ"   # a tensor record of the reference's container (tools/checkpoint.py:19 of the reference)


def write_reference_checkpoint(folder, cfg, prompt_len, seed=0):
    """A random checkpoint of the configuration's shape in the reference's own formats, written with numpy (its
    tools/checkpoint.py does the same row by row in pure Python, which takes hours at this size): the Q8 container
    (docs/FORMAT.md of the reference: 36-byte blocks of a float scale and 32 int8, tensors sorted by name, the tied
    head an alias of the embedding), config.ini, a tokenizer whose merges all begin with byte 0, and a prompt of
    ``prompt_len - 1`` bytes that are never 0: one token a byte after the BOS token it puts first. Weights are
    N(0, 0.02) rounded to the Q8 grid; the embedding rows of BOS and EOS are zero, so EOS never wins."""
    import struct
    import numpy as np
    d, h, v, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    heads, kv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    if cfg["head_dim"] * heads != d or d % 32 or h % 32:
        raise ValueError("the reference's Qwen2 layout needs head_dim = hidden / heads and widths that are multiples of 32")
    kd = kv * (d // heads)
    tied = bool(cfg["tie_word_embeddings"])
    specs = {"embed": (v, d, 1), "final_norm": (1, d, 0), "lm_head": (v, d, 1)}
    for layer in range(L):
        q = f"l.{layer}."
        specs.update({q + "attn_norm": (1, d, 0), q + "ffn_norm": (1, d, 0), q + "q": (d, d, 1), q + "k": (kd, d, 1),
                      q + "v": (kd, d, 1), q + "o": (d, d, 1), q + "router": (1, d, 1), q + "q_bias": (1, d, 0),
                      q + "k_bias": (1, kd, 0), q + "v_bias": (1, kd, 0), q + "e.0.gate": (h, d, 1), q + "e.0.up": (h, d, 1),
                      q + "e.0.down": (d, h, 1)})
    specs = dict(sorted(specs.items()))
    rng = np.random.default_rng(seed)
    block = np.dtype([("scale", "<f4"), ("q", "i1", (32,))])
    record = struct.Struct(REF_RECORD)
    entries, extents = [], {}
    with open(os.path.join(folder, "model.smoe"), "wb") as f:
        f.write(b"SMOEQ8\0" + (b"\2" if tied else b"\1") + struct.pack("<II", len(specs), 0))
        f.seek(16 + record.size * len(specs))
        for name, (rows, cols, q8) in specs.items():
            if tied and name == "lm_head":
                entries.append(record.pack(name.encode(), rows, cols, q8, 1, *extents["embed"]))
                continue
            offset = f.tell()
            if q8:
                for first in range(0, rows, 8192):
                    n = min(rows - first, 8192)
                    a = np.zeros((n, cols // 32), dtype=block)
                    if not name.endswith("router"):          # a dense model's router is zero (scripts/hf/qwen2.ts:170)
                        a["scale"] = 0.02 / 40.0
                        a["q"] = np.clip(np.rint(rng.standard_normal((n, cols // 32, 32), dtype=np.float32) * 40), -127, 127)
                    if name in ("embed", "lm_head") and first == 0:
                        a["q"][256:258] = 0
                    f.write(a.tobytes())
            else:
                vals = np.ones((rows, cols), "<f4") if name.endswith("norm") else (rng.standard_normal((rows, cols)) * 0.02).astype("<f4")
                f.write(vals.tobytes())
            extents[name] = (offset, f.tell() - offset)
            entries.append(record.pack(name.encode(), rows, cols, q8, 0, *extents[name]))
        f.seek(16)
        f.write(b"".join(entries))
    ini = dict(architecture="smolmoe_qwen2", dim=d, hidden_dim=h, layers=L, heads=heads, kv_heads=kv, experts=1, top_k=1,
               vocab_size=v, max_context=cfg["max_position_embeddings"], shared_experts=0, bos_id=256, eos_id=257,
               rms_eps=cfg["rms_norm_eps"], rope_theta=int(cfg["rope_theta"]))
    with open(os.path.join(folder, "config.ini"), "w") as f:
        f.write("".join(f"{k}={val}\n" for k, val in ini.items()))
    # vocab - 258 merges (src/tokenizer.c:138-178 of the reference): (0, x), then (a token made so, x), ...: none can
    # apply to a text without byte 0
    lines, firsts, nxt = [], [0], 258
    while len(lines) < v - 258:
        made = []
        for a in firsts:
            for x in range(256):
                if len(lines) == v - 258:
                    break
                lines.append(f"{a} {x}")
                made.append(nxt)
                nxt += 1
        firsts = made
    with open(os.path.join(folder, "tokenizer.bpe"), "w") as f:
        f.write("SMBPE1\n" + "\n".join(lines) + "\n")
    with open(os.path.join(folder, "prompt.bin"), "wb") as f:
        f.write(bytes(np.random.default_rng(seed + 1).integers(1, 256, size=prompt_len - 1, dtype=np.uint8).tolist()))


def reference_arm(args) -> int:
    """Builds and times the reference. Prints one JSON line; exits 0 whether or not it could be measured."""
    import shutil
    import tempfile

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if args.gpus != 1:
        return unavailable("ktfth/smolmoe-c99 is a CPU program for one sequence; there is nothing to run on several GPUs")
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref, "src", "main.c")):
        source = os.environ.get("SMOLMOE_C99_SOURCE", "/root/reference")
        if not os.path.exists(os.path.join(source, "src", "main.c")):
            return unavailable("no copy of ktfth/smolmoe-c99 under baseline/_ref and none to copy from")
        shutil.copytree(source, ref, ignore=shutil.ignore_patterns(".git"), dirs_exist_ok=True)
    if not shutil.which("make") or not (shutil.which("cc") or shutil.which("gcc")):
        return unavailable("this machine has no make or no C compiler to build ktfth/smolmoe-c99's command line with")
    raw = base_config()
    if args.shape != "0.5b":
        raw.update(OTHER_SHAPES[args.shape])
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    raw["max_position_embeddings"] = args.context
    if raw["head_dim"] * raw["num_attention_heads"] != raw["hidden_size"]:
        return unavailable("the reference's smolmoe_qwen2 layout has head_dim = hidden / heads; this shape has not")
    work = tempfile.mkdtemp(prefix="smolmoe_ref_")
    try:
        build = os.path.join(work, "build")
        binary = os.path.join(build, "smolmoe")
        made = subprocess.run(["make", "-C", ref, f"BUILD={build}", binary], capture_output=True, text=True)
        if made.returncode != 0 or not os.path.exists(binary):
            return unavailable("ktfth/smolmoe-c99's Makefile did not build its command line here: " +
                               (made.stderr.strip().splitlines() or ["no message"])[-1][:200])
        write_reference_checkpoint(work, raw, args.prompt_len)
        env = dict(os.environ, SMOLMOE_KV_CACHE="0")
        runs = []
        # its stock path: default threads (physical cores), default --batch 32, greedy; one sequence a run
        for tokens in (max(2, min(args.warmup, 4) + 1), args.steps + 1) + ((args.steps + 1,) if args.steps <= 64 else ()):
            stats_file = os.path.join(work, "stats.json")
            run = subprocess.run([binary, "--model", os.path.join(work, "model.smoe"), "--config", os.path.join(work, "config.ini"),
                                  "--tokenizer", os.path.join(work, "tokenizer.bpe"), "--prompt-file", os.path.join(work, "prompt.bin"),
                                  "--tokens", str(tokens), "--context", str(args.context), "--stats", stats_file],
                                 capture_output=True, env=env)   # (its output is the generated bytes: no text)
            if run.returncode != 0:
                return unavailable("ktfth/smolmoe-c99's command line failed on the random checkpoint: " +
                                   (run.stderr.decode("utf-8", "replace").strip().splitlines() or ["no message"])[-1][:200])
            with open(stats_file) as f:
                runs.append(json.load(f))
        timed = runs[1:]
        best = max(timed, key=lambda r: r["decode_tokens_per_second"])
        B = args.batch
    finally:
        shutil.rmtree(work, ignore_errors=True)
    value = best["decode_tokens_per_second"]
    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": B * 1000.0 / value if value else None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "q8 weights and activations, float accumulation (the reference's only format)",
        "data": "synthetic: uniform random byte tokens (seed 1), random weights N(0, 0.02) on the Q8 grid (seed 0)",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "global_batch": B, "seq_len": args.context,
                   "prompt_len": args.prompt_len, "parallelism": "none (CPU threads)", "layers": raw["num_hidden_layers"],
                   "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "backend": best["backend"],
                   "threads": best["threads"],
                   "same_config": "same layer sizes, prompt length and context; Q8 instead of bfloat16; a CPU program that holds "
                                  "one sequence: a batch of B is B runs one after another, so tokens a second do not grow with B"},
        "e2e": {"value": best["generated_tokens"] / best["decode_seconds"] if best["decode_seconds"] else None, "unit": "tok/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "its command line from prompt bytes to token ids on the host; no device is involved"},
        "gpu_launches": 0,
        "prefill": {"value": best["prefill_tokens_per_second"], "tokens": best["prompt_tokens"], "ms": best["prefill_seconds"] * 1000.0},
        "points": {"decode_b1": value},
        "impl": "reference",
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--shape", choices=sorted(OTHER_SHAPES) + ["0.5b"], default="0.5b",
                    help="layer sizes: BASELINE.json's configs[2] (default), or configs[3] / configs[4] as they state them")
    ap.add_argument("--prompt-min", type=int, default=None,
                    help="prompts of unequal lengths, uniform between this and --prompt-len (default: all of --prompt-len)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--profile-region", choices=["decode", "prefill"], default=None,
                    help="for ncu --profile-from-start off: run only this region between cudaProfilerStart/Stop "
                         "(decode: 2 eager steps of the batch; prefill: one 2,048-token prompt) and exit")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="float32: the true 32-bit path of the whole model (reported under its own metric name)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    args.warmup = max(3, args.warmup)

    import tempfile
    import torch
    from smolmoe_c99_b200 import Model
    from smolmoe_c99_b200.config import config_from_json
    from smolmoe_c99_b200.weights import write_random_model

    raw = base_config()
    if args.shape != "0.5b":
        raw.update(OTHER_SHAPES[args.shape])
    layers_full = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_json(raw)
    pk, pk_source = peaks()
    B, P, C = args.batch, args.prompt_len, args.context
    gen = torch.Generator().manual_seed(0)
    clocks = ClockSampler()

    with tempfile.TemporaryDirectory(prefix="bench_model_") as tmp:
        write_random_model(cfg, tmp, seed=0)
        biggest = B if args.no_points else max(B, 64)
        model = Model.from_folder(tmp, args.dtype, context=C, batch=biggest)
        model32 = None
        if args.dtype == "bfloat16" and not args.no_points and not args.profile_region:
            model32 = Model.from_folder(tmp, "float32", context=C, batch=B)   # the true 32-bit path, for two more points
    engine = model.engine
    V = cfg.vocab_size

    def prompts(n):
        lens = [P] * n if args.prompt_min is None else torch.randint(args.prompt_min, P + 1, (n,), generator=gen).tolist()
        return [torch.randint(0, V, (k,), generator=gen).tolist() for k in lens]

    def open_and_prefill(n):
        slots = [engine.open_sequence() for _ in range(n)]
        engine.step(slots, prompts(n))
        torch.cuda.synchronize()
        return slots

    def close(slots):
        for s in slots:
            engine.close_sequence(s)

    if args.profile_region:
        one = [torch.randint(0, V, (P,), generator=gen).tolist()]      # always of P tokens, whatever --prompt-min says of the batch
        if args.profile_region == "prefill":
            engine.use_graphs = False    # kernel by kernel: the same kernels that the captured step replays
            s = engine.open_sequence(); engine.step([s], one); engine.close_sequence(s)
            torch.cuda.synchronize()
            s = engine.open_sequence()
            torch.cuda.profiler.start(); engine.step([s], one); torch.cuda.synchronize(); torch.cuda.profiler.stop()
        else:
            slots = open_and_prefill(B)
            engine.use_graphs = False
            tok = torch.zeros(B, dtype=torch.int32, device=engine.device)
            tok = engine.runtime.ops.argmax(engine.step(slots, tok))
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            for _ in range(2):
                tok = engine.runtime.ops.argmax(engine.step(slots, tok))
            torch.cuda.synchronize(); torch.cuda.profiler.stop()
        print(json.dumps({"profiled": args.profile_region, "batch": B, "layers": raw["num_hidden_layers"]}))
        return 0

    # ---- prefill of one 2,048-token prompt ------------------------------------------------
    one = [torch.randint(0, V, (P,), generator=gen).tolist()]      # always of P tokens, whatever --prompt-min says of the batch
    # (the first GPU work of the process: a few more runs than the graph's capture needs, so that the clocks are up)
    for _ in range(8):
        s = engine.open_sequence(); engine.step([s], one); engine.close_sequence(s)
    torch.cuda.synchronize()
    reps, t_ms = 7, []
    for _ in range(reps):
        s = engine.open_sequence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); engine.step([s], one); e1.record()
        torch.cuda.synchronize()
        t_ms.append(e0.elapsed_time(e1))
        engine.close_sequence(s)
    pre_ms = sorted(t_ms)[reps // 2]
    prefill = {"value": P * 1000.0 / pre_ms, "tokens": P, "ms": pre_ms,
               "frac": prefill_flops(raw, P) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12) if args.dtype == "bfloat16" else None}
    if args.dtype == "float32":
        prefill["note"] = "CUDA-core float FMA, no tensor-core mode: no measured peak to set it against"

    # ---- launches of one decode step (counted on an eager step) ----------------------------
    slots = open_and_prefill(B)
    lib = engine.runtime.ops.lib
    engine.use_graphs = False
    tok = torch.zeros(B, dtype=torch.int32, device=engine.device)
    before = int(lib.sm_launch_count())
    tok = engine.runtime.ops.argmax(engine.step(slots, tok))
    launches_per_step = int(lib.sm_launch_count()) - before
    engine.use_graphs = True

    # ---- the headline: decode at the default batch -----------------------------------------
    clocks.start()
    value, ms = decode_tokens_per_second(engine, slots, args.steps, args.warmup)
    clock_summary = clocks.summary()
    lengths = [engine.length(s) for s in slots]
    close(slots)
    step_bytes = engine.weight_bytes() + engine.cache.bytes_per_token() * (sum(lengths) - args.steps * B // 2)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "bytes": step_bytes, "peaks": pk_source}

    # ---- end to end through the Python entry point -----------------------------------------
    host_prompts = prompts(B)
    model.generate(host_prompts, tokens=args.warmup + 1, stop_ids=(), batch=B)
    model.generate(host_prompts, tokens=args.steps + 1, stop_ids=(), batch=B)
    st = model.last_stats
    e2e = {"value": st.decode_forwards / st.decode_seconds, "unit": "tok/s",
           "h2d_bytes_per_step": 12 * B, "d2h_bytes_per_step": 4 * B,
           "note": "Model.generate: token ids on the host in and out; per step one 3x B int32 upload from pinned memory and one B int32 read"}

    points = {}
    if not args.no_points:
        for n in (1, 64):
            sl = open_and_prefill(n)
            points[f"decode_b{n}"], _ = decode_tokens_per_second(engine, sl, args.steps, args.warmup)
            close(sl)
    engine.check_status()
    l2_note = f"each step reads {engine.weight_bytes() / 1e9:.2f} GB of weights plus the cache (> 126 MB L2); no flush"
    if model32 is not None:
        # the same model in true 32-bit (float weights, cache and FMA chains): prefill of one prompt and decode at B
        del model, engine
        torch.cuda.empty_cache()
        e32 = model32.engine
        for timed in (False, True):
            s = e32.open_sequence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); e32.step([s], one); e1.record()
            torch.cuda.synchronize()
            e32.close_sequence(s)
        points["float32_prefill"] = P * 1000.0 / e0.elapsed_time(e1)
        sl = [e32.open_sequence() for _ in range(B)]
        e32.step(sl, prompts(B))
        points[f"float32_decode_b{B}"], _ = decode_tokens_per_second(e32, sl, min(args.steps, 64), 3)
        for s in sl:
            e32.close_sequence(s)
        e32.check_status()
    dtype_word = "bf16" if args.dtype == "bfloat16" else "float32"

    line = {
        "metric": METRIC if (args.shape, B, P, C, args.prompt_min, args.dtype) == ("0.5b", 8, 2048, 4096, None, "bfloat16") else
        f"decode tok/s at batch {B} (Qwen2.5-{args.shape.upper()} shape, {dtype_word}, prompts of up to {P} tokens, context {C})",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_word,
        "data": "synthetic: uniform random token ids (seed 0), random weights N(0, 0.02) (seed 0)",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "global_batch": B, "seq_len": C, "prompt_len": P,
                   "prompt_min": args.prompt_min if args.prompt_min is not None else P, "parallelism": "none (1 GPU)",
                   "layers": raw["num_hidden_layers"], "layers_of_configuration": layers_full, "hidden": raw["hidden_size"],
                   "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "tied_embeddings": bool(raw["tie_word_embeddings"]),
                   "l2": l2_note},
        "clocks": clock_summary, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step, "prefill": prefill, "roofline": roofline, "points": points,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
