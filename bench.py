#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen2.5-0.5B-shaped model with random weights on
one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A step is one decode step of the whole batch (default: 8 sequences that each hold a
2,048-token prompt, context 4,096). ``value`` is decoded tokens a second timed on the device
with CUDA events around K graph replays plus the greedy choice that feeds the next step;
``e2e`` is the same through ``Model.generate`` with token ids on the host going in and
coming out. Each decode step reads every weight (~1 GB) and the live cache, more than the
126 MB of L2, so no flush is needed between steps.
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
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "ktfth/smolmoe-c99 is a C99 CPU program with no Python package (no setup.py/pyproject.toml): pip install fails offline and online alike; it has no GPU path"}))
        return 0
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
        model = Model.from_folder(tmp, "bfloat16", context=C, batch=biggest)
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
        one = prompts(1)
        if args.profile_region == "prefill":
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
    one = prompts(1)
    for _ in range(2):
        s = engine.open_sequence(); engine.step([s], one); engine.close_sequence(s)
    torch.cuda.synchronize()
    reps, t_ms = 5, []
    for _ in range(reps):
        s = engine.open_sequence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); engine.step([s], one); e1.record()
        torch.cuda.synchronize()
        t_ms.append(e0.elapsed_time(e1))
        engine.close_sequence(s)
    pre_ms = sorted(t_ms)[reps // 2]
    prefill = {"value": P * 1000.0 / pre_ms, "tokens": P, "ms": pre_ms,
               "frac": prefill_flops(raw, P) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

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

    line = {
        "metric": METRIC if (args.shape, B, P, C, args.prompt_min) == ("0.5b", 8, 2048, 4096, None) else
        f"decode tok/s at batch {B} (Qwen2.5-{args.shape.upper()} shape, bf16, prompts of up to {P} tokens, context {C})",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids (seed 0), random weights N(0, 0.02) (seed 0)",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "global_batch": B, "seq_len": C, "prompt_len": P,
                   "prompt_min": args.prompt_min if args.prompt_min is not None else P, "parallelism": "none (1 GPU)",
                   "layers": raw["num_hidden_layers"], "layers_of_configuration": layers_full, "hidden": raw["hidden_size"],
                   "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "tied_embeddings": bool(raw["tie_word_embeddings"]),
                   "l2": f"each step reads {engine.weight_bytes() / 1e9:.2f} GB of weights plus the cache (> 126 MB L2); no flush"},
        "clocks": clock_summary, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step, "prefill": prefill, "roofline": roofline, "points": points,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
